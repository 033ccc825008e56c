/*
 * drone_b200.h — C ABI of the B200-native sparse-aggregation path.
 *
 * One shared library (libdrone_b200.so) exports everything below.  All entry
 * points are plain C: pointers, sizes and opaque handles only.  Pointers whose
 * name starts with d_ are device pointers on the plan's device, h_ are host
 * pointers.  `stream` is a cudaStream_t passed as void* (NULL = legacy default
 * stream).  Every function returns 0 on success and a negative DRONE_E_* code
 * on failure; drone_last_error() then holds a human-readable message for the
 * calling thread.  Nothing in the library calls exit(), traps, or falls back
 * to a CPU path.
 *
 * Each declaration names the reference interface it stands in for, as
 * <path inside the reference project>:<line>.
 */
#ifndef DRONE_B200_H
#define DRONE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DRONE_OK            0
#define DRONE_E_INVALID    -1   /* bad argument (NULL, negative size, misaligned, unsupported F) */
#define DRONE_E_CUDA       -2   /* a CUDA runtime call failed; message holds cudaGetErrorString */
#define DRONE_E_NCCL       -3   /* an NCCL call failed */
#define DRONE_E_STATE      -4   /* call order violated (e.g. PR_IncEVal before PR_PEVal) */
#define DRONE_E_TOO_LARGE  -5   /* size exceeds a stated static limit */

/* orientation of the aggregation */
#define DRONE_OP_A   0   /* Y = A  · X : rows are edge sources      (GraphSum backward) */
#define DRONE_OP_AT  1   /* Y = Aᵀ · X : rows are edge destinations (GraphSum forward)  */

/* bit flags for drone_plan_create: which orientations to prepare */
#define DRONE_PLAN_A    1
#define DRONE_PLAN_AT   2
#define DRONE_PLAN_BOTH 3

typedef struct drone_plan drone_plan;

/* Library/ABI version (major*1000 + minor). */
int drone_version(void);

/* Message of the last failure on the calling thread ("" if none). */
const char *drone_last_error(void);

/*
 * Edge coefficients of the normalised adjacency:
 *   values[i] = 1 / sqrtf(1.0 * outDegree[u] * inDegree[v])   for edge i = u -> v,
 * evaluated with the same float/double promotions as the reference kernel so
 * the result is bit-identical.  Degrees are GLOBAL degrees indexed by local id.
 * Replaces cuda_compute_csr_values, cuda_gcn/src/cuda/cuda_kernel.cu:144-155
 * (launched at cuda_gcn/src/cuda/cuda_module.cu:162-164).
 */
int drone_compute_csr_values(const int *d_index, const int *d_dst,
                             const int *d_in_degree, const int *d_out_degree,
                             int n_rows, float *d_values, void *stream);

/*
 * Aggregation plan for one local subgraph.
 *
 * Input is the reference's device graph: CSR by SOURCE vertex
 * (d_index[n_rows+1], d_dst[nnz]; struct Graph, cuda_gcn/src/cuda/graph.h:17-41,
 * built at cuda_gcn/src/cuda/graph.cu:94-103).  Coefficients come either from
 * d_values (nnz floats, copied) or, when d_values is NULL, from the global
 * degrees exactly as drone_compute_csr_values does.  The plan builds, once:
 * the transposed CSR (rows = destinations, sources ascending inside a row),
 * and for each prepared orientation the split of rows into short rows and
 * fixed-size nonzero chunks of long rows.
 * Replaces the cuSPARSE set-up in CUDAGraphSum::CUDAGraphSum,
 * cuda_gcn/src/cuda/cuda_module.cu:149-202 (cusparseCreateCsr,
 * cusparseCsr2cscEx2, cusparseCreateDnMat).
 *
 * d_index and d_dst are copied; the caller may free them after the call.
 */
int drone_plan_create(drone_plan **out, int n_rows, int nnz,
                      const int *d_index, const int *d_dst,
                      const float *d_values,
                      const int *d_in_degree, const int *d_out_degree,
                      int orientations, void *stream);

int drone_plan_destroy(drone_plan *plan);

typedef struct drone_plan_stats {
    int       n_rows;
    int       nnz;
    int       short_row_limit;   /* rows with at most this many nonzeros are summed by one lane group */
    int       chunk_nnz;         /* nonzeros per chunk of a long row */
    int       n_long_rows[2];    /* [DRONE_OP_A], [DRONE_OP_AT]: rows above short_row_limit */
    int       n_chunks[2];       /* chunks over all long rows */
    int       n_split_rows[2];   /* rows made of more than one chunk (need partial sums) */
    int       n_partials[2];     /* partial-sum slots = chunks of split rows */
    long long scratch_bytes;     /* bytes of partial-sum scratch currently held */
    int       last_slice_width;  /* columns per slice of the most recent aggregation call (0: it ran in one piece) */
    int       hot_rows_tagged;   /* columns tagged for the table of hot rows (0: the plan has no such table) */
} drone_plan_stats;

int drone_plan_get_stats(const drone_plan *plan, drone_plan_stats *out);

/*
 * Device pointers to the CSR arrays of one orientation (owned by the plan;
 * for tests and for callers that want the transposed graph).
 * Stands in for cscColPtr/cscRowInd/cscValues, cuda_gcn/src/cuda/cuda_module.cu:171-185.
 */
int drone_plan_get_csr(const drone_plan *plan, int orientation,
                       const int **d_rowptr, const int **d_col, const float **d_val);

/*
 * Y[r, 0:F] = sum over nonzeros k of row r:  val[k] * X[col[k], 0:F]
 * with row-major dense operands (leading dimensions ldx, ldy >= F, in floats).
 * Y is overwritten (beta = 0); X and Y must not overlap.
 * orientation DRONE_OP_AT replaces the forward cusparseSpMM call,
 * cuda_gcn/src/cuda/cuda_module.cu:233-246 (together with out->zero(), :214);
 * orientation DRONE_OP_A replaces the backward call, :323-336.
 * 1 <= F <= 1024.  fp32 data, fp32 accumulation, fixed summation order:
 * two calls on the same inputs give bit-identical results.
 * Asynchronous on `stream`.
 */
int drone_spmm(drone_plan *plan, int orientation, int F,
               const float *d_X, int ldx, float *d_Y, int ldy, void *stream);

/*
 * drone_spmm with options, for the element-wise step the reference runs as a pass of its own right after the
 * aggregation and for the coefficient stream:
 *   epilogue = DRONE_EPILOGUE_RELU   Y is stored as max(Y, 0): CUDAReLU::forward in place on the layer's output
 *                                    (cuda_gcn/src/cuda/cuda_module.cu:498-511, kernel cuda_kernel.cu:384-391) done in
 *                                    the store of the aggregation.  The mask the reference keeps for the backward
 *                                    pass is (Y > 0) of the stored result.
 *   d_row_scale                      Y[r,:] is multiplied by d_row_scale[r] before the epilogue (NULL: not scaled).
 *   unit_values = 1                  every stored coefficient counts as 1 and the coefficient stream is not read
 *                                    (4 bytes per nonzero instead of 8).  With the reference's coefficients
 *                                    1/sqrt(outDegree[u]*inDegree[v]) (cuda_kernel.cu:144-155), which are a product
 *                                    of a per-row and a per-column factor, the layer becomes
 *                                      Y = diag(row factor) · pattern · (diag(column factor) · X):
 *                                    the caller scales X's rows (or folds the factor into what produces X) and passes
 *                                    the row factor as d_row_scale; drone_degree_scales computes both factors.
 *                                    Results differ from the stored-coefficient path by rounding only.
 *   row_class                        -1: all rows; >= 0: as drone_spmm_rows.
 *   push_up_to                       an exchange plan with the peer-memory transport enabled (drone_xplan_enable_p2p),
 *                                    made for this plan's local rows: the call also performs the upward half of the
 *                                    mirror/master exchange of Y.  The kernels store every finished mirror row
 *                                    straight into its owner's memory over NVLink instead of into Y (pack kernel,
 *                                    send and receive of GraphSum_sync_value_nccl, cuda_communicate.cu:374-409, fused
 *                                    into the aggregation), so the transfer runs while the aggregation computes and
 *                                    the rows are neither written locally nor read again.  drone_exchange_finish on
 *                                    the same Y must follow on every rank; until then the mirror rows of Y are
 *                                    unspecified.  After both calls Y holds bit for bit what drone_spmm followed by
 *                                    drone_exchange_sum gives.  Not with DRONE_EPILOGUE_RELU (the sum over the
 *                                    replicas comes first).  Widths that are not a multiple of 4 are aggregated
 *                                    as usual and sent with the exchange's own copy kernel; the call sequence is
 *                                    the same.
 * opts == NULL is drone_spmm.  Zero-initialise the struct, set row_class = -1, then set what is needed.
 */
#define DRONE_EPILOGUE_NONE 0
#define DRONE_EPILOGUE_RELU 1
struct drone_xplan;
typedef struct drone_spmm_opts {
    int          epilogue;
    int          row_class;
    int          unit_values;
    int          reserved_;
    const float *d_row_scale;
    struct drone_xplan *push_up_to;
} drone_spmm_opts;
int drone_spmm_ex(drone_plan *plan, int orientation, int F,
                  const float *d_X, int ldx, float *d_Y, int ldy,
                  const drone_spmm_opts *opts, void *stream);

/* in_scale[i] = inDegree[i]^-1/2, out_scale[i] = outDegree[i]^-1/2 (0 where the degree is 0): the per-row and
 * per-column factors of cuda_compute_csr_values, cuda_gcn/src/cuda/cuda_kernel.cu:144-155. */
int drone_degree_scales(const int *d_in_degree, const int *d_out_degree, int n_rows,
                        float *d_in_scale, float *d_out_scale, void *stream);

/*
 * Row classes: a way to compute the aggregation a group of output rows at a time, so that what follows the
 * aggregation for a group (the mirror/master exchange of those rows, cuda_gcn/src/cuda/cuda_module.cu:267-272)
 * can run on another stream while the next group is still being aggregated.
 *
 * drone_plan_set_row_classes gives every row a class in 0..n_classes-1 (d_row_class[n_rows], device memory; at most
 * 16 classes; n_classes = 1 removes the classes) and rebuilds the plan's work lists class by class; it synchronises
 * the device.  drone_spmm is unaffected (all rows, same bits as before).  drone_spmm_rows computes only the rows of
 * one class and leaves every other row of Y as it is; calling it for every class gives bit for bit what drone_spmm
 * gives.  Calls of one plan must still be ordered among themselves (they share the partial-sum scratch).
 * The reference has no counterpart: it runs cusparseSpMM over all rows and only then starts the exchange.
 */
int drone_plan_set_row_classes(drone_plan *plan, const int *d_row_class, int n_classes, void *stream);
int drone_spmm_rows(drone_plan *plan, int orientation, int row_class, int F,
                    const float *d_X, int ldx, float *d_Y, int ldy, void *stream);

/*
 * Allocates, ahead of time, everything later calls of this plan would otherwise allocate on first use: the
 * partial-sum buffer of split rows for feature widths up to max_features and, as `what` asks,
 *   DRONE_RESERVE_HOST_OPERANDS  the device staging of drone_spmm_host for [n_rows, max_features] operands;
 *   DRONE_RESERVE_PADDED_ROWS    two [n_rows, max_features rounded up to 4] buffers for operands whose rows cannot
 *                                be read 16 bytes at a time where they lie (a width that is not a multiple of 4 such
 *                                as the class widths 41 and 47, odd leading dimensions, unaligned addresses).  With
 *                                them, such calls copy X into rows padded to a multiple of 4 floats, run the float4
 *                                kernels and copy the result out (two extra passes over [n_rows, F], small beside the
 *                                gathers); without them the scalar kernels run.  The two routes add in different
 *                                (each fixed) orders, so they agree to rounding, not bit for bit.
 * After it, drone_spmm / drone_spmm_rows / drone_spmm_host with F <= max_features reach neither cudaMalloc nor a
 * device-wide synchronisation.
 * Stands where the reference sizes its cuSPARSE workspace on the first training step,
 * cuda_gcn/src/cuda/cuda_module.cu:234-244 (cusparseSpMM_bufferSize, cudaFree + cudaMalloc of sparseBuffer).
 */
#define DRONE_RESERVE_HOST_OPERANDS 1
#define DRONE_RESERVE_PADDED_ROWS   2
int drone_plan_reserve(drone_plan *plan, int max_features, int what);

/*
 * Same operation with HOST operands: copies X to the device, aggregates, and
 * copies Y back, synchronising before it returns.  Device staging buffers are
 * owned by the plan and reused across calls.  h_X and h_Y are dense
 * [n_rows, F] row-major; pinned memory makes the copies asynchronous DMA.
 * This is the call a host-side (cgo / CPU) user of the path makes.
 */
int drone_spmm_host(drone_plan *plan, int orientation, int F,
                    const float *h_X, float *h_Y);

/*
 * The same with a queue, for a caller that has a series of host-operand calls to make (a batch of feature blocks,
 * one call per layer and direction over several inputs).  drone_spmm_host_submit queues Y = op(A) X and returns a
 * ticket without waiting; drone_spmm_host_wait returns when h_Y of that ticket is complete.  At most two calls of a
 * plan are in flight: a third submit first waits for the call two tickets earlier.  Inside the library a call is
 * three stages on three streams (copy in, aggregation, copy out) over two sets of staging buffers, so the operands of
 * call k cross PCIe while call k-1 is aggregated and the result of call k-2 crosses it in the other direction.  One
 * call alone takes as long as drone_spmm_host; a series approaches the time of the copies in one direction.
 * h_X must not change and h_Y must not be read until the wait returns; pinned memory on both, or the copies are not
 * asynchronous.  Calls of one plan are queued in order; results are bit-identical to drone_spmm.  Not to be mixed
 * with other calls on the same plan while tickets are outstanding.  No counterpart in the reference, whose operands
 * never leave the device.
 */
int drone_spmm_host_submit(drone_plan *plan, int orientation, int F,
                           const float *h_X, float *h_Y, long long *ticket);
int drone_spmm_host_wait(drone_plan *plan, long long ticket);

/*
 * drone_spmm for callers that cannot allocate device memory: programs that give
 * all of it to their own pool at start-up, so that an allocation made behind
 * their back fails or fragments the pool, and threads that must never block on
 * the driver's allocator.  drone_spmm grows a per-plan buffer for the partial
 * sums of split rows with cudaMalloc when it needs to; this entry point keeps
 * those partial sums in an array built into the library instead
 * (DRONE_STATIC_SCRATCH_BYTES, resident on every GPU that loads the library
 * until the process exits) and calls no cudaMalloc, cudaFree or any other
 * allocating routine.  Inputs, outputs, arguments and results are those of
 * drone_spmm: the same kernels run in the same order, so the output is
 * bit-identical.
 * Limits and rules:
 *  - a call whose plan needs more than DRONE_STATIC_SCRATCH_BYTES of partial
 *    sums (n_partials[orientation] * F * 4 bytes, see drone_plan_get_stats)
 *    fails with DRONE_E_TOO_LARGE and launches nothing;
 *  - the first call on a device looks up the array's device address; make that
 *    first call before any stream capture;
 *  - all calls on a device share the one array: two calls whose kernels may
 *    overlap on the GPU (different streams, or different plans on different
 *    streams) race on it; order them on one stream or with events.  Nothing
 *    in the array has to be zero beforehand: every slot a call reads was
 *    written earlier in the same call.
 * It has no counterpart in the reference.
 */
#define DRONE_STATIC_SCRATCH_BYTES (16u << 20)
int drone_spmm_static_scratch(drone_plan *plan, int orientation, int F,
                              const float *d_X, int ldx, float *d_Y, int ldy, void *stream);

/* Pinned host memory for drone_spmm_host operands. */
int drone_host_alloc(void **out, size_t bytes);
int drone_host_free(void *ptr);

/* ------------------------------------------------------------------------- */
/* EBV vertex-cut exchange                                                     */
/* ------------------------------------------------------------------------- */

typedef struct drone_comm drone_comm;     /* one NCCL communicator + this process's rank */
typedef struct drone_xplan drone_xplan;   /* static routing plan of one rank */

#define DRONE_UNIQUE_ID_BYTES 128

/*
 * Communicator bootstrap without MPI: rank 0 calls drone_comm_unique_id and
 * hands the 128 bytes to the other ranks by any means (file, socket,
 * torch.distributed); every rank then calls drone_comm_create with its device
 * current.  Replaces ncclGetUniqueId + MPI_Bcast + ncclCommInitRank in
 * build_graph, cuda_gcn/src/cuda/graph.cu:39-52 (DRONE/src/cuda/graph.cu:31-37,
 * 122-128 passes the id through the file ./nccl.id).
 * drone_comm_adopt wraps a communicator the caller already owns (the
 * reference's Comm.comm, cuda_gcn/src/cuda/graph.h:43-46); it is not destroyed
 * with the handle.
 */
int drone_comm_unique_id(void *id_out, size_t id_bytes);
int drone_comm_create(drone_comm **out, int rank, int nranks, const void *id, size_t id_bytes);
int drone_comm_adopt(drone_comm **out, void *nccl_comm, int rank, int nranks);
int drone_comm_destroy(drone_comm *comm);

/* In-place sum over ranks of `count` floats (is_double = 0) or doubles (1).
 * Replaces ncclAllReduce(globalDiff), DRONE/src/cuda/algorithm/pr.cu:365. */
int drone_comm_allreduce_sum(drone_comm *comm, void *d_buf, size_t count, int is_double, void *stream);

/*
 * The data-parallel treatment of the dense layers' weights around the aggregation, in place on `count` floats:
 * drone_comm_bcast copies rank `root`'s buffer to every rank (weight_broadcast_value_nccl,
 * cuda_gcn/src/cuda/cuda_communicate.cu:99-105, called with root 0 at the start of every forward pass);
 * drone_comm_reduce_sum leaves the sum over ranks on `root` (weight_reduce_grad_nccl, :107-115; the other ranks'
 * buffers are unspecified afterwards, as with ncclReduce).  Asynchronous on `stream`.
 */
int drone_comm_bcast(drone_comm *comm, float *d_buf, size_t count, int root, void *stream);
int drone_comm_reduce_sum(drone_comm *comm, float *d_buf, size_t count, int root, void *stream);

/*
 * Zeroes the rows of a [n_rows, F] row-major matrix (leading dimension ld) that belong to mirror vertices
 * (d_mirror2worker[row] != -1), so that the weight gradient dW = X^T · dY that follows counts every replicated
 * vertex once.  Replaces clear_mirror_grad, cuda_gcn/src/cuda/cuda_module.cu:50-61 (launched at :88-91 between
 * the two cublasSgemm calls of CUDAMatmul::backward).
 */
int drone_clear_mirror_rows(float *d_rows, int n_rows, int F, int ld, const int *d_mirror2worker, void *stream);

/*
 * Routing plan of one rank, from the reference's routing tables (host arrays,
 * indexed by local vertex id):
 *   h_local2global[n_local]          Graph.Local2Global
 *   h_mirror2worker[n_local]         Graph.Mirror2Worker: -1, or the rank owning the master copy
 *   h_master_worker_index[n_local+1] Graph.MasterWorkerIndex  } CSR: ranks that hold a mirror
 *   h_master2workers[...]            Graph.Master2Workers     } of each local master
 * (cuda_gcn/src/cuda/graph.h:21-26, filled by addMasterRoute / addMirrorRoute,
 * cuda_gcn/src/cuda/graph.cu:281-367).  Needs no GPU; device copies are made on
 * first use.  max_features bounds F of later exchanges (it sizes the buffers).
 * Replaces buffer_init / generateLen / calSendRecvLen / buffer_initIdx,
 * cuda_gcn/src/cuda/cuda_communicate.cu:7-74,117-124.
 */
int drone_xplan_create(drone_xplan **out, int rank, int nranks, int n_local,
                       const int *h_local2global, const int *h_mirror2worker,
                       const int *h_master_worker_index, const int *h_master2workers,
                       int max_features);
int drone_xplan_destroy(drone_xplan *plan);

/* Rows sent up (mirror -> master) and down (master -> mirror) per peer rank
 * (arrays of nranks ints, either may be NULL), and the number of local master
 * rows that receive contributions. */
int drone_xplan_counts(const drone_xplan *plan, int *up_rows_per_peer, int *down_rows_per_peer,
                       int *n_master_rows);
/* The row lists themselves (local row ids, grouped by peer in rank order, ascending
 * global id inside a group); sizes are the sums of drone_xplan_counts. */
int drone_xplan_lists(const drone_xplan *plan, int *up_rows, int *down_rows);

/*
 * d_rows is [n_local, F] row-major with leading dimension ld.  On return every
 * replica row of a vertex holds the sum of that vertex's rows over all ranks;
 * rows of unreplicated vertices are untouched.  The master adds its mirrors'
 * rows to its own in ascending rank order, so results are bit-reproducible.
 * Collective over the communicator; asynchronous on `stream`.
 * Replaces GraphSum_sync_value_nccl and GraphSum_sync_grad_nccl,
 * cuda_gcn/src/cuda/cuda_communicate.cu:374-448 and :502-556 (pack kernels
 * :126-207, sendID_Value :296-372, apply_sum :239-249, apply_assign :264-274).
 */
int drone_exchange_sum(drone_xplan *plan, drone_comm *comm, float *d_rows, int F, int ld, void *stream);

/*
 * The rest of an exchange whose upward half an aggregation call performed (drone_spmm_ex with push_up_to = plan):
 * masters wait for their mirrors' rows, add them in ascending rank order and store the totals into the mirrors'
 * memory; mirror rows take the totals (apply_sum / apply_assign and the second send of GraphSum_sync_value_nccl,
 * cuda_communicate.cu:410-448).  Same F and rows as the aggregation call wrote.  DRONE_E_STATE when no such call
 * precedes.  Asynchronous on `stream`, which must be the aggregation call's stream or ordered behind it.
 */
int drone_exchange_finish(drone_xplan *plan, float *d_rows, int F, int ld, void *stream);

/*
 * Switch a plan to the peer-memory transport (one process per GPU, all GPUs in one NVLink domain): later
 * drone_exchange_sum calls on this plan fuse packing, transfer and unpacking into three kernels that store rows
 * directly into the receiving GPU's memory (CUDA IPC mappings of one buffer per rank) and order themselves with
 * epoch flags in that memory; waits are bounded (about two seconds), after which the call sequence reports
 * DRONE_E_STATE instead of hanging.  Results are bit-identical to the NCCL transport.  Collective over `comm`
 * (it exchanges the IPC handles with one ncclAllGather) and synchronous.  Every rank must enable it, with plans
 * created for the same max_features, and all ranks must then issue the same sequence of exchanges.
 * Before destroying a plan, make sure no peer is still inside an exchange (e.g. a barrier).
 * The reference has no counterpart (it always goes through grouped ncclSend/ncclRecv,
 * cuda_gcn/src/cuda/cuda_communicate.cu:296-372).
 */
int drone_xplan_enable_p2p(drone_xplan *plan, drone_comm *comm, void *stream);

/*
 * The exchange as two dense collectives, ncclReduceScatter (mirror -> master, summed) + ncclAllGather
 * (master -> mirror), over a buffer that lists every replicated vertex once, grouped by owning rank and padded to
 * equal groups.  Needs the partition's global tables: h_owner[v] = rank of v's master copy, h_replicas[v] = number
 * of ranks holding v (as drone_ebv_partition returns them).  Moves rows a rank does not hold, so it pays off only
 * when most boundary vertices are replicated on most ranks; results agree with the other transports to rounding
 * (the order of additions inside the collective is NCCL's).  Same dataflow as GraphSum_sync_value_nccl,
 * cuda_gcn/src/cuda/cuda_communicate.cu:374-448, expressed with collectives instead of grouped send/recv.
 */
typedef struct drone_dense_xplan drone_dense_xplan;
int drone_dense_xplan_create(drone_dense_xplan **out, int rank, int nranks, int n_local,
                             const int *h_local2global, int global_v, const int *h_owner,
                             const int *h_replicas, int max_features);
int drone_dense_xplan_destroy(drone_dense_xplan *plan);
/* Rows of the boundary buffer (nranks equal groups); bytes on the wire per rank and call are about
 * 2 * (nranks-1)/nranks * rows * F * 4. */
long long drone_dense_xplan_boundary_rows(const drone_dense_xplan *plan);
int drone_exchange_sum_dense(drone_dense_xplan *plan, drone_comm *comm, float *d_rows, int F, int ld, void *stream);

/*
 * The same exchange among n_parts plans held by ONE process on ONE device
 * (plans[p] is rank p of n_parts, d_rows[p] its rows): messages become
 * device-to-device copies.  For running all parts of a partition on a single
 * GPU; no counterpart in the reference.
 */
int drone_exchange_sum_local(int n_parts, drone_xplan **plans, float **d_rows, int F, const int *ld,
                             void *stream);

/* ------------------------------------------------------------------------- */
/* PageRank (the sparse aggregation at feature width 1)                        */
/* ------------------------------------------------------------------------- */

typedef struct drone_pr drone_pr;

/* Same fields, order and types as struct Response, DRONE/src/cuda/algorithm/common.h:23-27;
 * the Go worker stops when the four exchange sizes are all zero
 * (DRONE/src/tools/cuda_convert.go:47-52). */
typedef struct drone_pr_response {
    int Mirror2MasterSendSize, Mirror2MasterRecvSize, Master2MirrorSendSize, Master2MirrorRecvSize;
    int VisitedSize, LocalVertexSize;
    float CalTime, SendTime;
} drone_pr_response;

/*
 * PageRank state of one rank over its local graph (device CSR by source as in
 * drone_plan_create), the GLOBAL out-degree of every local vertex
 * (loadOutDegree / setOutDegree, DRONE/src/cuda/algorithm/pr.cu:490-515) and
 * Graph.Mirror2Worker on the device.  The exchange plan and communicator are
 * borrowed and must outlive the handle; comm may be NULL for a single rank.
 * use_double = 0 computes in float like the reference, 1 in double.
 * eps is the push threshold (1e-6 in DRONE/src/cuda/algorithm/pr.cu:11,
 * 0.01 in the CPU job DRONE/src/algorithm/PageRank.go:10).
 * Owns what struct PRValues holds (DRONE/src/cuda/algorithm/pr.h:7-16); all
 * buffers are allocated here once, none per superstep.
 */
int drone_pr_create(drone_pr **out, int n_local, int global_v, int nnz,
                    const int *d_index, const int *d_dst, const int *d_out_degree,
                    const int *d_mirror2worker, drone_xplan *xplan, drone_comm *comm,
                    int use_double, double eps);
int drone_pr_destroy(drone_pr *pr);

/* First superstep (pr = 1, push pr/outDegree, exchange).  Replaces PR_PEVal,
 * DRONE/src/cuda/algorithm/pr.cu:375-428.  Collective; synchronous. */
int drone_pr_peval(drone_pr *pr, drone_pr_response *res, void *stream);
/* Later supersteps.  Replaces PR_IncEVal, DRONE/src/cuda/algorithm/pr.cu:450-488. */
int drone_pr_inceval(drone_pr *pr, drone_pr_response *res, void *stream);

/* Synchronous power iteration: pr = 1/|V|, then `iterations` times
 * pr' = (1-d)/|V| + d * (sum over in-edges of pr[u]/outDegree[u] + dangling/|V|),
 * with the same boundary exchange.  Collective; asynchronous on `stream`. */
int drone_pr_power_iterate(drone_pr *pr, int iterations, double damping, void *stream);

/* Number of vertex ids in 0..|V|-1 that occur in no part (no edge at all).  The power iteration counts
 * them as dangling vertices so that the result is the PageRank of the whole id range; the delta
 * schedule ignores them, as the reference does.  Must be the same on every rank.  Default 0. */
int drone_pr_set_isolated_count(drone_pr *pr, long long n_isolated);

/* The same procedures over n_parts handles held by one process on one device
 * (prs[p] built with part p's exchange plan, comm NULL); res has n_parts entries. */
int drone_pr_step_local(int n_parts, drone_pr **prs, int is_peval, drone_pr_response *res, void *stream);
int drone_pr_power_iterate_local(int n_parts, drone_pr **prs, int iterations, double damping, void *stream);

/* Device arrays of the state, indexed by local id (float or double as chosen at creation): what
 * PRValues.prValue / accValue / diffValue and Graph.active / updateByMessage point to in the reference
 * (DRONE/src/cuda/algorithm/pr.h:7-16, DRONE/src/cuda/graph.h:33-35).  Owned by the handle. */
int drone_pr_device_arrays(drone_pr *pr, void **d_pr, void **d_acc, void **d_diff, int **d_active,
                           int **d_update_by_message);

/* Current values by local id into h_out (n_local floats or doubles); synchronises. */
int drone_pr_values(drone_pr *pr, void *h_out, void *stream);

/* ------------------------------------------------------------------------- */
/* Connected components and shortest paths (minimum propagation)               */
/* ------------------------------------------------------------------------- */

/*
 * The "cc_cuda" and "sssp_cuda" jobs: a value is pushed along the local out-edges until nothing changes (a label
 * as it is, a distance plus the edge length), then mirrors and masters exchange minima over the same static plan
 * as the aggregation.  One handle is one worker's state; it replaces CCValues / SSSPValues and the Graph.active /
 * Graph.updateByMessage arrays (DRONE/src/cuda/algorithm/cc.h:18-22, sssp.h:8-12, DRONE/src/cuda/graph.h:33-35).
 *
 * drone_mp_create: d_index / d_dst = the worker's CSR by source (build_graph, DRONE/src/cuda/graph.cu:94-103),
 *   d_edge_len = Graph.edgeLen (NULL: every edge has length 1, what build_graph stores), d_local2global =
 *   Graph.Local2Global; all four are device arrays the caller keeps alive while the handle exists.
 * drone_mp_peval   = CC_PEVal (cc.cu:319-383) or SSSP_PEVal (sssp.cu:398-476): start values, local run, exchange.
 *   source_global_id is SSSP's startId (ignored for labels; a worker that does not hold it starts idle).
 * drone_mp_inceval = CC_IncEVal (cc.cu:400-447) / SSSP_IncEVal (sssp.cu:494-538): vertices lowered by a message
 *   form the new frontier, local run, exchange.
 * The returned Response has the reference's meaning field by field: the four sizes count the boundary vertices that
 * changed and were sent / received, VisitedSize counts the non-zero entries of `active` (common.cu:6-16); the
 * job is over when all four sizes are zero on every worker (DRONE/src/tools/cuda_convert.go:47-52).
 *
 * Two differences from the reference's kernels, both on purpose: labels start as the GLOBAL vertex id, as in the CPU
 * job (DRONE/src/algorithm/CC.go:73-79) — cc_init (cc.cu:14) writes the local index, which workers cannot compare;
 * and a shorter distance always re-activates its vertex — sssp_exec (sssp.cu:67) asks for an improvement above
 * 1e-6.  With unit lengths the second rule gives the same distances.  Results do not depend on the order of the
 * atomics: the fixed point of a minimum is unique.  Distances use 1e8 for "not reached" (sssp.cu:33).
 */
#define DRONE_MP_CC   0
#define DRONE_MP_SSSP 1
typedef struct drone_mp drone_mp;
int drone_mp_create(drone_mp **out, int kind, int n_local, int nnz, const int *d_index, const int *d_dst,
                    const float *d_edge_len, const int *d_local2global, drone_xplan *xplan, drone_comm *comm);
int drone_mp_destroy(drone_mp *job);
int drone_mp_peval(drone_mp *job, int source_global_id, drone_pr_response *res, void *stream);
int drone_mp_inceval(drone_mp *job, drone_pr_response *res, void *stream);
/* One superstep of ALL parts of a partition held by one process on one device (jobs[p] is worker p of n_parts):
 * messages become device-to-device copies; res[n_parts].  No counterpart in the reference. */
int drone_mp_step_local(int n_parts, drone_mp **jobs, int is_peval, int source_global_id, drone_pr_response *res,
                        void *stream);
/* Device arrays of the state by local id, owned by the handle: what CCValues.ccValue / SSSPValues.distance and
 * Graph.active / Graph.updateByMessage point to in the reference (int32 labels or float32 distances). */
int drone_mp_device_arrays(drone_mp *job, void **d_value, int **d_active, int **d_update_by_message);
/* Current values by local id into h_out: n_local int32 labels or float32 distances; synchronises. */
int drone_mp_values(drone_mp *job, void *h_out, void *stream);

/*
 * EBV vertex-cut partitioner (host, single process).  Input: directed edge
 * list in global ids.  Output: the edges grouped by part in the order the
 * reference writes them to G.<p> (h_out_u/h_out_v hold all kept edges,
 * h_part_offset[n_parts+1] delimits the parts), h_replicas[v] = number of parts
 * holding v, h_owner[v] = part of v's master copy (-1 if v has no edge).
 * flags: DRONE_EBV_KEEP_SELF_LOOPS keeps edges u==u (cuda_gcn/src/tools/EBV_mpi.cpp:217, the variant used for GCN
 * inputs; EBV_mpi.cpp:219 drops them).  DRONE_EBV_STD_SORT_TIES sorts every rank's share with std::sort, the call
 * the reference makes (EBV_mpi.cpp:265), instead of the default stable sort: edges with equal degree sums then come
 * in the order the C++ library's algorithm leaves them, and a build against the same library returns the
 * reference's parts edge for edge (checked against files the reference's partitioner wrote).  The default order
 * does not depend on the library.
 * Restates EBV_mpi.cpp:212-374 (deal, local-degree sort, batched scoring) and
 * :549-581 (master = replica number id mod #replicas), as a simulation of its
 * n_parts MPI ranks.
 */
#define DRONE_EBV_KEEP_SELF_LOOPS 1
#define DRONE_EBV_STD_SORT_TIES 2
int drone_ebv_partition(int n_vertices, long long n_edges, const int *h_u, const int *h_v,
                        int n_parts, int flags,
                        int *h_out_u, int *h_out_v, long long *h_part_offset,
                        int *h_owner, int *h_replicas);

/*
 * Which parts hold which vertex, from the partitioned edge list drone_ebv_partition returned: h_bits[v] has bit p
 * set when v is an endpoint of an edge of part p.  One word per vertex is what a rank needs of the other parts to
 * write its Master.<p> rows (EBV_mpi.cpp:583-603 walks the parts' vertex sets for the same purpose).
 */
int drone_presence_bits_host(int n_vertices, int n_parts, const int *h_u, const int *h_v,
                             const long long *h_part_offset, unsigned long long *h_bits);

/*
 * Loading from disk (host code).
 *
 * drone_text_ints_count / drone_text_ints_read: all integers of a text file in file order, and for every line that
 * holds at least one integer the index of its first value (line_start[n_lines] = n_values closes the list; pass
 * NULL when lines do not matter).  Reads the three formats of a partition directory — G.<p> ("u v"), Master.<p>
 * ("vertex worker worker ..."), Mirror.<p> ("vertex worker") — with all host threads; replaces the fscanf / getline
 * loops of Parser::parseGraph, cuda_gcn/src/common/parser.cu:72-131, and the line-by-line reader of the Go loader,
 * DRONE/src/graph/cuda_graph.go:32-60.  Anything but digits, signs and white space is an error (byte offset in the
 * message).  Call count first, allocate, then read; or read straight away into buffers of file size / 2 + 1 entries,
 * which always suffice (an integer takes at least one digit and one separator), and take the counts it returns.
 *
 * drone_partition_write / _read_header / _read: one binary file for a whole partition: header, part offsets, owner,
 * replicas, presence words (see drone_presence_bits_host), then u and v of all parts, parts one after the other in
 * G.<p> order.  drone_partition_read with part >= 0 reads that part's edges only (part = -1: all edges); any output
 * pointer may be NULL.  part_offset needs n_parts + 1 entries (at most 65).  No counterpart in the reference, whose
 * workers each parse their text files at every start.
 */
int drone_text_ints_count(const char *path, long long *n_values, long long *n_lines);
int drone_text_ints_read(const char *path, int *values, long long cap_values, long long *line_start, long long cap_lines,
                         long long *n_values, long long *n_lines);
/* The integers of a "u v" per line file dealt into two arrays (each needs room for file size / 4 + 1 entries). */
int drone_text_edges_read(const char *path, int *u, int *v, long long cap_edges, long long *n_edges);
int drone_partition_write(const char *path, int n_vertices, int n_parts, const long long *part_offset,
                          const int *u, const int *v, const int *owner, const int *replicas,
                          const unsigned long long *present_bits);
int drone_partition_read_header(const char *path, int *n_vertices, int *n_parts, long long *part_offset);
int drone_partition_read(const char *path, int part, int *u, int *v, int *owner, int *replicas,
                         unsigned long long *present_bits);

/*
 * One rank's local graph from the edge list of its G.<p> file (host arrays in,
 * host arrays out): local ids in first-seen order, CSR by source vertex with
 * destinations in edge-list order.  h_g2l[global_v] gets -1 for absent
 * vertices; h_l2g / h_index need room for min(global_v, 2*n_edges) (+1)
 * entries.  The host half of build_graph, cuda_gcn/src/cuda/graph.cu:54-103
 * (twin: DRONE/src/cuda/graph.cu).
 */
int drone_graph_build_host(int global_v, int n_edges, const int *h_u, const int *h_v,
                           int *h_g2l, int *h_l2g, int *h_index, int *h_dst, int *n_local_out);

/*
 * The same local graph built on the device from device arrays d_u / d_v (n_edges < 2^30): d_g2l[global_v],
 * d_l2g and d_index with room for min(global_v, 2*n_edges) (+1) entries, d_dst[n_edges]; *n_local_out is written on
 * the host.  Output identical to drone_graph_build_host; the call synchronises `stream` and allocates scratch of
 * about 12 bytes per vertex id and 12 bytes per edge.  Replaces the serial host loops of build_graph,
 * cuda_gcn/src/cuda/graph.cu:54-103.
 */
int drone_graph_build_device(int global_v, int n_edges, const int *d_u, const int *d_v,
                             int *d_g2l, int *d_l2g, int *d_index, int *d_dst, int *n_local_out, void *stream);

/*
 * Routing tables by local id from the rows of Master.<p> (master_vertex[i] has
 * mirror_number[i] mirrors on the ranks listed consecutively in mirror_workers)
 * and Mirror.<p> (mirror_vertex[i]'s master lives on master_worker[i]).
 * Same tables as addMasterRoute / addMirrorRoute, cuda_gcn/src/cuda/graph.cu:281-367.
 */
int drone_route_tables_host(int n_local, const int *h_g2l,
                            const int *master_vertex, const int *mirror_number, const int *mirror_workers,
                            int master_size, int mirror_worker_size,
                            const int *mirror_vertex, const int *master_worker, int mirror_size,
                            int *h_master_worker_index, int *h_master2workers, int *h_mirror2worker);

/*
 * Seeded R-MAT edge list (quadrant probabilities a, b, c, 1-a-b-c; `scale` bits
 * per endpoint).  Edge number e depends only on (seed, e): the device and host
 * entry points return identical edges, and a range [first_edge, first_edge+n)
 * can be produced independently of the rest.  Self-loops and duplicates are
 * NOT removed here.  No counterpart in the reference (it reads edge-list
 * files); this produces the synthetic graphs the tests and benchmarks use.
 */
int drone_rmat_edges(int scale, long long n_edges, unsigned long long seed,
                     double a, double b, double c, long long first_edge,
                     int *d_u, int *d_v, void *stream);
int drone_rmat_edges_host(int scale, long long n_edges, unsigned long long seed,
                          double a, double b, double c, long long first_edge,
                          int *h_u, int *h_v);

/* Number of kernels the library has launched on behalf of the calling process. */
long long drone_kernel_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* DRONE_B200_H */
