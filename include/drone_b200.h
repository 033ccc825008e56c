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
 * Same operation with HOST operands: copies X to the device, aggregates, and
 * copies Y back, synchronising before it returns.  Device staging buffers are
 * owned by the plan and reused across calls.  h_X and h_Y are dense
 * [n_rows, F] row-major; pinned memory makes the copies asynchronous DMA.
 * This is the call a host-side (cgo / CPU) user of the path makes.
 */
int drone_spmm_host(drone_plan *plan, int orientation, int F,
                    const float *h_X, float *h_Y);

/* Pinned host memory for drone_spmm_host operands. */
int drone_host_alloc(void **out, size_t bytes);
int drone_host_free(void *ptr);

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
