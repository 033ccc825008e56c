// PageRank over an EBV-partitioned graph: the propagation step is the same sparse
// aggregation as GraphSum at feature width 1.
//
// Two schedules share the kernels below:
//  * DRONE's delta PageRank (PR_PEVal / PR_IncEVal, DRONE/src/cuda/algorithm/pr.cu:375-488):
//    pr starts at 1, a vertex whose value moved by at least eps pushes (new-old)/outDegree
//    to its out-neighbours, boundary vertices are reconciled mirror -> master (add) and
//    master -> mirror (assign), dangling mass goes through a one-element all-reduce.
//  * synchronous power iteration (damping d, fixed iteration count, start 1/|V|).
//
// Where the reference pushes along out-edges with atomicAdd (pr.cu:14-87), this
// implementation pulls along in-edges of the transposed local graph: every vertex
// publishes {delta, pushed} once and every vertex sums what its in-neighbours
// published.  Same arithmetic, no atomics on values, fixed summation order.
// The boundary exchange is static and dense (all mirrors of a peer in one
// message, ordered by global id); each entry carries the flag that the
// reference expresses by sending or not sending the vertex, so the counts the
// caller uses to detect termination (Response, common.h:23-27) are reproduced.
#include "exchange.cuh"
#include "plan.cuh"

#include <chrono>
#include <cstdlib>
#include <new>
#include <vector>

namespace drone {
int xplan_ensure_device(drone_xplan *x);
}

struct drone_pr {
    int device = 0, n_local = 0, global_v = 0, nnz = 0;
    bool dbl = false;
    double eps = 1e-6;
    drone_plan *plan = nullptr;       // owned: transposed local graph + chunk lists (values unused)
    drone_xplan *xplan = nullptr;     // borrowed
    drone_comm *comm = nullptr;       // borrowed (may be NULL for a single part)
    int *out_degree = nullptr, *mirror2worker = nullptr;
    void *pr = nullptr, *acc = nullptr, *diff = nullptr, *push = nullptr;   // real[n], real[n], real[n], real2[n]
    // Large parts: where vertex i publishes its {delta, pushed} pair.  The pairs lie in the order of how often they are
    // gathered (most gathered first) and the pull lists' columns are renumbered to match, so that the hot pairs are
    // contiguous and stay in L2 (a pair is 8 bytes of a 32-byte sector).  NULL: pair i lies at i.
    int *place = nullptr;
    int *active = nullptr, *ubm = nullptr;
    void *scalars = nullptr;          // real[4]: globalDiff, globalAcc, dangling (power mode), spare
    void *block_sums = nullptr;       // real[kReduceBlocks]
    void *partials = nullptr;         // real2[n_partials]
    void *send = nullptr, *recv = nullptr;   // real2[max(up, down)]
    int *counters = nullptr;          // [0..3] exchange counts, [4] active count
    bool started = false;
    long long n_isolated = 0;         // vertex ids that occur in no part (power iteration treats them as dangling)
};

namespace drone {

static const int kReduceBlocks = 1024;

template <typename R> struct alignas(2 * sizeof(R)) Pair { R val, flag; };
template <typename R> struct NcclType;
template <> struct NcclType<float> { static constexpr ncclDataType_t value = ncclFloat; };
template <> struct NcclType<double> { static constexpr ncclDataType_t value = ncclDouble; };

template <typename R> __device__ __forceinline__ R fma_r(R a, R b, R c);
template <> __device__ __forceinline__ float fma_r<float>(float a, float b, float c) { return fmaf(a, b, c); }
template <> __device__ __forceinline__ double fma_r<double>(double a, double b, double c) { return fma(a, b, c); }

// Sum of v over the block in a fixed order (tree over warps), result in thread 0.
template <typename R>
__device__ R block_sum(R v) {
    __shared__ double sm[32];
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) sm[w] = (double)v;
    __syncthreads();
    R tot = 0;
    if (threadIdx.x == 0)
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += (R)sm[i];
    return tot;
}

// pr = 1, acc = diff = 0, flags cleared; publish pr/outDegree; dangling mass of non-mirror vertices to block sums.
// (pr_init, DRONE/src/cuda/algorithm/pr.cu:14-37, plus the fills of PR_PEVal :391-394.)
template <typename R>
__global__ void pr_init_kernel(R *pr, R *acc, R *diff, Pair<R> *push, int *active, int *ubm,
                               const int *__restrict__ out_degree, const int *__restrict__ mirror2worker, int n,
                               int global_v, R start, R *block_sums, const int *__restrict__ place) {
    R dangling = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        pr[i] = start;
        acc[i] = 0;
        diff[i] = 0;
        active[i] = 0;
        ubm[i] = 0;
        Pair<R> p;
        p.val = 0;
        p.flag = 0;
        const int od = out_degree[i];
        if (od == 0) {
            if (mirror2worker[i] == -1) dangling += start / global_v;
        } else {
            p.val = start / od;
            p.flag = 1;
        }
        push[place ? place[i] : i] = p;
    }
    const R tot = block_sum<R>(dangling);
    if (threadIdx.x == 0) block_sums[blockIdx.x] = tot;
}

// scalars[0] (globalDiff) += sum of block sums, in block order.
template <typename R>
__global__ void pr_fold_block_sums_kernel(const R *block_sums, int n_blocks, R *scalars, int slot) {
    if (blockIdx.x != 0 || threadIdx.x >= 32) return;
    R s = 0;                                          // lane l adds blocks l, l+32, ...; then a fixed tree
    for (int i = threadIdx.x; i < n_blocks; i += 32) s += block_sums[i];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) scalars[slot] += s;
}

// globalAcc += globalDiff; globalDiff = 0   (pr_process_messages, pr.cu:435-438)
template <typename R>
__global__ void pr_roll_scalars_kernel(R *scalars) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        scalars[1] += scalars[0];
        scalars[0] = 0;
    }
}

// pr_process_messages (pr.cu:430-448) fused with pr_increment (pr.cu:51-87).
template <typename R>
__global__ void pr_increment_kernel(R *pr, R *acc, R *diff, Pair<R> *push, int *active, int *ubm,
                                    const int *__restrict__ out_degree, const int *__restrict__ mirror2worker, int n,
                                    int global_v, R eps, const R *scalars, R *block_sums,
                                    const int *__restrict__ place) {
    const R alpha = (R)0.85f;                // pr.cu:12 declares a float constant
    const R one_minus_alpha = (R)1 - alpha;
    const R gacc = scalars[1];
    R dangling = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        active[i] = 0;
        ubm[i] = 0;
        const R a = acc[i] + diff[i];
        acc[i] = a;
        diff[i] = 0;
        const R old = pr[i];
        const R now = fma_r<R>(alpha, a + gacc, one_minus_alpha);
        R d = now - old;
        if (d < 0) d = -d;
        Pair<R> p;
        p.val = 0;
        p.flag = 0;
        if (!(d < eps)) {
            const int od = out_degree[i];
            if (od == 0) {
                if (mirror2worker[i] == -1) dangling += (now - old) / global_v;
            } else {
                p.val = (now - old) / od;
                p.flag = 1;
            }
            pr[i] = now;
        }
        push[place ? place[i] : i] = p;
    }
    const R tot = block_sum<R>(dangling);
    if (threadIdx.x == 0) block_sums[blockIdx.x] = tot;
}

// ---- pull along in-edges: diff[v] = sum of published deltas, active[v] = any in-neighbour pushed ----

// Short rows through the plan's short-row stream (columns with an end-of-row flag, ranges of whole rows): one warp
// per range, one lane per entry, so the column reads are coalesced and 32 gathers are in flight per warp; the sums of
// the rows inside a batch come from a segmented scan (fixed tree order), rows that continue into the next batch
// carry their partial sum over.
template <typename R>
__global__ void pr_pull_stream_kernel(const int *__restrict__ s_range_row, int n_ranges, const int *__restrict__ s_rowptr,
                                      const int *__restrict__ s_rows, const int *__restrict__ s_col,
                                      const Pair<R> *__restrict__ push, R *diff, int *active) {
    const int lane = threadIdx.x & 31;
    const long long range = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    if (range >= n_ranges) return;
    int ri = s_range_row[range];
    const int k0 = s_rowptr[ri], k1 = s_rowptr[s_range_row[range + 1]];
    R carry_v = 0, carry_f = 0;
    unsigned c_next = (k0 + lane < k1) ? (unsigned)s_col[k0 + lane] : 0u;
    for (int base = k0; base < k1; base += 32) {
        const unsigned c = c_next;
        const bool live = base + lane < k1;
        c_next = (base + 32 + lane < k1) ? (unsigned)s_col[base + 32 + lane] : 0u;
        R v = 0, f = 0;
        if (live && !(c & kPlaceholder)) {
            const Pair<R> p = push[c & kColMask];
            v = p.val;
            f = p.flag;
        }
        const bool end = live && (c & kLastInRow);
        const unsigned ends = __ballot_sync(0xffffffffu, end);
        const unsigned heads = (ends << 1) | 1u;                       // lane starts a row if the lane before ended one
        const int start = 31 - __clz(heads & (0xffffffffu >> (31 - lane)));
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const R tv = __shfl_up_sync(0xffffffffu, v, d);
            const R tf = __shfl_up_sync(0xffffffffu, f, d);
            if (lane - d >= start) { v += tv; f += tf; }
        }
        if (start == 0) { v += carry_v; f += carry_f; }                // the row open at the start of this batch
        if (end) {
            const int row = s_rows[ri + __popc(ends & ((1u << lane) - 1u))];
            diff[row] = v;
            active[row] = f > 0 ? 1 : 0;
        }
        const R last_v = __shfl_sync(0xffffffffu, v, 31), last_f = __shfl_sync(0xffffffffu, f, 31);
        const bool open = !(ends >> 31);
        carry_v = open ? last_v : (R)0;
        carry_f = open ? last_f : (R)0;
        ri += __popc(ends);
    }
}

template <typename R>
__global__ void pr_pull_chunks_kernel(const Chunk *__restrict__ chunks, int n_chunks, const int *__restrict__ col,
                                      const Pair<R> *__restrict__ push, R *diff, int *active, Pair<R> *partials) {
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    if (warp >= n_chunks) return;
    const Chunk ch = chunks[warp];
    R sum = 0, flag = 0;
    int k = lane;
    for (; k + 96 < ch.len; k += 128) {          // four independent gathers in flight per lane
        const int c0 = col[ch.k0 + k], c1 = col[ch.k0 + k + 32], c2 = col[ch.k0 + k + 64], c3 = col[ch.k0 + k + 96];
        const Pair<R> p0 = push[c0], p1 = push[c1], p2 = push[c2], p3 = push[c3];
        sum += p0.val; flag += p0.flag;
        sum += p1.val; flag += p1.flag;
        sum += p2.val; flag += p2.flag;
        sum += p3.val; flag += p3.flag;
    }
    for (; k < ch.len; k += 32) {
        const Pair<R> p = push[col[ch.k0 + k]];
        sum += p.val;
        flag += p.flag;
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
        flag += __shfl_xor_sync(0xffffffffu, flag, o);
    }
    if (lane == 0) {
        if (ch.slot < 0) {
            diff[ch.row] = sum;
            active[ch.row] = flag > 0 ? 1 : 0;
        } else {
            Pair<R> p;
            p.val = sum;
            p.flag = flag;
            partials[ch.slot] = p;
        }
    }
}

template <typename R>
__global__ void pr_pull_reduce_kernel(const SplitRow *__restrict__ split, int n_split,
                                      const Pair<R> *__restrict__ partials, R *diff, int *active) {
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    if (warp >= n_split) return;
    const SplitRow sr = split[warp];
    R sum = 0, flag = 0;
    for (int k = lane; k < sr.nslots; k += 32) {
        const Pair<R> p = partials[sr.slot0 + k];
        sum += p.val;
        flag += p.flag;
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
        flag += __shfl_xor_sync(0xffffffffu, flag, o);
    }
    if (lane == 0) {
        diff[sr.row] = sum;
        active[sr.row] = flag > 0 ? 1 : 0;
    }
}

// ---- boundary exchange (Mirror2MasterSend pr.cu:215-297, Master2MirrorSend :299-373) ----

// every mirror row, in plan order; active mirrors carry their diff (pr_generate_sendBuff_mirror :125-148)
template <typename R>
__global__ void pr_pack_up_kernel(const int *__restrict__ up_rows, int n_up, const R *diff, const int *active,
                                  Pair<R> *send, int *counters) {
    int cnt = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_up; i += gridDim.x * blockDim.x) {
        const int row = up_rows[i];
        Pair<R> p;
        const int a = active[row];
        p.val = a ? diff[row] : (R)0;
        p.flag = (R)a;
        send[i] = p;
        cnt += a;
    }
    if (cnt) atomicAdd(counters + 0, cnt);
}

// master rows add what their mirrors sent, ascending rank order (pr_process_recvBuff_Add :167-187)
template <typename R>
__global__ void pr_apply_up_kernel(const int *__restrict__ m_rows, const int *__restrict__ m_off,
                                   const int *__restrict__ m_pos, int n_masters, const Pair<R> *recv, R *diff, int *ubm,
                                   int *counters) {
    int cnt = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_masters; i += gridDim.x * blockDim.x) {
        const int row = m_rows[i];
        R d = diff[row];
        int got = 0;
        for (int k = m_off[i]; k < m_off[i + 1]; ++k) {
            const Pair<R> p = recv[m_pos[k]];
            if (p.flag > 0) {
                d += p.val;
                ++got;
            }
        }
        if (got) {
            diff[row] = d;
            ubm[row] = 1;
            cnt += got;
        }
    }
    if (cnt) atomicAdd(counters + 1, cnt);
}

// masters that changed publish their total to every mirror (pr_generate_sendBuff_master :150-172)
template <typename R>
__global__ void pr_pack_down_kernel(const int *__restrict__ down_rows, int n_down, const R *diff, const int *active,
                                    const int *ubm, Pair<R> *send, int *counters) {
    int cnt = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_down; i += gridDim.x * blockDim.x) {
        const int row = down_rows[i];
        const int f = (active[row] != 0 || ubm[row] != 0) ? 1 : 0;
        Pair<R> p;
        p.val = diff[row];
        p.flag = (R)f;
        send[i] = p;
        cnt += f;
    }
    if (cnt) atomicAdd(counters + 2, cnt);
}

// mirrors take the master's total (pr_process_recvBuff_Exch :189-213)
template <typename R>
__global__ void pr_apply_down_kernel(const int *__restrict__ up_rows, int n_up, const Pair<R> *recv, R *diff, int *ubm,
                                     int *counters) {
    int cnt = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_up; i += gridDim.x * blockDim.x) {
        const Pair<R> p = recv[i];
        if (p.flag > 0) {
            const int row = up_rows[i];
            diff[row] = p.val;
            ubm[row] = 1;
            ++cnt;
        }
    }
    if (cnt) atomicAdd(counters + 3, cnt);
}

__global__ void pr_count_active_kernel(const int *active, int n, int *counters) {
    int cnt = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) cnt += active[i] != 0;
    if (cnt) atomicAdd(counters + 4, cnt);
}

// ---- power iteration ----

// publish pr/outDegree, collect dangling mass (non-mirror copies only) into block sums
template <typename R>
__global__ void pr_power_prepare_kernel(const R *pr, Pair<R> *push, const int *__restrict__ out_degree,
                                        const int *__restrict__ mirror2worker, int n, R *block_sums,
                                        const int *__restrict__ place) {
    R dangling = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        Pair<R> p;
        p.val = 0;
        p.flag = 0;
        const int od = out_degree[i];
        if (od == 0) {
            if (mirror2worker[i] == -1) dangling += pr[i];
        } else {
            p.val = pr[i] / od;
            p.flag = 1;
        }
        push[place ? place[i] : i] = p;
    }
    const R tot = block_sum<R>(dangling);
    if (threadIdx.x == 0) block_sums[blockIdx.x] = tot;
}

// scalars[2] += n_isolated * (common value of the isolated vertices): ids that occur in no part have no
// edges at all, so they are dangling and all hold scalars[3]; one rank adds their mass.
template <typename R>
__global__ void pr_power_isolated_kernel(R *scalars, long long n_isolated) {
    if (threadIdx.x == 0 && blockIdx.x == 0) scalars[2] += (R)n_isolated * scalars[3];
}

// pr' = (1-d)/V + d * (sum over in-edges + dangling/V); the isolated vertices' value follows the same rule.
// The same pass publishes pr'/outDegree and collects the dangling mass for the next iteration.
template <typename R>
__global__ void pr_power_apply_kernel(R *pr, const R *diff, Pair<R> *push, const int *__restrict__ out_degree,
                                      const int *__restrict__ mirror2worker, int n, int global_v, R damping, R *scalars,
                                      R *block_sums, const int *__restrict__ place) {
    const R dang = scalars[2];
    const R base = ((R)1 - damping) / global_v;
    R dangling = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const R now = base + damping * (diff[i] + dang / global_v);
        pr[i] = now;
        Pair<R> p;
        p.val = 0;
        p.flag = 0;
        const int od = out_degree[i];
        if (od == 0) {
            if (mirror2worker[i] == -1) dangling += now;
        } else {
            p.val = now / od;
            p.flag = 1;
        }
        push[place ? place[i] : i] = p;
    }
    const R tot = block_sum<R>(dangling);
    if (threadIdx.x == 0) block_sums[blockIdx.x] = tot;
    if (blockIdx.x == 0 && threadIdx.x == 0) scalars[3] = base + damping * (dang / global_v);
}

template <typename R>
__global__ void pr_set_scalar_kernel(R *scalars, int slot, R value) {
    if (threadIdx.x == 0 && blockIdx.x == 0) scalars[slot] = value;
}

static inline int grid1d(long long n, int cap = 148 * 16) {
    long long g = (n + 255) / 256;
    if (g < 1) g = 1;
    if (g > cap) g = cap;
    return (int)g;
}

// Moves the packed boundary entries: up == true sends my `up` slices and receives `down` slices.
struct Transport {
    virtual int move(std::vector<drone_pr *> &parts, bool up, size_t pair_bytes, bool dbl, cudaStream_t st) = 0;
    // where the entries sent to part p lie after move(): its receive buffer unless the transport delivers elsewhere
    virtual const void *received(drone_pr *p) { return p->recv; }
    virtual int allreduce(std::vector<drone_pr *> &parts, int slot, bool dbl, cudaStream_t st) = 0;
    virtual ~Transport() {}
};

struct NcclTransport : Transport {
    int move(std::vector<drone_pr *> &parts, bool up, size_t pair_bytes, bool dbl, cudaStream_t st) override {
        drone_pr *p = parts[0];
        const drone_xplan *x = p->xplan;
        if (x->nranks == 1) return DRONE_OK;
        const std::vector<int> &s_off = up ? x->up_off : x->down_off;
        const std::vector<int> &r_off = up ? x->down_off : x->up_off;
        const ncclDataType_t ty = dbl ? ncclDouble : ncclFloat;
        DRONE_NCCL(ncclGroupStart());
        for (int q = 0; q < x->nranks; ++q) {
            if (q == x->rank) continue;
            const size_t ns = (size_t)(s_off[q + 1] - s_off[q]) * 2, nr = (size_t)(r_off[q + 1] - r_off[q]) * 2;
            if (ns) DRONE_NCCL(ncclSend((char *)p->send + (size_t)s_off[q] * pair_bytes, ns, ty, q, p->comm->comm, st));
            if (nr) DRONE_NCCL(ncclRecv((char *)p->recv + (size_t)r_off[q] * pair_bytes, nr, ty, q, p->comm->comm, st));
        }
        DRONE_NCCL(ncclGroupEnd());
        return DRONE_OK;
    }
    int allreduce(std::vector<drone_pr *> &parts, int slot, bool dbl, cudaStream_t st) override {
        drone_pr *p = parts[0];
        if (!p->comm || p->comm->nranks == 1) return DRONE_OK;
        char *ptr = (char *)p->scalars + (size_t)slot * (dbl ? 8 : 4);
        DRONE_NCCL(ncclAllReduce(ptr, ptr, 1, dbl ? ncclDouble : ncclFloat, ncclSum, p->comm->comm, st));
        return DRONE_OK;
    }
};

// One process per GPU on one NVLink domain: entries are stored straight into the receiver's memory
// (the exchange plan's peer-memory transport, exchange_p2p.cu); the scalar sums stay on NCCL.
struct PeerTransport : NcclTransport {
    const void *landed = nullptr;
    int move(std::vector<drone_pr *> &parts, bool up, size_t pair_bytes, bool, cudaStream_t st) override {
        drone_pr *p = parts[0];
        if (p->xplan->nranks == 1) return DRONE_OK;
        return p2p_move_elements(p->xplan, p->send, pair_bytes, up, st, &landed);
    }
    const void *received(drone_pr *p) override { return p->xplan->nranks == 1 ? p->recv : landed; }
};

// The transport of a job that runs as one process per GPU: peer memory when the exchange plan has it enabled and its
// receive areas are wide enough for a {value, flag} pair, grouped send/recv otherwise.
static bool use_peer_transport(const drone_pr *p) {
    return p->xplan->p2p != nullptr && (size_t)p->xplan->max_features * 4 >= (p->dbl ? 16u : 8u);
}

template <typename R>
__global__ void pr_sum_scalars_kernel(R **scalars, int n_parts, int slot) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        R s = 0;
        for (int p = 0; p < n_parts; ++p) s += scalars[p][slot];
        for (int p = 0; p < n_parts; ++p) scalars[p][slot] = s;
    }
}

// all parts in one process on one device: messages are device-to-device copies
struct LocalTransport : Transport {
    void **d_ptrs = nullptr;
    ~LocalTransport() override { cudaFree(d_ptrs); }
    int move(std::vector<drone_pr *> &parts, bool up, size_t pair_bytes, bool, cudaStream_t st) override {
        const int P = (int)parts.size();
        for (int p = 0; p < P; ++p)
            for (int q = 0; q < P; ++q) {
                if (p == q) continue;
                const std::vector<int> &s_off = up ? parts[p]->xplan->up_off : parts[p]->xplan->down_off;
                const std::vector<int> &r_off = up ? parts[q]->xplan->down_off : parts[q]->xplan->up_off;
                const size_t ns = (size_t)(s_off[q + 1] - s_off[q]), nr = (size_t)(r_off[p + 1] - r_off[p]);
                if (ns != nr)
                    return set_error(DRONE_E_STATE, "exchange plans disagree between parts %d and %d (%zu vs %zu rows)", p, q,
                                     ns, nr);
                if (ns)
                    DRONE_CUDA(cudaMemcpyAsync((char *)parts[q]->recv + (size_t)r_off[p] * pair_bytes,
                                               (char *)parts[p]->send + (size_t)s_off[q] * pair_bytes, ns * pair_bytes,
                                               cudaMemcpyDeviceToDevice, st));
            }
        return DRONE_OK;
    }
    int allreduce(std::vector<drone_pr *> &parts, int slot, bool dbl, cudaStream_t st) override {
        const int P = (int)parts.size();
        if (!d_ptrs) DRONE_CUDA(cudaMalloc(&d_ptrs, sizeof(void *) * 64));
        std::vector<void *> h(P);
        for (int p = 0; p < P; ++p) h[p] = parts[p]->scalars;
        DRONE_CUDA(cudaMemcpyAsync(d_ptrs, h.data(), sizeof(void *) * P, cudaMemcpyHostToDevice, st));
        DRONE_CUDA(cudaStreamSynchronize(st));  // h goes out of scope
        if (dbl) pr_sum_scalars_kernel<double><<<1, 32, 0, st>>>((double **)d_ptrs, P, slot);
        else pr_sum_scalars_kernel<float><<<1, 32, 0, st>>>((float **)d_ptrs, P, slot);
        DRONE_LAUNCH_CHECK("pr_sum_scalars_kernel");
        return DRONE_OK;
    }
};

template <typename R>
static int pull(drone_pr *p, cudaStream_t st) {
    const Side &s = p->plan->side[DRONE_OP_AT];
    const int n = p->n_local;
    (void)n;
    if (s.n_short_ranges > 0) {
        pr_pull_stream_kernel<R><<<ceil_div(s.n_short_ranges, 8), 256, 0, st>>>(
            s.s_range_row, s.n_short_ranges, s.s_rowptr, s.s_rows, s.s_col, (const Pair<R> *)p->push, (R *)p->diff,
            p->active);
        DRONE_LAUNCH_CHECK("pr_pull_stream_kernel");
    }
    if (s.n_chunks > 0) {
        pr_pull_chunks_kernel<R><<<ceil_div(s.n_chunks, 8), 256, 0, st>>>(s.chunks, s.n_chunks, s.col,
                                                                           (const Pair<R> *)p->push, (R *)p->diff,
                                                                           p->active, (Pair<R> *)p->partials);
        DRONE_LAUNCH_CHECK("pr_pull_chunks_kernel");
    }
    if (s.n_split_rows > 0) {
        pr_pull_reduce_kernel<R><<<ceil_div(s.n_split_rows, 8), 256, 0, st>>>(s.split, s.n_split_rows,
                                                                               (const Pair<R> *)p->partials, (R *)p->diff,
                                                                               p->active);
        DRONE_LAUNCH_CHECK("pr_pull_reduce_kernel");
    }
    return DRONE_OK;
}

// mirror -> master (add), master -> mirror (assign), over all parts in the list
template <typename R>
static int exchange(std::vector<drone_pr *> &parts, Transport &tr, cudaStream_t st) {
    int rc;
    for (drone_pr *p : parts) {
        const drone_xplan *x = p->xplan;
        const int n_up = (int)x->up_rows.size();
        if (n_up) {
            pr_pack_up_kernel<R><<<grid1d(n_up), 256, 0, st>>>(x->d_up_rows, n_up, (const R *)p->diff, p->active,
                                                              (Pair<R> *)p->send, p->counters);
            DRONE_LAUNCH_CHECK("pr_pack_up_kernel");
        }
    }
    if ((rc = tr.move(parts, true, sizeof(Pair<R>), sizeof(R) == 8, st))) return rc;
    for (drone_pr *p : parts) {
        const drone_xplan *x = p->xplan;
        const int n_m = (int)x->m_rows.size(), n_down = (int)x->down_rows.size();
        if (n_m) {
            pr_apply_up_kernel<R><<<grid1d(n_m), 256, 0, st>>>(x->d_m_rows, x->d_m_off, x->d_m_pos, n_m,
                                                              (const Pair<R> *)tr.received(p), (R *)p->diff, p->ubm, p->counters);
            DRONE_LAUNCH_CHECK("pr_apply_up_kernel");
        }
        if (n_down) {
            pr_pack_down_kernel<R><<<grid1d(n_down), 256, 0, st>>>(x->d_down_rows, n_down, (const R *)p->diff, p->active,
                                                                  p->ubm, (Pair<R> *)p->send, p->counters);
            DRONE_LAUNCH_CHECK("pr_pack_down_kernel");
        }
    }
    if ((rc = tr.move(parts, false, sizeof(Pair<R>), sizeof(R) == 8, st))) return rc;
    for (drone_pr *p : parts) {
        const drone_xplan *x = p->xplan;
        const int n_up = (int)x->up_rows.size();
        if (n_up) {
            pr_apply_down_kernel<R><<<grid1d(n_up), 256, 0, st>>>(x->d_up_rows, n_up, (const Pair<R> *)tr.received(p), (R *)p->diff,
                                                                 p->ubm, p->counters);
            DRONE_LAUNCH_CHECK("pr_apply_down_kernel");
        }
    }
    return DRONE_OK;
}

template <typename R>
static int delta_step(std::vector<drone_pr *> &parts, bool peval, Transport &tr, drone_pr_response *res,
                      cudaStream_t st) {
    using clock = std::chrono::steady_clock;
    const auto t0 = clock::now();
    int rc;
    for (drone_pr *p : parts) {
        if (!peval && !p->started) return set_error(DRONE_E_STATE, "PR_IncEVal called before PR_PEVal");
        DRONE_CUDA(cudaMemsetAsync(p->counters, 0, sizeof(int) * 8, st));
        const int n = p->n_local;
        const int grid = grid1d(n, kReduceBlocks);
        if (peval) {
            DRONE_CUDA(cudaMemsetAsync(p->scalars, 0, sizeof(R) * 4, st));
            pr_init_kernel<R><<<grid, 256, 0, st>>>((R *)p->pr, (R *)p->acc, (R *)p->diff, (Pair<R> *)p->push, p->active,
                                                    p->ubm, p->out_degree, p->mirror2worker, n, p->global_v, (R)1,
                                                    (R *)p->block_sums, p->place);
            DRONE_LAUNCH_CHECK("pr_init_kernel");
        } else {
            pr_roll_scalars_kernel<R><<<1, 32, 0, st>>>((R *)p->scalars);
            DRONE_LAUNCH_CHECK("pr_roll_scalars_kernel");
            pr_increment_kernel<R><<<grid, 256, 0, st>>>((R *)p->pr, (R *)p->acc, (R *)p->diff, (Pair<R> *)p->push,
                                                         p->active, p->ubm, p->out_degree, p->mirror2worker, n,
                                                         p->global_v, (R)p->eps, (const R *)p->scalars,
                                                         (R *)p->block_sums, p->place);
            DRONE_LAUNCH_CHECK("pr_increment_kernel");
        }
        pr_fold_block_sums_kernel<R><<<1, 32, 0, st>>>((const R *)p->block_sums, grid, (R *)p->scalars, 0);
        DRONE_LAUNCH_CHECK("pr_fold_block_sums_kernel");
        if ((rc = pull<R>(p, st))) return rc;
        p->started = true;
    }
    DRONE_CUDA(cudaStreamSynchronize(st));
    const auto t1 = clock::now();
    if ((rc = exchange<R>(parts, tr, st))) return rc;
    if ((rc = tr.allreduce(parts, 0, sizeof(R) == 8, st))) return rc;
    for (size_t i = 0; i < parts.size(); ++i) {
        drone_pr *p = parts[i];
        if (p->n_local > 0) {
            pr_count_active_kernel<<<grid1d(p->n_local), 256, 0, st>>>(p->active, p->n_local, p->counters);
            DRONE_LAUNCH_CHECK("pr_count_active_kernel");
        }
    }
    std::vector<int> h(8 * parts.size());
    for (size_t i = 0; i < parts.size(); ++i)
        DRONE_CUDA(cudaMemcpyAsync(h.data() + 8 * i, parts[i]->counters, sizeof(int) * 8, cudaMemcpyDeviceToHost, st));
    DRONE_CUDA(cudaStreamSynchronize(st));
    const auto t2 = clock::now();
    for (size_t i = 0; i < parts.size(); ++i) {
        drone_pr_response &r = res[i];
        r.Mirror2MasterSendSize = h[8 * i + 0];
        r.Mirror2MasterRecvSize = h[8 * i + 1];
        r.Master2MirrorSendSize = h[8 * i + 2];
        r.Master2MirrorRecvSize = h[8 * i + 3];
        r.VisitedSize = h[8 * i + 4];
        r.LocalVertexSize = parts[i]->n_local;
        r.CalTime = std::chrono::duration<float>(t1 - t0).count();
        r.SendTime = std::chrono::duration<float>(t2 - t1).count();
    }
    return DRONE_OK;
}

template <typename R>
static int power_iterations(std::vector<drone_pr *> &parts, int iterations, double damping, Transport &tr,
                            cudaStream_t st) {
    int rc;
    for (drone_pr *p : parts) {
        const int n = p->n_local;
        DRONE_CUDA(cudaMemsetAsync(p->scalars, 0, sizeof(R) * 4, st));
        pr_init_kernel<R><<<grid1d(n, kReduceBlocks), 256, 0, st>>>(
            (R *)p->pr, (R *)p->acc, (R *)p->diff, (Pair<R> *)p->push, p->active, p->ubm, p->out_degree,
            p->mirror2worker, n, p->global_v, (R)1 / (R)p->global_v, (R *)p->block_sums, p->place);
        DRONE_LAUNCH_CHECK("pr_init_kernel");
        pr_set_scalar_kernel<R><<<1, 32, 0, st>>>((R *)p->scalars, 3, (R)1 / (R)p->global_v);
        DRONE_LAUNCH_CHECK("pr_set_scalar_kernel");
        p->started = false;
    }
    for (drone_pr *p : parts) {
        pr_power_prepare_kernel<R><<<grid1d(p->n_local, kReduceBlocks), 256, 0, st>>>(
            (const R *)p->pr, (Pair<R> *)p->push, p->out_degree, p->mirror2worker, p->n_local, (R *)p->block_sums,
            p->place);
        DRONE_LAUNCH_CHECK("pr_power_prepare_kernel");
    }
    for (int it = 0; it < iterations; ++it) {
        for (drone_pr *p : parts) {
            const int grid = grid1d(p->n_local, kReduceBlocks);
            DRONE_CUDA(cudaMemsetAsync((char *)p->scalars + 2 * sizeof(R), 0, sizeof(R), st));
            pr_fold_block_sums_kernel<R><<<1, 32, 0, st>>>((const R *)p->block_sums, grid, (R *)p->scalars, 2);
            DRONE_LAUNCH_CHECK("pr_fold_block_sums_kernel");
            if (p->xplan->rank == 0 && p->n_isolated > 0) {
                pr_power_isolated_kernel<R><<<1, 32, 0, st>>>((R *)p->scalars, p->n_isolated);
                DRONE_LAUNCH_CHECK("pr_power_isolated_kernel");
            }
            if ((rc = pull<R>(p, st))) return rc;
        }
        if ((rc = exchange<R>(parts, tr, st))) return rc;
        if ((rc = tr.allreduce(parts, 2, sizeof(R) == 8, st))) return rc;
        for (drone_pr *p : parts) {
            // new values, and what they publish for the next iteration, in one pass
            pr_power_apply_kernel<R><<<grid1d(p->n_local, kReduceBlocks), 256, 0, st>>>(
                (R *)p->pr, (const R *)p->diff, (Pair<R> *)p->push, p->out_degree, p->mirror2worker, p->n_local,
                p->global_v, (R)damping, (R *)p->scalars, (R *)p->block_sums, p->place);
            DRONE_LAUNCH_CHECK("pr_power_apply_kernel");
        }
    }
    return DRONE_OK;
}

static int prepare_parts(std::vector<drone_pr *> &parts) {
    for (drone_pr *p : parts) {
        if (!p) return set_error(DRONE_E_INVALID, "PageRank handle is NULL");
        const int rc = xplan_ensure_device(p->xplan);
        if (rc) return rc;
    }
    return DRONE_OK;
}

}  // namespace drone

using namespace drone;

extern "C" {

int drone_pr_destroy(drone_pr *p);

int drone_pr_create(drone_pr **out, int n_local, int global_v, int nnz, const int *d_index, const int *d_dst,
                    const int *d_out_degree, const int *d_mirror2worker, drone_xplan *xplan, drone_comm *comm,
                    int use_double, double eps) {
    DRONE_REQUIRE(out != nullptr, "drone_pr_create: out is NULL");
    *out = nullptr;
    DRONE_REQUIRE(n_local >= 0 && global_v > 0 && nnz >= 0, "drone_pr_create: bad sizes");
    DRONE_REQUIRE(xplan != nullptr, "drone_pr_create: exchange plan is NULL");
    DRONE_REQUIRE(xplan->n_local == n_local, "drone_pr_create: exchange plan has %d rows, graph has %d", xplan->n_local,
                  n_local);
    DRONE_REQUIRE(xplan->nranks == 1 || comm == nullptr || (comm->nranks == xplan->nranks && comm->rank == xplan->rank),
                  "drone_pr_create: communicator and exchange plan disagree on rank");
    DRONE_REQUIRE(n_local == 0 || (d_index && d_out_degree && d_mirror2worker), "drone_pr_create: NULL device array");
    DRONE_REQUIRE(eps >= 0, "drone_pr_create: eps=%g is negative", eps);
    drone_pr *p = new (std::nothrow) drone_pr();
    if (!p) return set_error(DRONE_E_INVALID, "drone_pr_create: out of host memory");
    p->n_local = n_local;
    p->global_v = global_v;
    p->nnz = nnz;
    p->dbl = use_double != 0;
    p->eps = eps;
    p->xplan = xplan;
    p->comm = comm;
    cudaGetDevice(&p->device);
    const size_t rs = p->dbl ? 8 : 4;
    const size_t n1 = (size_t)(n_local > 0 ? n_local : 1);
    int rc = DRONE_OK;
    do {
        // transposed graph and the split of long rows: reuse the aggregation plan (coefficients unused)
        float *ones = nullptr;
        if (cudaMalloc(&ones, sizeof(float) * (size_t)(nnz > 0 ? nnz : 1)) != cudaSuccess) { rc = set_error(DRONE_E_CUDA, "drone_pr_create: out of device memory"); break; }
        cudaMemset(ones, 0, sizeof(float) * (size_t)(nnz > 0 ? nnz : 1));
        rc = plan_create_untagged(&p->plan, n_local, nnz, d_index, d_dst, ones, nullptr, nullptr, DRONE_PLAN_AT, nullptr);
        cudaFree(ones);
        if (rc) break;
        {
            const char *v = getenv("DRONE_PR_ORDER_MIN_ROWS");
            const long long min_rows = (v && *v) ? atoll(v) : (1LL << 22);
            if (min_rows > 0 && n_local >= min_rows && nnz > 0) {
                rc = plan_order_columns_by_frequency(p->plan, DRONE_OP_AT, d_index, &p->place, nullptr);
                if (rc) break;
            }
        }
        cudaError_t e = cudaSuccess;
        auto alloc = [&](void **ptr, size_t bytes) { if (e == cudaSuccess) e = cudaMalloc(ptr, bytes > 0 ? bytes : 16); };
        alloc((void **)&p->out_degree, sizeof(int) * n1);
        alloc((void **)&p->mirror2worker, sizeof(int) * n1);
        alloc(&p->pr, rs * n1);
        alloc(&p->acc, rs * n1);
        alloc(&p->diff, rs * n1);
        alloc(&p->push, 2 * rs * n1);
        alloc((void **)&p->active, sizeof(int) * n1);
        alloc((void **)&p->ubm, sizeof(int) * n1);
        alloc(&p->scalars, 8 * 4);
        alloc(&p->block_sums, 8 * kReduceBlocks);
        alloc(&p->partials, 2 * rs * (size_t)p->plan->side[DRONE_OP_AT].n_partials);
        const size_t nb = std::max(xplan->up_rows.size(), xplan->down_rows.size());
        alloc(&p->send, 2 * rs * nb);
        alloc(&p->recv, 2 * rs * nb);
        alloc((void **)&p->counters, sizeof(int) * 8);
        if (e != cudaSuccess) { rc = set_error(DRONE_E_CUDA, "drone_pr_create: cudaMalloc failed: %s", cudaGetErrorString(e)); break; }
        if (n_local > 0) {
            e = cudaMemcpy(p->out_degree, d_out_degree, sizeof(int) * (size_t)n_local, cudaMemcpyDeviceToDevice);
            if (e == cudaSuccess) e = cudaMemcpy(p->mirror2worker, d_mirror2worker, sizeof(int) * (size_t)n_local, cudaMemcpyDeviceToDevice);
            if (e != cudaSuccess) { rc = set_error(DRONE_E_CUDA, "drone_pr_create: copy failed: %s", cudaGetErrorString(e)); break; }
        }
    } while (0);
    if (rc) {
        drone_pr_destroy(p);
        return rc;
    }
    *out = p;
    return DRONE_OK;
}

int drone_pr_destroy(drone_pr *p) {
    if (!p) return DRONE_OK;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(p->device);
    drone_plan_destroy(p->plan);
    cudaFree(p->place);
    cudaFree(p->out_degree); cudaFree(p->mirror2worker); cudaFree(p->pr); cudaFree(p->acc); cudaFree(p->diff);
    cudaFree(p->push); cudaFree(p->active); cudaFree(p->ubm); cudaFree(p->scalars); cudaFree(p->block_sums);
    cudaFree(p->partials); cudaFree(p->send); cudaFree(p->recv); cudaFree(p->counters);
    if (prev >= 0) cudaSetDevice(prev);
    delete p;
    return DRONE_OK;
}

static int run_delta(std::vector<drone_pr *> &parts, bool peval, Transport &tr, drone_pr_response *res, void *stream) {
    int rc = prepare_parts(parts);
    if (rc) return rc;
    int dev = -1;
    DRONE_CUDA(cudaGetDevice(&dev));
    if (dev != parts[0]->device) DRONE_CUDA(cudaSetDevice(parts[0]->device));
    rc = parts[0]->dbl ? delta_step<double>(parts, peval, tr, res, (cudaStream_t)stream)
                       : delta_step<float>(parts, peval, tr, res, (cudaStream_t)stream);
    if (dev != parts[0]->device) cudaSetDevice(dev);
    return rc;
}

int drone_pr_peval(drone_pr *p, drone_pr_response *res, void *stream) {
    DRONE_REQUIRE(p && res, "drone_pr_peval: NULL argument");
    DRONE_REQUIRE(p->xplan->nranks == 1 || p->comm, "drone_pr_peval: %d ranks but no communicator", p->xplan->nranks);
    std::vector<drone_pr *> parts{p};
    if (use_peer_transport(p)) {
        PeerTransport tr;
        return run_delta(parts, true, tr, res, stream);
    }
    NcclTransport tr;
    return run_delta(parts, true, tr, res, stream);
}

int drone_pr_inceval(drone_pr *p, drone_pr_response *res, void *stream) {
    DRONE_REQUIRE(p && res, "drone_pr_inceval: NULL argument");
    std::vector<drone_pr *> parts{p};
    if (use_peer_transport(p)) {
        PeerTransport tr;
        return run_delta(parts, false, tr, res, stream);
    }
    NcclTransport tr;
    return run_delta(parts, false, tr, res, stream);
}

int drone_pr_step_local(int n_parts, drone_pr **prs, int is_peval, drone_pr_response *res, void *stream) {
    DRONE_REQUIRE(n_parts >= 1 && n_parts <= 64 && prs && res, "drone_pr_step_local: bad arguments");
    std::vector<drone_pr *> parts(prs, prs + n_parts);
    for (int i = 0; i < n_parts; ++i)
        DRONE_REQUIRE(parts[i] && parts[i]->xplan->nranks == n_parts && parts[i]->xplan->rank == i &&
                          parts[i]->dbl == parts[0]->dbl,
                      "drone_pr_step_local: handle %d is not part %d of %d", i, i, n_parts);
    LocalTransport tr;
    return run_delta(parts, is_peval != 0, tr, res, stream);
}

static int run_power(std::vector<drone_pr *> &parts, int iterations, double damping, Transport &tr, void *stream) {
    int rc = prepare_parts(parts);
    if (rc) return rc;
    int dev = -1;
    DRONE_CUDA(cudaGetDevice(&dev));
    if (dev != parts[0]->device) DRONE_CUDA(cudaSetDevice(parts[0]->device));
    rc = parts[0]->dbl ? power_iterations<double>(parts, iterations, damping, tr, (cudaStream_t)stream)
                       : power_iterations<float>(parts, iterations, damping, tr, (cudaStream_t)stream);
    if (dev != parts[0]->device) cudaSetDevice(dev);
    return rc;
}

int drone_pr_power_iterate(drone_pr *p, int iterations, double damping, void *stream) {
    DRONE_REQUIRE(p != nullptr, "drone_pr_power_iterate: handle is NULL");
    DRONE_REQUIRE(iterations >= 0 && damping >= 0 && damping <= 1, "drone_pr_power_iterate: iterations=%d damping=%g",
                  iterations, damping);
    DRONE_REQUIRE(p->xplan->nranks == 1 || p->comm, "drone_pr_power_iterate: %d ranks but no communicator",
                  p->xplan->nranks);
    std::vector<drone_pr *> parts{p};
    if (use_peer_transport(p)) {
        PeerTransport tr;
        return run_power(parts, iterations, damping, tr, stream);
    }
    NcclTransport tr;
    return run_power(parts, iterations, damping, tr, stream);
}

int drone_pr_power_iterate_local(int n_parts, drone_pr **prs, int iterations, double damping, void *stream) {
    DRONE_REQUIRE(n_parts >= 1 && n_parts <= 64 && prs, "drone_pr_power_iterate_local: bad arguments");
    DRONE_REQUIRE(iterations >= 0 && damping >= 0 && damping <= 1, "drone_pr_power_iterate_local: iterations=%d damping=%g",
                  iterations, damping);
    std::vector<drone_pr *> parts(prs, prs + n_parts);
    for (int i = 0; i < n_parts; ++i)
        DRONE_REQUIRE(parts[i] && parts[i]->xplan->nranks == n_parts && parts[i]->xplan->rank == i &&
                          parts[i]->dbl == parts[0]->dbl,
                      "drone_pr_power_iterate_local: handle %d is not part %d of %d", i, i, n_parts);
    LocalTransport tr;
    return run_power(parts, iterations, damping, tr, stream);
}

int drone_pr_set_isolated_count(drone_pr *p, long long n_isolated) {
    DRONE_REQUIRE(p != nullptr && n_isolated >= 0, "drone_pr_set_isolated_count: bad argument");
    p->n_isolated = n_isolated;
    return DRONE_OK;
}

int drone_pr_device_arrays(drone_pr *p, void **d_pr, void **d_acc, void **d_diff, int **d_active,
                           int **d_update_by_message) {
    DRONE_REQUIRE(p != nullptr, "drone_pr_device_arrays: handle is NULL");
    if (d_pr) *d_pr = p->pr;
    if (d_acc) *d_acc = p->acc;
    if (d_diff) *d_diff = p->diff;
    if (d_active) *d_active = p->active;
    if (d_update_by_message) *d_update_by_message = p->ubm;
    return DRONE_OK;
}

int drone_pr_values(drone_pr *p, void *h_out, void *stream) {
    DRONE_REQUIRE(p && (h_out || p->n_local == 0), "drone_pr_values: NULL argument");
    if (p->n_local == 0) return DRONE_OK;
    DRONE_CUDA(cudaMemcpyAsync(h_out, p->pr, (p->dbl ? 8 : 4) * (size_t)p->n_local, cudaMemcpyDeviceToHost,
                               (cudaStream_t)stream));
    DRONE_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return DRONE_OK;
}

}  // extern "C"
