// Minimum propagation over an EBV-partitioned graph: the "cc_cuda" and "sssp_cuda" jobs.
//
// Both jobs push a value along the local out-edges until nothing changes (labels: the value itself; distances: value +
// edge length), then exchange the boundary: mirror -> master minimum, master -> mirror minimum.  Restated from
// DRONE/src/cuda/algorithm/cc.cu and sssp.cu (PEval / IncEval and their helper kernels) with these changes:
//   * one state, one set of kernels for both jobs: distances are non-negative floats, whose bit patterns order like
//     unsigned integers, so both kinds are "atomicMin on a 32-bit word";
//   * a warp works on 32 vertices; rows above kSerialDegree edges are spread over the warp's lanes, and rows above
//     kHeavyDegree are cut into chunks that a second kernel hands to all warps of the grid (the reference walks
//     every row with one thread, which a hub row turns into one long serial loop);
//   * the exchange uses the static plan (rows in a fixed order, no ids on the wire, no allocation per superstep);
//     every boundary vertex travels as {value, flag} and only flagged entries count and are applied, which gives the
//     same values and the same Response sizes as the reference's lists of changed vertices;
//   * several relaxation steps are launched per look at the "anything changed" word.
// Labels start as GLOBAL vertex ids (the CPU job's choice, DRONE/src/algorithm/CC.go:73-79; cc_init writes the local
// index, cc.cu:14, which cannot be compared between workers).  A shorter distance always re-activates its vertex
// (sssp_exec asks for an improvement above 1e-6, sssp.cu:67; with the unit lengths build_graph stores both agree).
#include "exchange.cuh"

#include <chrono>
#include <new>
#include <vector>

#include "../../include/drone_b200.h"

namespace drone {
int xplan_ensure_device(drone_xplan *x);
}

struct drone_mp {
    int device = 0, kind = 0, n_local = 0, nnz = 0;
    const int *index = nullptr, *dst = nullptr, *l2g = nullptr;   // borrowed device arrays
    const float *len = nullptr;                                   // borrowed, NULL = 1.0
    drone_xplan *xplan = nullptr;                                 // borrowed
    drone_comm *comm = nullptr;                                   // borrowed, may be NULL for one part
    unsigned *value = nullptr;     // [n] label, or the bits of a non-negative float distance
    int *active = nullptr;         // [n] -1 idle, s = in the frontier of step s; > 0 after a run: lowered in that run
    int *ubm = nullptr;            // [n] lowered by a received message since the last sweep
    uint2 *send = nullptr, *recv = nullptr;   // [max(up, down)] {value, flag}
    int *counters = nullptr;       // [0..3] exchange sizes, [4] VisitedSize, [5] "a step lowered something",
                                   // [6] entries in `heavy`
    int2 *heavy = nullptr;         // [heavy_cap] {vertex, chunk}: this step's chunks of frontier rows above kHeavyDegree
    int heavy_cap = 0;
    bool started = false;
};

namespace drone {

constexpr int kSerialDegree = 8;     // rows up to this many edges are walked by their own lane
constexpr int kHeavyDegree = 4096;   // rows above this many edges are cut into chunks for the whole grid
constexpr int kHeavyChunk = 2048;    // edges per chunk
constexpr int kStepsPerLook = 4;     // relaxation steps launched between two reads of the changed word
constexpr unsigned kFarBits = 0x4CBEBC20u;   // 1e8f, the reference's "not reached" (sssp.cu:33)

static inline int grid_mp(long long n, int cap = 148 * 16) {
    long long g = (n + 255) / 256;
    if (g < 1) g = 1;
    if (g > cap) g = cap;
    return (int)g;
}

// PEval start.  Labels: every vertex is in the frontier of step 0 with its global id.  Distances: only the source.
__global__ void mp_init_kernel(int kind, unsigned *value, int *active, int *ubm, const int *__restrict__ l2g, int n,
                               int source_global, int *counters) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        ubm[i] = 0;
        if (kind == DRONE_MP_CC) {
            value[i] = (unsigned)l2g[i];
            active[i] = 0;
            counters[5] = 1;
        } else if (l2g[i] == source_global) {
            value[i] = 0u;      // 0.0f
            active[i] = 0;
            counters[5] = 1;
        } else {
            value[i] = kFarBits;
            active[i] = -1;
        }
    }
}

// IncEval start: vertices lowered by a message form the frontier of step 0 (cc_process_messages, cc.cu:385-398).
__global__ void mp_sweep_kernel(int *active, int *ubm, int n, int *counters) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        if (ubm[i] != 0) {
            active[i] = 0;
            ubm[i] = 0;
            counters[5] = 1;
        } else {
            active[i] = -1;
        }
    }
}

template <int KIND>
__device__ __forceinline__ void mp_relax_edge(unsigned now, int k, const int *__restrict__ dst, const float *__restrict__ len,
                                              unsigned *value, int *active, int step, int *counters) {
    const int w = dst[k];
    unsigned nv = now;
    if (KIND == DRONE_MP_SSSP) nv = __float_as_uint(__uint_as_float(now) + (len ? len[k] : 1.0f));
    if (nv < value[w]) {                       // cheap filter; the atomic decides
        const unsigned old = atomicMin(value + w, nv);
        if (old > nv) {
            active[w] = step + 1;
            counters[5] = 1;
        }
    }
}

// One step: every vertex in the frontier of `step` offers its value to its out-neighbours (cc_exec, cc.cu:21-46;
// sssp_exec, sssp.cu:41-74).
template <int KIND>
__global__ void __launch_bounds__(256)
mp_relax_kernel(const int *__restrict__ index, const int *__restrict__ dst, const float *__restrict__ len,
                unsigned *value, int *active, int n, int step, int *counters, int2 *heavy, int heavy_cap) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long base = warp0 * 32; base < n; base += n_warps * 32) {
        const long long v = base + lane;
        bool front = v < n && active[v] == step;
        int beg = 0, end = 0;
        unsigned now = 0;
        if (front) {
            beg = index[v];
            end = index[v + 1];
            now = value[v];
            if (end - beg <= kSerialDegree) {
                for (int k = beg; k < end; ++k) mp_relax_edge<KIND>(now, k, dst, len, value, active, step, counters);
                front = false;
            } else if (end - beg > kHeavyDegree) {
                const int n_chunks = (end - beg + kHeavyChunk - 1) / kHeavyChunk;
                const int at = atomicAdd(counters + 6, n_chunks);
                if (at + n_chunks <= heavy_cap) {          // always true: the capacity covers every row at once
                    for (int c = 0; c < n_chunks; ++c) heavy[at + c] = make_int2((int)v, c);
                    front = false;
                }
            }
        }
        unsigned todo = __ballot_sync(0xffffffffu, front);
        while (todo) {
            const int src = __ffs(todo) - 1;
            todo &= todo - 1;
            const int b = __shfl_sync(0xffffffffu, beg, src), e = __shfl_sync(0xffffffffu, end, src);
            const unsigned x = __shfl_sync(0xffffffffu, now, src);
            for (int k = b + lane; k < e; k += 32) mp_relax_edge<KIND>(x, k, dst, len, value, active, step, counters);
        }
    }
}

// The chunks queued by mp_relax_kernel in the same step, one warp per chunk.
template <int KIND>
__global__ void __launch_bounds__(256)
mp_relax_heavy_kernel(const int *__restrict__ index, const int *__restrict__ dst, const float *__restrict__ len,
                      unsigned *value, int *active, int step, int *counters, const int2 *heavy, int heavy_cap) {
    const int lane = threadIdx.x & 31;
    const int count = min(counters[6], heavy_cap);
    const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long i = warp0; i < count; i += n_warps) {
        const int2 item = heavy[i];
        const int b = index[item.x] + item.y * kHeavyChunk;
        const int e = min(b + kHeavyChunk, index[item.x + 1]);
        const unsigned x = value[item.x];
        for (int k = b + lane; k < e; k += 32) mp_relax_edge<KIND>(x, k, dst, len, value, active, step, counters);
    }
}

// Mirrors lowered in this run go up (cc_generate_sendBuff_mirror, cc.cu:82-106: active > 0).
__global__ void mp_pack_up_kernel(const int *__restrict__ up_rows, int n_up, const unsigned *value, const int *active,
                                  uint2 *send, int *counters) {
    int mine = 0;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_up; i += (long long)gridDim.x * blockDim.x) {
        const int r = up_rows[i];
        const unsigned flag = active[r] > 0 ? 1u : 0u;
        send[i] = make_uint2(value[r], flag);
        mine += (int)flag;
    }
    if (mine) atomicAdd(counters + 0, mine);
}

// A master takes the minimum of what its mirrors sent (cc_process_recvBuff, cc.cu:135-157).
__global__ void mp_apply_up_kernel(const int *__restrict__ m_rows, const int *__restrict__ m_off,
                                   const int *__restrict__ m_pos, int n_m, const uint2 *recv, unsigned *value, int *ubm,
                                   int *counters) {
    int got = 0;
    for (long long m = blockIdx.x * (long long)blockDim.x + threadIdx.x; m < n_m; m += (long long)gridDim.x * blockDim.x) {
        const int r = m_rows[m];
        unsigned best = value[r];
        bool lowered = false;
        for (int k = m_off[m]; k < m_off[m + 1]; ++k) {
            const uint2 e = recv[m_pos[k]];
            if (!e.y) continue;
            ++got;
            if (e.x < best) { best = e.x; lowered = true; }
        }
        if (lowered) { value[r] = best; ubm[r] = 1; }
    }
    if (got) atomicAdd(counters + 1, got);
}

// Masters lowered in this run or by a message go down, once per mirror (cc_generate_sendBuff_master, cc.cu:108-133).
__global__ void mp_pack_down_kernel(const int *__restrict__ down_rows, int n_down, const unsigned *value, const int *active,
                                    const int *ubm, uint2 *send, int *counters) {
    int mine = 0;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_down; i += (long long)gridDim.x * blockDim.x) {
        const int r = down_rows[i];
        const unsigned flag = (active[r] > 0 || ubm[r] != 0) ? 1u : 0u;
        send[i] = make_uint2(value[r], flag);
        mine += (int)flag;
    }
    if (mine) atomicAdd(counters + 2, mine);
}

__global__ void mp_apply_down_kernel(const int *__restrict__ up_rows, int n_up, const uint2 *recv, unsigned *value, int *ubm,
                                     int *counters) {
    int got = 0;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_up; i += (long long)gridDim.x * blockDim.x) {
        const uint2 e = recv[i];
        if (!e.y) continue;
        ++got;
        const int r = up_rows[i];
        if (e.x < value[r]) { value[r] = e.x; ubm[r] = 1; }
    }
    if (got) atomicAdd(counters + 3, got);
}

// VisitedSize as the reference counts it: entries of `active` that are not 0 (countActive, common.cu:6-16).
__global__ void mp_count_visited_kernel(const int *active, int n, int *counters) {
    int mine = 0;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        mine += active[i] != 0;
    if (mine) atomicAdd(counters + 4, mine);
}

// Moves the packed boundary entries of all parts: over NCCL (one part per process) or as device-to-device copies
// (all parts in this process).
static int mp_move(std::vector<drone_mp *> &parts, bool up, bool local, cudaStream_t st) {
    if (!local) {
        drone_mp *p = parts[0];
        const drone_xplan *x = p->xplan;
        if (x->nranks == 1) return DRONE_OK;
        const std::vector<int> &s_off = up ? x->up_off : x->down_off;
        const std::vector<int> &r_off = up ? x->down_off : x->up_off;
        DRONE_NCCL(ncclGroupStart());
        for (int q = 0; q < x->nranks; ++q) {
            if (q == x->rank) continue;
            const size_t ns = (size_t)(s_off[q + 1] - s_off[q]) * 2, nr = (size_t)(r_off[q + 1] - r_off[q]) * 2;
            if (ns) DRONE_NCCL(ncclSend(p->send + s_off[q], ns, ncclUint32, q, p->comm->comm, st));
            if (nr) DRONE_NCCL(ncclRecv(p->recv + r_off[q], nr, ncclUint32, q, p->comm->comm, st));
        }
        DRONE_NCCL(ncclGroupEnd());
        return DRONE_OK;
    }
    const int P = (int)parts.size();
    for (int p = 0; p < P; ++p)
        for (int q = 0; q < P; ++q) {
            if (p == q) continue;
            const std::vector<int> &s_off = up ? parts[p]->xplan->up_off : parts[p]->xplan->down_off;
            const std::vector<int> &r_off = up ? parts[q]->xplan->down_off : parts[q]->xplan->up_off;
            const size_t ns = (size_t)(s_off[q + 1] - s_off[q]), nr = (size_t)(r_off[p + 1] - r_off[p]);
            if (ns != nr)
                return set_error(DRONE_E_STATE, "exchange plans disagree between parts %d and %d (%zu vs %zu rows)", p, q, ns, nr);
            if (ns)
                DRONE_CUDA(cudaMemcpyAsync(parts[q]->recv + r_off[p], parts[p]->send + s_off[q], ns * sizeof(uint2),
                                           cudaMemcpyDeviceToDevice, st));
        }
    return DRONE_OK;
}

// Relaxation steps until a whole group of kStepsPerLook steps lowers nothing.
static int mp_local_run(drone_mp *p, cudaStream_t st) {
    const int n = p->n_local;
    if (n == 0) return DRONE_OK;
    int step = 0, changed = 0;
    DRONE_CUDA(cudaMemcpyAsync(&changed, p->counters + 5, sizeof(int), cudaMemcpyDeviceToHost, st));
    DRONE_CUDA(cudaStreamSynchronize(st));
    const int grid = grid_mp((long long)n, 148 * 8);
    while (changed) {
        DRONE_CUDA(cudaMemsetAsync(p->counters + 5, 0, sizeof(int), st));
        for (int i = 0; i < kStepsPerLook; ++i, ++step) {
            DRONE_CUDA(cudaMemsetAsync(p->counters + 6, 0, sizeof(int), st));
            if (p->kind == DRONE_MP_CC) {
                mp_relax_kernel<DRONE_MP_CC><<<grid, 256, 0, st>>>(p->index, p->dst, nullptr, p->value, p->active, n, step,
                                                                   p->counters, p->heavy, p->heavy_cap);
                DRONE_LAUNCH_CHECK("mp_relax_kernel");
                mp_relax_heavy_kernel<DRONE_MP_CC><<<grid, 256, 0, st>>>(p->index, p->dst, nullptr, p->value, p->active, step,
                                                                         p->counters, p->heavy, p->heavy_cap);
            } else {
                mp_relax_kernel<DRONE_MP_SSSP><<<grid, 256, 0, st>>>(p->index, p->dst, p->len, p->value, p->active, n, step,
                                                                     p->counters, p->heavy, p->heavy_cap);
                DRONE_LAUNCH_CHECK("mp_relax_kernel");
                mp_relax_heavy_kernel<DRONE_MP_SSSP><<<grid, 256, 0, st>>>(p->index, p->dst, p->len, p->value, p->active, step,
                                                                           p->counters, p->heavy, p->heavy_cap);
            }
            DRONE_LAUNCH_CHECK("mp_relax_heavy_kernel");
        }
        DRONE_CUDA(cudaMemcpyAsync(&changed, p->counters + 5, sizeof(int), cudaMemcpyDeviceToHost, st));
        DRONE_CUDA(cudaStreamSynchronize(st));
    }
    return DRONE_OK;
}

static int mp_exchange(std::vector<drone_mp *> &parts, bool local, cudaStream_t st) {
    int rc;
    for (drone_mp *p : parts) {
        const drone_xplan *x = p->xplan;
        const int n_up = (int)x->up_rows.size();
        if (n_up) {
            mp_pack_up_kernel<<<grid_mp(n_up), 256, 0, st>>>(x->d_up_rows, n_up, p->value, p->active, p->send, p->counters);
            DRONE_LAUNCH_CHECK("mp_pack_up_kernel");
        }
    }
    if ((rc = mp_move(parts, true, local, st))) return rc;
    for (drone_mp *p : parts) {
        const drone_xplan *x = p->xplan;
        const int n_m = (int)x->m_rows.size(), n_down = (int)x->down_rows.size();
        if (n_m) {
            mp_apply_up_kernel<<<grid_mp(n_m), 256, 0, st>>>(x->d_m_rows, x->d_m_off, x->d_m_pos, n_m, p->recv, p->value, p->ubm,
                                                            p->counters);
            DRONE_LAUNCH_CHECK("mp_apply_up_kernel");
        }
        if (n_down) {
            mp_pack_down_kernel<<<grid_mp(n_down), 256, 0, st>>>(x->d_down_rows, n_down, p->value, p->active, p->ubm, p->send,
                                                                p->counters);
            DRONE_LAUNCH_CHECK("mp_pack_down_kernel");
        }
    }
    if ((rc = mp_move(parts, false, local, st))) return rc;
    for (drone_mp *p : parts) {
        const drone_xplan *x = p->xplan;
        const int n_up = (int)x->up_rows.size();
        if (n_up) {
            mp_apply_down_kernel<<<grid_mp(n_up), 256, 0, st>>>(x->d_up_rows, n_up, p->recv, p->value, p->ubm, p->counters);
            DRONE_LAUNCH_CHECK("mp_apply_down_kernel");
        }
    }
    return DRONE_OK;
}

// One superstep of all given parts (one part over NCCL, or all parts of a partition held in this process).
static int mp_step(std::vector<drone_mp *> &parts, bool peval, int source_global, bool local, drone_pr_response *res,
                   cudaStream_t st) {
    using clock = std::chrono::steady_clock;
    const auto t0 = clock::now();
    int rc;
    for (drone_mp *p : parts) {
        if (!peval && !p->started) return set_error(DRONE_E_STATE, "IncEVal called before PEVal");
        DRONE_CUDA(cudaMemsetAsync(p->counters, 0, sizeof(int) * 8, st));
        const int n = p->n_local;
        if (n > 0) {
            if (peval) {
                mp_init_kernel<<<grid_mp(n), 256, 0, st>>>(p->kind, p->value, p->active, p->ubm, p->l2g, n, source_global,
                                                          p->counters);
                DRONE_LAUNCH_CHECK("mp_init_kernel");
            } else {
                mp_sweep_kernel<<<grid_mp(n), 256, 0, st>>>(p->active, p->ubm, n, p->counters);
                DRONE_LAUNCH_CHECK("mp_sweep_kernel");
            }
        }
        if ((rc = mp_local_run(p, st))) return rc;
        p->started = true;
    }
    DRONE_CUDA(cudaStreamSynchronize(st));
    const auto t1 = clock::now();
    if ((rc = mp_exchange(parts, local, st))) return rc;
    for (drone_mp *p : parts)
        if (p->n_local > 0) {
            mp_count_visited_kernel<<<grid_mp(p->n_local), 256, 0, st>>>(p->active, p->n_local, p->counters);
            DRONE_LAUNCH_CHECK("mp_count_visited_kernel");
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

static int mp_prepare(std::vector<drone_mp *> &parts) {
    for (drone_mp *p : parts) {
        DRONE_REQUIRE(p != nullptr, "NULL job handle");
        const int rc = xplan_ensure_device(p->xplan);
        if (rc) return rc;
    }
    return DRONE_OK;
}

}  // namespace drone

using namespace drone;

extern "C" {

int drone_mp_destroy(drone_mp *p);

int drone_mp_create(drone_mp **out, int kind, int n_local, int nnz, const int *d_index, const int *d_dst,
                    const float *d_edge_len, const int *d_local2global, drone_xplan *xplan, drone_comm *comm) {
    DRONE_REQUIRE(out != nullptr, "drone_mp_create: out is NULL");
    *out = nullptr;
    DRONE_REQUIRE(kind == DRONE_MP_CC || kind == DRONE_MP_SSSP, "drone_mp_create: kind=%d", kind);
    DRONE_REQUIRE(n_local >= 0 && nnz >= 0, "drone_mp_create: negative size");
    DRONE_REQUIRE(xplan != nullptr, "drone_mp_create: exchange plan is NULL");
    DRONE_REQUIRE(xplan->n_local == n_local, "drone_mp_create: the exchange plan was made for %d rows, the graph has %d",
                  xplan->n_local, n_local);
    DRONE_REQUIRE(xplan->nranks == 1 || comm == nullptr || (comm->nranks == xplan->nranks && comm->rank == xplan->rank),
                  "drone_mp_create: communicator and exchange plan disagree on rank / size");
    DRONE_REQUIRE(n_local == 0 || (d_index && d_local2global), "drone_mp_create: NULL graph array");
    DRONE_REQUIRE(nnz == 0 || d_dst != nullptr, "drone_mp_create: d_dst is NULL with nnz=%d", nnz);
    if (n_local > 0) {   // the relax kernels index the value arrays with d_dst: reject what would run out of bounds
        const int bad = validate_csr("drone_mp_create", d_index, d_dst, n_local, n_local, nnz, nullptr);
        if (bad) return bad;
    }
    drone_mp *p = new (std::nothrow) drone_mp();
    if (!p) return set_error(DRONE_E_INVALID, "drone_mp_create: out of host memory");
    p->kind = kind;
    p->n_local = n_local;
    p->nnz = nnz;
    p->index = d_index;
    p->dst = d_dst;
    p->len = d_edge_len;
    p->l2g = d_local2global;
    p->xplan = xplan;
    p->comm = comm;
    cudaError_t err = cudaGetDevice(&p->device);
    const size_t n1 = (size_t)(n_local > 0 ? n_local : 1);
    const size_t nb = std::max<size_t>(std::max(xplan->up_rows.size(), xplan->down_rows.size()), 1);
    if (err == cudaSuccess) err = cudaMalloc(&p->value, sizeof(unsigned) * n1);
    if (err == cudaSuccess) err = cudaMalloc(&p->active, sizeof(int) * n1);
    if (err == cudaSuccess) err = cudaMalloc(&p->ubm, sizeof(int) * n1);
    if (err == cudaSuccess) err = cudaMalloc(&p->send, sizeof(uint2) * nb);
    if (err == cudaSuccess) err = cudaMalloc(&p->recv, sizeof(uint2) * nb);
    if (err == cudaSuccess) err = cudaMalloc(&p->counters, sizeof(int) * 8);
    // every row above kHeavyDegree in the frontier at once: at most nnz / kHeavyChunk full chunks plus one partial
    // chunk per such row, of which there are fewer than nnz / kHeavyDegree
    p->heavy_cap = nnz / kHeavyChunk + nnz / kHeavyDegree + 16;
    if (err == cudaSuccess) err = cudaMalloc(&p->heavy, sizeof(int2) * (size_t)p->heavy_cap);
    if (err != cudaSuccess) {
        drone_mp_destroy(p);
        return set_error(DRONE_E_CUDA, "drone_mp_create: %s", cudaGetErrorString(err));
    }
    *out = p;
    return DRONE_OK;
}

int drone_mp_destroy(drone_mp *p) {
    if (!p) return DRONE_OK;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(p->device);
    cudaFree(p->value); cudaFree(p->active); cudaFree(p->ubm); cudaFree(p->send); cudaFree(p->recv); cudaFree(p->counters);
    cudaFree(p->heavy);
    if (prev >= 0) cudaSetDevice(prev);
    delete p;
    return DRONE_OK;
}

static int mp_run(std::vector<drone_mp *> &parts, bool peval, int source_global, bool local, drone_pr_response *res,
                  void *stream) {
    DRONE_REQUIRE(res != nullptr, "Response pointer is NULL");
    int prev = -1;
    DRONE_CUDA(cudaGetDevice(&prev));
    const int dev = parts[0]->device;
    if (prev != dev) DRONE_CUDA(cudaSetDevice(dev));     // calls may arrive on any host thread
    int rc = mp_prepare(parts);
    if (rc == DRONE_OK) rc = mp_step(parts, peval, source_global, local, res, (cudaStream_t)stream);
    if (prev != dev) cudaSetDevice(prev);
    return rc;
}

int drone_mp_peval(drone_mp *p, int source_global_id, drone_pr_response *res, void *stream) {
    DRONE_REQUIRE(p != nullptr, "drone_mp_peval: NULL job");
    DRONE_REQUIRE(p->xplan->nranks == 1 || p->comm != nullptr, "drone_mp_peval: %d ranks but no communicator", p->xplan->nranks);
    std::vector<drone_mp *> parts{p};
    return mp_run(parts, true, source_global_id, false, res, stream);
}

int drone_mp_inceval(drone_mp *p, drone_pr_response *res, void *stream) {
    DRONE_REQUIRE(p != nullptr, "drone_mp_inceval: NULL job");
    DRONE_REQUIRE(p->xplan->nranks == 1 || p->comm != nullptr, "drone_mp_inceval: %d ranks but no communicator", p->xplan->nranks);
    std::vector<drone_mp *> parts{p};
    return mp_run(parts, false, -1, false, res, stream);
}

int drone_mp_step_local(int n_parts, drone_mp **jobs, int is_peval, int source_global_id, drone_pr_response *res,
                        void *stream) {
    DRONE_REQUIRE(n_parts >= 1 && jobs != nullptr, "drone_mp_step_local: no parts");
    std::vector<drone_mp *> parts(jobs, jobs + n_parts);
    for (int i = 0; i < n_parts; ++i) {
        DRONE_REQUIRE(parts[i] != nullptr, "drone_mp_step_local: part %d is NULL", i);
        DRONE_REQUIRE(parts[i]->xplan->nranks == n_parts && parts[i]->xplan->rank == i,
                      "drone_mp_step_local: part %d carries the plan of rank %d of %d", i, parts[i]->xplan->rank,
                      parts[i]->xplan->nranks);
        DRONE_REQUIRE(parts[i]->kind == parts[0]->kind && parts[i]->device == parts[0]->device,
                      "drone_mp_step_local: parts differ in kind or device");
    }
    return mp_run(parts, is_peval != 0, source_global_id, true, res, stream);
}

int drone_mp_device_arrays(drone_mp *p, void **d_value, int **d_active, int **d_update_by_message) {
    DRONE_REQUIRE(p != nullptr, "drone_mp_device_arrays: NULL job");
    if (d_value) *d_value = p->value;
    if (d_active) *d_active = p->active;
    if (d_update_by_message) *d_update_by_message = p->ubm;
    return DRONE_OK;
}

int drone_mp_values(drone_mp *p, void *h_out, void *stream) {
    DRONE_REQUIRE(p != nullptr && h_out != nullptr, "drone_mp_values: NULL argument");
    if (p->n_local == 0) return DRONE_OK;
    int prev = -1;
    DRONE_CUDA(cudaGetDevice(&prev));
    if (prev != p->device) DRONE_CUDA(cudaSetDevice(p->device));
    DRONE_CUDA(cudaMemcpyAsync(h_out, p->value, sizeof(unsigned) * (size_t)p->n_local, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    DRONE_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (prev != p->device) cudaSetDevice(prev);
    return DRONE_OK;
}

}  // extern "C"
