// Mirror/master exchange over peer memory (NVLink, one process per GPU).
//
// Same result as the NCCL transport of exchange.cu, with the packing, the transfer and the unpacking of each
// direction fused into one kernel per direction that stores rows straight into the receiver's memory:
//   push_up:        every mirror row -> the owner's up-receive area (position fixed by the static plan)
//   add_push_down:  wait for the up flags; master row += its mirrors' rows in ascending rank order; the total goes
//                   to every mirror's down-receive area
//   scatter:        wait for the down flags; mirror rows take the totals
// Ordering between GPUs uses one epoch word per (receiver, sender, direction): the sender's signal kernel runs after
// its stores in stream order, fences, and writes the call's epoch; the receiver polls its own words.  Every wait is
// bounded: when it runs out the kernel records an error code in pinned host memory, skips its work and returns, and
// the next call reports DRONE_E_STATE.  Nothing here uses TMA or cluster multicast; peers are reached with plain
// loads and stores.
//
// Why no host synchronisation is needed between calls: a rank stores into a peer's up-receive area in call k+1 only
// after its own scatter of call k, which waited for that peer's down flag of call k, which the peer wrote after it
// had consumed its up-receive area of call k.  Symmetrically a rank stores into a peer's down-receive area in call
// k+1 only after the peer's up flag of call k+1, which the peer wrote after its scatter of call k.
#include "exchange.cuh"

#include <algorithm>
#include <new>

namespace drone {

int xplan_ensure_device(drone_xplan *x);

static const long long kWaitLimit = 20000000;   // polls of ~100 ns each: about two seconds

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Threads 0..nranks-1 of the block poll flags[q] until it reaches `epoch` (for peers with need[q] != 0).
// Returns false for the whole block when a wait ran out or an earlier kernel of the sequence failed.
// `error` is a word in device memory (polled here); `host_error` is its pinned twin, written only on failure, so that
// the host can see the failure without a copy and the normal path never touches host memory.
__device__ bool wait_for_peers(const unsigned *flags, const int *need, int nranks, unsigned epoch, int *error,
                               int *host_error, int code) {
    __shared__ int failed;
    if (threadIdx.x == 0) failed = *(volatile int *)error != 0;
    __syncthreads();
    if (!failed && (int)threadIdx.x < nranks && need[threadIdx.x]) {
        long long polls = 0;
        while ((int)(ld_acquire_sys(flags + threadIdx.x) - epoch) < 0) {
            if (++polls > kWaitLimit) {
                atomicExch(error, code + (int)threadIdx.x);
                *(volatile int *)host_error = code + (int)threadIdx.x;
                failed = 1;
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    return failed == 0;
}

template <int VEC> struct PVec;
template <> struct PVec<4> { using type = float4; };
template <> struct PVec<1> { using type = float; };
__device__ __forceinline__ void vadd(float4 &a, const float4 &b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
__device__ __forceinline__ void vadd(float &a, const float &b) { a += b; }

// rows[up_rows[i], :] -> peer_up_recv[owner][dest_row[i], :]      (nvec = F / VEC vectors per row)
// The list is walked in the order `order` gives: the mirror rows are grouped by owner, and walking them as they
// lie would make every rank store to the same owner at the same time, whose NVLink ingress then limits all of them.
template <int VEC>
__global__ void p2p_push_up_kernel(const float *__restrict__ rows, long long ld, const int *__restrict__ up_rows,
                                   const int *__restrict__ up_peer, const int *__restrict__ up_dest_row,
                                   const int *__restrict__ order, int n_up, int nvec,
                                   float *const *__restrict__ peer_up_recv) {
    using V = typename PVec<VEC>::type;
    const long long total = (long long)n_up * nvec;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int k = (int)(i / nvec), j = (int)(i - (long long)k * nvec);
        const int r = order[k];
        V *dst = reinterpret_cast<V *>(peer_up_recv[up_peer[r]]) + (long long)up_dest_row[r] * nvec + j;
        *dst = *(reinterpret_cast<const V *>(rows + (long long)up_rows[r] * ld) + j);
    }
}

// After the stores of the preceding kernel: publish `epoch` in every peer that expects a flag from this rank.
__global__ void p2p_signal_kernel(unsigned *const *__restrict__ peer_flag, const int *__restrict__ send_to, int nranks,
                                  unsigned epoch) {
    __threadfence_system();
    if ((int)threadIdx.x < nranks && send_to[threadIdx.x]) st_release_sys(peer_flag[threadIdx.x], epoch);
}

// Master rows: add the mirrors' rows (fixed order), keep the total, and store it into every mirror's down-receive area.
template <int VEC>
__global__ void p2p_add_push_down_kernel(float *__restrict__ rows, long long ld, const int *__restrict__ m_rows,
                                         const int *__restrict__ m_off, const int *__restrict__ m_pos, int n_masters,
                                         int nvec, const float *up_recv, const int *__restrict__ down_peer,
                                         const int *__restrict__ down_dest_row, float *const *__restrict__ peer_down_recv,
                                         const unsigned *flags_up, const int *__restrict__ need_up, int nranks,
                                         unsigned epoch, int *error, int *host_error) {
    using V = typename PVec<VEC>::type;
    if (!wait_for_peers(flags_up, need_up, nranks, epoch, error, host_error, 100)) return;
    const V *recv = reinterpret_cast<const V *>(up_recv);
    const long long total = (long long)n_masters * nvec;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int m = (int)(i / nvec), j = (int)(i - (long long)m * nvec);
        V *mine = reinterpret_cast<V *>(rows + (long long)m_rows[m] * ld) + j;
        V acc = *mine;
        const int k0 = m_off[m], k1 = m_off[m + 1];
        for (int k = k0; k < k1; ++k) vadd(acc, __ldcv(recv + (long long)m_pos[k] * nvec + j));
        *mine = acc;
        for (int k = k0; k < k1; ++k) {
            const int p = m_pos[k];
            *(reinterpret_cast<V *>(peer_down_recv[down_peer[p]]) + (long long)down_dest_row[p] * nvec + j) = acc;
        }
    }
}

// Mirror rows take the totals their masters stored.
template <int VEC>
__global__ void p2p_scatter_kernel(float *__restrict__ rows, long long ld, const int *__restrict__ up_rows, int n_up,
                                   int nvec, const float *down_recv, const unsigned *flags_down,
                                   const int *__restrict__ need_down, int nranks, unsigned epoch, int *error,
                                   int *host_error) {
    using V = typename PVec<VEC>::type;
    if (!wait_for_peers(flags_down, need_down, nranks, epoch, error, host_error, 200)) return;
    const V *recv = reinterpret_cast<const V *>(down_recv);
    const long long total = (long long)n_up * nvec;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / nvec), j = (int)(i - (long long)r * nvec);
        *(reinterpret_cast<V *>(rows + (long long)up_rows[r] * ld) + j) = __ldcv(recv + i);
    }
}

static inline int p2p_grid(long long n) {
    long long g = (n + 255) / 256;
    if (g < 1) g = 1;
    if (g > 148 * 8) g = 148 * 8;
    return (int)g;
}

}  // namespace drone

using namespace drone;

namespace {

const size_t kFlagBytes = 1024;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

template <typename T>
int upload_vec(T **dst, const std::vector<T> &src) {
    DRONE_CUDA(cudaMalloc(dst, sizeof(T) * (src.size() > 0 ? src.size() : 1)));
    if (!src.empty()) DRONE_CUDA(cudaMemcpy(*dst, src.data(), sizeof(T) * src.size(), cudaMemcpyHostToDevice));
    return DRONE_OK;
}

void p2p_free(drone_p2p *p) {
    if (!p) return;
    for (char *s : p->peer_segment)
        if (s) cudaIpcCloseMemHandle(s);
    cudaFree(p->segment);
    cudaFree(p->d_peer_up_recv); cudaFree(p->d_peer_down_recv); cudaFree(p->d_peer_flag_up); cudaFree(p->d_peer_flag_down);
    cudaFree(p->d_up_peer); cudaFree(p->d_up_dest_row); cudaFree(p->d_up_order); cudaFree(p->d_down_peer); cudaFree(p->d_down_dest_row);
    cudaFree(p->d_need_up); cudaFree(p->d_need_down);
    if (p->h_error) cudaFreeHost(p->h_error);
    cudaFree(p->d_error);
    delete p;
}

}  // namespace

namespace drone {
void xplan_p2p_release(drone_xplan *x) {
    if (x && x->p2p) {
        p2p_free(x->p2p);
        x->p2p = nullptr;
    }
}
}  // namespace drone

extern "C" {

int drone_xplan_enable_p2p(drone_xplan *x, drone_comm *c, void *stream) {
    DRONE_REQUIRE(x && c, "drone_xplan_enable_p2p: NULL plan or communicator");
    DRONE_REQUIRE(c->nranks == x->nranks && c->rank == x->rank, "drone_xplan_enable_p2p: plan is rank %d/%d, comm %d/%d",
                  x->rank, x->nranks, c->rank, c->nranks);
    DRONE_REQUIRE(x->nranks <= 64, "drone_xplan_enable_p2p: at most 64 ranks");
    if (x->p2p || x->nranks == 1) return DRONE_OK;
    int rc = xplan_ensure_device(x);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const int P = x->nranks, me = x->rank;
    const size_t n_up = x->up_rows.size(), n_down = x->down_rows.size();
    drone_p2p *p = new (std::nothrow) drone_p2p();
    if (!p) return set_error(DRONE_E_INVALID, "drone_xplan_enable_p2p: out of host memory");
    x->p2p = p;   // released by drone_xplan_destroy, also after a failure below
    p->peer_segment.assign(P, nullptr);

    const size_t up_bytes = align_up(n_down * (size_t)x->max_features * 4, 256);
    const size_t down_bytes = align_up(n_up * (size_t)x->max_features * 4, 256);
    p->segment_bytes = kFlagBytes + up_bytes + down_bytes;
    DRONE_CUDA(cudaMalloc(&p->segment, p->segment_bytes));
    DRONE_CUDA(cudaMemsetAsync(p->segment, 0, p->segment_bytes, st));
    DRONE_CUDA(cudaHostAlloc(&p->h_error, sizeof(int), cudaHostAllocMapped));
    *p->h_error = 0;
    DRONE_CUDA(cudaHostGetDevicePointer(&p->d_host_error, p->h_error, 0));
    DRONE_CUDA(cudaMalloc(&p->d_error, sizeof(int)));
    DRONE_CUDA(cudaMemsetAsync(p->d_error, 0, sizeof(int), st));

    // what every rank tells the others: IPC handle, sizes, its two offset tables
    const size_t ints_per_rank = 4 + 2 * (size_t)(P + 1);
    const size_t rec_bytes = align_up(sizeof(cudaIpcMemHandle_t) + ints_per_rank * 4, 16);
    std::vector<char> mine(rec_bytes, 0), all(rec_bytes * P, 0);
    cudaIpcMemHandle_t handle;
    DRONE_CUDA(cudaIpcGetMemHandle(&handle, p->segment));
    memcpy(mine.data(), &handle, sizeof(handle));
    int *ints = reinterpret_cast<int *>(mine.data() + sizeof(handle));
    ints[0] = (int)n_down;
    ints[1] = (int)n_up;
    ints[2] = x->max_features;
    ints[3] = 0;
    for (int q = 0; q <= P; ++q) {
        ints[4 + q] = x->down_off[q];
        ints[4 + (P + 1) + q] = x->up_off[q];
    }
    char *d_mine = nullptr, *d_all = nullptr;
    DRONE_CUDA(cudaMalloc(&d_mine, rec_bytes));
    DRONE_CUDA(cudaMalloc(&d_all, rec_bytes * P));
    DRONE_CUDA(cudaMemcpyAsync(d_mine, mine.data(), rec_bytes, cudaMemcpyHostToDevice, st));
    DRONE_NCCL(ncclAllGather(d_mine, d_all, rec_bytes, ncclChar, c->comm, st));
    DRONE_CUDA(cudaMemcpyAsync(all.data(), d_all, rec_bytes * P, cudaMemcpyDeviceToHost, st));
    DRONE_CUDA(cudaStreamSynchronize(st));
    cudaFree(d_mine);
    cudaFree(d_all);

    std::vector<float *> up_base(P, nullptr), down_base(P, nullptr);
    std::vector<unsigned *> flag_up(P, nullptr), flag_down(P, nullptr);
    std::vector<int> need_up(P, 0), need_down(P, 0);
    std::vector<int> up_peer(n_up), up_dest(n_up), down_peer(n_down), down_dest(n_down);
    for (int q = 0; q < P; ++q) {
        if (q == me) continue;
        const int up_cnt = x->up_off[q + 1] - x->up_off[q], down_cnt = x->down_off[q + 1] - x->down_off[q];
        need_up[q] = down_cnt > 0;     // q holds mirrors of my masters: it sends up to me
        need_down[q] = up_cnt > 0;     // q owns masters of my mirrors: it sends down to me
        if (!up_cnt && !down_cnt) continue;
        const char *rec = all.data() + rec_bytes * q;
        const int *qi = reinterpret_cast<const int *>(rec + sizeof(cudaIpcMemHandle_t));
        const int q_n_down = qi[0], q_maxf = qi[2];
        const int *q_down_off = qi + 4, *q_up_off = qi + 4 + (P + 1);
        if (q_maxf != x->max_features)
            return set_error(DRONE_E_INVALID, "drone_xplan_enable_p2p: rank %d was planned for %d features, this rank for %d", q,
                             q_maxf, x->max_features);
        if (q_down_off[me + 1] - q_down_off[me] != up_cnt || q_up_off[me + 1] - q_up_off[me] != down_cnt)
            return set_error(DRONE_E_STATE, "drone_xplan_enable_p2p: plans of rank %d and %d disagree on their row counts", me, q);
        cudaIpcMemHandle_t qh;
        memcpy(&qh, rec, sizeof(qh));
        void *mapped = nullptr;
        DRONE_CUDA(cudaIpcOpenMemHandle(&mapped, qh, cudaIpcMemLazyEnablePeerAccess));
        p->peer_segment[q] = (char *)mapped;
        up_base[q] = reinterpret_cast<float *>(p->peer_segment[q] + kFlagBytes);
        down_base[q] = reinterpret_cast<float *>(p->peer_segment[q] + kFlagBytes +
                                                 align_up((size_t)q_n_down * (size_t)x->max_features * 4, 256));
        flag_up[q] = reinterpret_cast<unsigned *>(p->peer_segment[q]) + me;
        flag_down[q] = reinterpret_cast<unsigned *>(p->peer_segment[q]) + P + me;
        for (int i = x->up_off[q]; i < x->up_off[q + 1]; ++i) {
            up_peer[i] = q;
            up_dest[i] = q_down_off[me] + (i - x->up_off[q]);
        }
        for (int i = x->down_off[q]; i < x->down_off[q + 1]; ++i) {
            down_peer[i] = q;
            down_dest[i] = q_up_off[me] + (i - x->down_off[q]);
        }
    }
    // Walk order of push_up: runs of kRun rows taken in turn from every owner's group, starting with the rank after
    // this one, so that at any time a rank stores to all owners and no two ranks start on the same one.
    std::vector<int> up_order;
    up_order.reserve(n_up);
    {
        const int kRun = 16;
        std::vector<int> next(P);
        for (int q = 0; q < P; ++q) next[q] = x->up_off[q];
        while (up_order.size() < n_up)
            for (int d = 1; d <= P; ++d) {
                const int q = (me + d) % P;
                const int end = std::min(next[q] + kRun, x->up_off[q + 1]);
                for (int i = next[q]; i < end; ++i) up_order.push_back(i);
                next[q] = end;
            }
    }
    if ((rc = upload_vec(&p->d_up_order, up_order))) return rc;
    if ((rc = upload_vec(&p->d_peer_up_recv, up_base))) return rc;
    if ((rc = upload_vec(&p->d_peer_down_recv, down_base))) return rc;
    if ((rc = upload_vec(&p->d_peer_flag_up, flag_up))) return rc;
    if ((rc = upload_vec(&p->d_peer_flag_down, flag_down))) return rc;
    if ((rc = upload_vec(&p->d_up_peer, up_peer))) return rc;
    if ((rc = upload_vec(&p->d_up_dest_row, up_dest))) return rc;
    if ((rc = upload_vec(&p->d_down_peer, down_peer))) return rc;
    if ((rc = upload_vec(&p->d_down_dest_row, down_dest))) return rc;
    if ((rc = upload_vec(&p->d_need_up, need_up))) return rc;
    if ((rc = upload_vec(&p->d_need_down, need_down))) return rc;
    // nobody may store into a segment before every rank has mapped what it needs: one more collective
    float *d_token = nullptr;
    DRONE_CUDA(cudaMalloc(&d_token, sizeof(float)));
    DRONE_CUDA(cudaMemsetAsync(d_token, 0, sizeof(float), st));
    DRONE_NCCL(ncclAllReduce(d_token, d_token, 1, ncclFloat, ncclSum, c->comm, st));
    DRONE_CUDA(cudaStreamSynchronize(st));
    cudaFree(d_token);
    return DRONE_OK;
}

}  // extern "C"

namespace drone {

// DRONE_P2P_TIMING=1 in the environment makes every exchange measure its five launches with CUDA events, wait for
// them and print one line per call on standard error (a diagnosis aid: it serialises the host with the device).
static bool p2p_timing_enabled() {
    static const bool on = [] {
        const char *v = getenv("DRONE_P2P_TIMING");
        return v && v[0] == '1';
    }();
    return on;
}

struct PhaseTimer {
    bool on;
    cudaStream_t st;
    cudaEvent_t ev[6];
    int n = 0;
    PhaseTimer(bool enabled, cudaStream_t stream) : on(enabled), st(stream) {
        if (on)
            for (auto &e : ev) cudaEventCreate(&e);
    }
    void mark() {
        if (on && n < 6) cudaEventRecord(ev[n++], st);
    }
    void report(int rank, int n_up, int n_m, int F) {
        if (!on) return;
        cudaStreamSynchronize(st);
        float ms[5] = {0, 0, 0, 0, 0};
        for (int i = 0; i + 1 < n; ++i) cudaEventElapsedTime(&ms[i], ev[i], ev[i + 1]);
        fprintf(stderr, "p2p rank %d: push_up %.3f signal %.3f add_push_down %.3f signal %.3f scatter %.3f ms (n_up %d n_m %d F %d)\n",
                rank, ms[0], ms[1], ms[2], ms[3], ms[4], n_up, n_m, F);
        for (auto &e : ev) cudaEventDestroy(e);
    }
};

// One exchange over peer memory; called by drone_exchange_sum when the plan has the transport enabled.
int exchange_sum_p2p(drone_xplan *x, float *d_rows, int F, int ld, cudaStream_t st) {
    drone_p2p *p = x->p2p;
    if (*(volatile int *)p->h_error != 0)
        return set_error(DRONE_E_STATE,
                         "peer-memory exchange: an earlier call gave up waiting for rank %d (%s flag); the ranks are out of step",
                         *p->h_error % 100, *p->h_error >= 200 ? "down" : "up");
    const int P = x->nranks;
    const int n_up = (int)x->up_rows.size(), n_m = (int)x->m_rows.size();
    const unsigned epoch = ++p->epoch;
    unsigned *my_flags = reinterpret_cast<unsigned *>(p->segment);
    float *my_up_recv = reinterpret_cast<float *>(p->segment + kFlagBytes);
    float *my_down_recv = reinterpret_cast<float *>(
        p->segment + kFlagBytes + align_up(x->down_rows.size() * (size_t)x->max_features * 4, 256));
    const bool vec4 = (F % 4 == 0) && (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_rows) & 15) == 0);
    const int nvec = vec4 ? F / 4 : F;
    PhaseTimer timer(p2p_timing_enabled(), st);
    timer.mark();
    if (n_up) {
        const int grid = p2p_grid((long long)n_up * nvec);
        if (vec4) p2p_push_up_kernel<4><<<grid, 256, 0, st>>>(d_rows, ld, x->d_up_rows, p->d_up_peer, p->d_up_dest_row, p->d_up_order, n_up, nvec, p->d_peer_up_recv);
        else p2p_push_up_kernel<1><<<grid, 256, 0, st>>>(d_rows, ld, x->d_up_rows, p->d_up_peer, p->d_up_dest_row, p->d_up_order, n_up, nvec, p->d_peer_up_recv);
        DRONE_LAUNCH_CHECK("p2p_push_up_kernel");
    }
    timer.mark();
    p2p_signal_kernel<<<1, 64, 0, st>>>(p->d_peer_flag_up, p->d_need_down, P, epoch);   // to the owners of my mirrors
    DRONE_LAUNCH_CHECK("p2p_signal_kernel");
    timer.mark();
    if (n_m) {
        const int grid = p2p_grid((long long)n_m * nvec);
        if (vec4) p2p_add_push_down_kernel<4><<<grid, 256, 0, st>>>(d_rows, ld, x->d_m_rows, x->d_m_off, x->d_m_pos, n_m, nvec, my_up_recv, p->d_down_peer, p->d_down_dest_row, p->d_peer_down_recv, my_flags, p->d_need_up, P, epoch, p->d_error, p->d_host_error);
        else p2p_add_push_down_kernel<1><<<grid, 256, 0, st>>>(d_rows, ld, x->d_m_rows, x->d_m_off, x->d_m_pos, n_m, nvec, my_up_recv, p->d_down_peer, p->d_down_dest_row, p->d_peer_down_recv, my_flags, p->d_need_up, P, epoch, p->d_error, p->d_host_error);
        DRONE_LAUNCH_CHECK("p2p_add_push_down_kernel");
    }
    timer.mark();
    p2p_signal_kernel<<<1, 64, 0, st>>>(p->d_peer_flag_down, p->d_need_up, P, epoch);   // to the holders of my mirrors
    DRONE_LAUNCH_CHECK("p2p_signal_kernel");
    timer.mark();
    if (n_up) {
        const int grid = p2p_grid((long long)n_up * nvec);
        if (vec4) p2p_scatter_kernel<4><<<grid, 256, 0, st>>>(d_rows, ld, x->d_up_rows, n_up, nvec, my_down_recv, my_flags + P, p->d_need_down, P, epoch, p->d_error, p->d_host_error);
        else p2p_scatter_kernel<1><<<grid, 256, 0, st>>>(d_rows, ld, x->d_up_rows, n_up, nvec, my_down_recv, my_flags + P, p->d_need_down, P, epoch, p->d_error, p->d_host_error);
        DRONE_LAUNCH_CHECK("p2p_scatter_kernel");
    }
    timer.mark();
    timer.report(x->rank, n_up, n_m, F);
    return DRONE_OK;
}

}  // namespace drone
