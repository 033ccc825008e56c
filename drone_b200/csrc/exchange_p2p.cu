// Mirror/master exchange over peer memory (NVLink, one process per GPU).
//
// Same result as the NCCL transport of exchange.cu, with the packing, the transfer and the unpacking of each
// direction fused into one kernel per direction that stores rows straight into the receiver's memory:
//   push_up:        every mirror row -> the owner's up-receive area (position fixed by the static plan)
//   add_push_down:  master row += its mirrors' rows in ascending rank order; the total goes to every mirror's
//                   down-receive area
//   scatter:        mirror rows take the totals
// Ordering between GPUs uses one epoch word per (receiver, sender, direction): the last block of the sender's store
// kernel to finish (every block fences its stores and counts itself) writes the call's epoch; the receiver polls its
// own words in a ONE-BLOCK
// wait kernel launched in front of add_push_down and scatter.  (Waiting inside the row kernels themselves held every
// SM slot those kernels were given for as long as the slowest peer took, which starved whatever ran beside the
// exchange.)  Every wait is bounded: when it runs out the kernel records an error code in device memory and in pinned
// host memory, the kernels behind it skip their work, this rank publishes no further epoch (so that its peers' waits
// run out too instead of reading rows that were never written), and the next call reports DRONE_E_STATE.  Nothing here uses TMA or cluster multicast; peers are reached with plain
// loads and stores.
//
// The upward half has a second form: an aggregation call (drone_spmm_ex with push_up_to) is given this plan's route
// table and the peers' receive areas, and its kernels store every finished mirror row where push_up would have put
// it; a one-block kernel behind them publishes the epoch (p2p_route_begin / p2p_route_publish), and
// drone_exchange_finish runs add_push_down and scatter.  The ordering argument below holds unchanged with "the
// aggregation of call k+1" in the place of "push_up of call k+1", as long as that aggregation is ordered behind this
// rank's scatter of call k (same stream, or an event between the streams).
//
// Why no host synchronisation is needed between calls: a rank stores into a peer's up-receive area in call k+1 only
// after its own scatter of call k, which waited for that peer's down flag of call k, which the peer wrote after it
// had consumed its up-receive area of call k.  Symmetrically a rank stores into a peer's down-receive area in call
// k+1 only after the peer's up flag of call k+1, which the peer wrote after its scatter of call k.
#include "exchange.cuh"

#include <algorithm>
#include <cstdlib>
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

// The wait as a launch of its own: one block polls, the kernel that follows in the stream does the work.
__global__ void p2p_wait_kernel(const unsigned *flags, const int *need, int nranks, unsigned epoch, int *error,
                                int *host_error, int code) {
    wait_for_peers(flags, need, nranks, epoch, error, host_error, code);
}

// The flags of a direction as a launch of its own, for rows that earlier kernels of the stream stored into the
// peers' memory (those kernels have completed, so their stores are performed; the fence orders the flag behind them).
__global__ void p2p_publish_kernel(unsigned *const *peer_flag, const int *send_to, int nranks, unsigned epoch,
                                   const int *error) {
    if (*(volatile const int *)error != 0) return;      // an earlier wait of this rank gave up: stay silent
    __threadfence_system();
    if ((int)threadIdx.x < nranks && send_to[threadIdx.x]) st_release_sys(peer_flag[threadIdx.x], epoch);
}

// End of a kernel that stored rows into peers' memory: every block fences its stores and counts itself; the last
// one to arrive publishes `epoch` in every peer that expects a flag from this rank (and resets the counter for the
// next launch).  Saves the one-block signal launch that would otherwise sit between the store kernel and the
// peers' waits.
__device__ void publish_when_all_blocks_done(unsigned *done, unsigned *const *peer_flag, const int *send_to, int nranks,
                                             unsigned epoch) {
    __shared__ int last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned arrived = atomicAdd(done, 1u);
        last = arrived == gridDim.x - 1;
        if (last) *done = 0;
    }
    __syncthreads();
    if (last) {
        __threadfence_system();
        if ((int)threadIdx.x < nranks && send_to[threadIdx.x]) st_release_sys(peer_flag[threadIdx.x], epoch);
    }
}

template <int VEC> struct PVec;
template <> struct PVec<4> { using type = float4; };
template <> struct PVec<1> { using type = float; };
__device__ __forceinline__ void vadd(float4 &a, const float4 &b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
__device__ __forceinline__ void vadd(float &a, const float &b) { a += b; }

// One mirror row of the walk: {local row, owner, row in the owner's up-receive area, position in this rank's up list}.
// rows[rec.x, :] -> peer_up_recv[rec.y][rec.z, :]      (nvec = F / VEC vectors per row)
// The records lie in walk order: the mirror rows are grouped by owner, and walking them as they lie would make every
// rank store to the same owner at the same time, whose NVLink ingress then limits all of them.
template <int VEC>
__global__ void p2p_push_up_kernel(const float *__restrict__ rows, long long ld, const int4 *__restrict__ walk, int n_up,
                                   int nvec, float *const *__restrict__ peer_up_recv, const int *error, unsigned *done,
                                   unsigned *const *__restrict__ peer_flag, const int *__restrict__ send_to, int nranks,
                                   unsigned epoch) {
    using V = typename PVec<VEC>::type;
    if (*(volatile const int *)error != 0) return;      // an earlier wait of this rank gave up: stay silent
    const long long total = (long long)n_up * nvec;
    const long long first = blockIdx.x * (long long)blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
    RowColumn at(first, stride, nvec);
    for (long long i = first; i < total; i += stride, at.advance()) {
        const int k = at.row, j = at.col;
        const int4 rec = __ldg(walk + k);
        V *dst = reinterpret_cast<V *>(peer_up_recv[rec.y]) + (long long)rec.z * nvec + j;
        *dst = *(reinterpret_cast<const V *>(rows + (long long)rec.x * ld) + j);
    }
    publish_when_all_blocks_done(done, peer_flag, send_to, nranks, epoch);
}

// Master rows: add the mirrors' rows (fixed order), keep the total, and store it into every mirror's down-receive area.
// pairs[k] = {position of the contribution in my up-receive area, mirroring peer, row in that peer's down-receive area}
// for the k-th (master, mirror) pair; the pairs of master m are m_off[m] .. m_off[m+1]-1, peers ascending.
template <int VEC>
__global__ void p2p_add_push_down_kernel(float *__restrict__ rows, long long ld, const int *__restrict__ m_rows,
                                         const int *__restrict__ m_off, const int4 *__restrict__ pairs, int n_masters,
                                         int nvec, const float *up_recv, float *const *__restrict__ peer_down_recv,
                                         const int *error, unsigned *done, unsigned *const *__restrict__ peer_flag,
                                         const int *__restrict__ send_to, int nranks, unsigned epoch) {
    using V = typename PVec<VEC>::type;
    if (*(volatile const int *)error != 0) return;      // the wait in front of this launch gave up
    const V *recv = reinterpret_cast<const V *>(up_recv);
    const long long total = (long long)n_masters * nvec;
    const long long first = blockIdx.x * (long long)blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
    RowColumn at(first, stride, nvec);
    for (long long i = first; i < total; i += stride, at.advance()) {
        const int m = at.row, j = at.col;
        V *mine = reinterpret_cast<V *>(rows + (long long)m_rows[m] * ld) + j;
        V acc = *mine;
        const int k0 = m_off[m], k1 = m_off[m + 1];
        for (int k = k0; k < k1; ++k) vadd(acc, __ldcv(recv + (long long)__ldg(pairs + k).x * nvec + j));
        *mine = acc;
        for (int k = k0; k < k1; ++k) {
            const int4 pr = __ldg(pairs + k);
            *(reinterpret_cast<V *>(peer_down_recv[pr.y]) + (long long)pr.z * nvec + j) = acc;
        }
    }
    publish_when_all_blocks_done(done, peer_flag, send_to, nranks, epoch);
}

// Mirror rows take the totals their masters stored.
template <int VEC>
__global__ void p2p_scatter_kernel(float *__restrict__ rows, long long ld, const int *__restrict__ up_rows, int n_up,
                                   int nvec, const float *down_recv, const int *error) {
    using V = typename PVec<VEC>::type;
    if (*(volatile const int *)error != 0) return;
    const V *recv = reinterpret_cast<const V *>(down_recv);
    const long long total = (long long)n_up * nvec;
    const long long first = blockIdx.x * (long long)blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
    RowColumn at(first, stride, nvec);
    for (long long i = first; i < total; i += stride, at.advance()) {
        const int r = at.row, j = at.col;
        *(reinterpret_cast<V *>(rows + (long long)up_rows[r] * ld) + j) = __ldcv(recv + i);
    }
}

// The same transport for one small element per boundary vertex instead of a row of features (the PageRank job's
// {value, flag} pairs): send[i] of this rank's up (or down) list goes to its fixed place in the peer's receive area.
// table[k] = {.., peer, place at the peer, position i in this rank's list}; T is 8 or 16 bytes.
template <typename T, bool UP>
__global__ void p2p_move_elements_kernel(const T *__restrict__ send, const int4 *__restrict__ table, int n,
                                         float *const *__restrict__ peer_recv, const int *error, unsigned *done,
                                         unsigned *const *__restrict__ peer_flag, const int *__restrict__ send_to,
                                         int nranks, unsigned epoch) {
    if (*(volatile const int *)error != 0) return;
    for (long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x; k < n; k += (long long)gridDim.x * blockDim.x) {
        const int4 rec = __ldg(table + k);
        const int src = UP ? rec.w : rec.x;
        reinterpret_cast<T *>(peer_recv[rec.y])[rec.z] = send[src];
    }
    publish_when_all_blocks_done(done, peer_flag, send_to, nranks, epoch);
}

// Blocks of a row kernel: at most DRONE_P2P_BLOCKS_PER_SM (default 8) per SM of a 148-SM part.
static inline int p2p_grid(long long n) {
    static const int per_sm = [] {
        const char *v = getenv("DRONE_P2P_BLOCKS_PER_SM");
        const int k = (v && *v) ? atoi(v) : 8;
        return k >= 1 && k <= 8 ? k : 8;
    }();
    long long g = (n + 255) / 256;
    if (g < 1) g = 1;
    if (g > 148 * per_sm) g = 148 * per_sm;
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
    cudaFree(p->d_walk); cudaFree(p->d_pairs); cudaFree(p->d_route);
    cudaFree(p->d_need_up); cudaFree(p->d_need_down);
    if (p->h_error) cudaFreeHost(p->h_error);
    cudaFree(p->d_error);
    cudaFree(p->d_done);
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

// What drone_xplan_enable_p2p does between its two collectives: reads the other ranks' records, maps their segments
// and uploads this rank's tables.  Returns the first local failure; the caller folds it into the closing collective.
static int p2p_connect(drone_xplan *x, drone_p2p *p, const std::vector<char> &all, size_t rec_bytes) {
    const int P = x->nranks, me = x->rank;
    const size_t n_up = x->up_rows.size(), n_down = x->down_rows.size();
    std::vector<float *> up_base(P, nullptr), down_base(P, nullptr);
    std::vector<unsigned *> flag_up(P, nullptr), flag_down(P, nullptr);
    std::vector<int> need_up(P, 0), need_down(P, 0);
    std::vector<int> up_peer(n_up), up_dest(n_up), down_peer(n_down), down_dest(n_down);
    for (int q = 0; q < P; ++q) {
        if (q == me) continue;
        const int up_cnt = x->up_off[q + 1] - x->up_off[q], down_cnt = x->down_off[q + 1] - x->down_off[q];
        need_up[q] = down_cnt > 0;     // q holds mirrors of my masters: it sends up to me
        need_down[q] = up_cnt > 0;     // q owns masters of my mirrors: it sends down to me
        const char *rec = all.data() + rec_bytes * q;
        const int *qi = reinterpret_cast<const int *>(rec + sizeof(cudaIpcMemHandle_t));
        const int q_n_down = qi[0], q_maxf = qi[2];
        const int *q_down_off = qi + 4, *q_up_off = qi + 4 + (P + 1);
        if (q_maxf != x->max_features)
            return set_error(DRONE_E_INVALID, "drone_xplan_enable_p2p: rank %d was planned for %d features, this rank for %d", q,
                             q_maxf, x->max_features);
        if (q_down_off[me + 1] - q_down_off[me] != up_cnt || q_up_off[me + 1] - q_up_off[me] != down_cnt)
            return set_error(DRONE_E_STATE, "drone_xplan_enable_p2p: plans of rank %d and %d disagree on their row counts", me, q);
        if (!up_cnt && !down_cnt) continue;
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
    std::vector<int4> walk;
    walk.reserve(n_up);
    {
        const int kRun = 16;
        std::vector<int> next(P);
        for (int q = 0; q < P; ++q) next[q] = x->up_off[q];
        while (walk.size() < n_up)
            for (int d = 1; d <= P; ++d) {
                const int q = (me + d) % P;
                const int end = std::min(next[q] + kRun, x->up_off[q + 1]);
                for (int i = next[q]; i < end; ++i) walk.push_back(make_int4(x->up_rows[i], up_peer[i], up_dest[i], i));
                next[q] = end;
            }
    }
    std::vector<int4> pairs(x->m_pos.size());
    for (size_t k = 0; k < pairs.size(); ++k) {
        const int pos = x->m_pos[k];
        pairs[k] = make_int4(pos, down_peer[pos], down_dest[pos], 0);
    }
    std::vector<int2> route((size_t)x->n_local, make_int2(-1, 0));
    for (size_t i = 0; i < n_up; ++i) route[(size_t)x->up_rows[i]] = make_int2(up_peer[i], up_dest[i]);
    int rc;
    if ((rc = upload_vec(&p->d_route, route))) return rc;
    if ((rc = upload_vec(&p->d_walk, walk))) return rc;
    if ((rc = upload_vec(&p->d_pairs, pairs))) return rc;
    if ((rc = upload_vec(&p->d_peer_up_recv, up_base))) return rc;
    if ((rc = upload_vec(&p->d_peer_down_recv, down_base))) return rc;
    if ((rc = upload_vec(&p->d_peer_flag_up, flag_up))) return rc;
    if ((rc = upload_vec(&p->d_peer_flag_down, flag_down))) return rc;
    if ((rc = upload_vec(&p->d_need_up, need_up))) return rc;
    if ((rc = upload_vec(&p->d_need_down, need_down))) return rc;
    return DRONE_OK;
}

int drone_xplan_enable_p2p(drone_xplan *x, drone_comm *c, void *stream) {
    DRONE_REQUIRE(x && c, "drone_xplan_enable_p2p: NULL plan or communicator");
    DRONE_REQUIRE(c->nranks == x->nranks && c->rank == x->rank, "drone_xplan_enable_p2p: plan is rank %d/%d, comm %d/%d",
                  x->rank, x->nranks, c->rank, c->nranks);
    DRONE_REQUIRE(x->nranks <= 64, "drone_xplan_enable_p2p: at most 64 ranks");
    if (x->p2p || x->nranks == 1) return DRONE_OK;
    int rc = xplan_ensure_device(x);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const int P = x->nranks;
    const size_t n_up = x->up_rows.size(), n_down = x->down_rows.size();

    // Everything that can fail on this rank alone comes first: a rank that returns from here has started no
    // collective, so its peers are not left inside one that this rank never joins half-way.
    struct Temp {
        char *d_mine = nullptr, *d_all = nullptr;
        int *d_status = nullptr;
        ~Temp() { cudaFree(d_mine); cudaFree(d_all); cudaFree(d_status); }
    } t;
    const size_t ints_per_rank = 4 + 2 * (size_t)(P + 1);
    const size_t rec_bytes = align_up(sizeof(cudaIpcMemHandle_t) + ints_per_rank * 4, 16);
    drone_p2p *p = new (std::nothrow) drone_p2p();
    if (!p) return set_error(DRONE_E_INVALID, "drone_xplan_enable_p2p: out of host memory");
    x->p2p = p;
    p->peer_segment.assign(P, nullptr);
    const size_t up_bytes = align_up(n_down * (size_t)x->max_features * 4, 256);
    const size_t down_bytes = align_up(n_up * (size_t)x->max_features * 4, 256);
    p->segment_bytes = kFlagBytes + up_bytes + down_bytes;
    std::vector<char> mine(rec_bytes, 0), all(rec_bytes * P, 0);
    auto local_setup = [&]() -> int {
        DRONE_CUDA(cudaMalloc(&p->segment, p->segment_bytes));
        DRONE_CUDA(cudaMemsetAsync(p->segment, 0, p->segment_bytes, st));
        DRONE_CUDA(cudaHostAlloc(&p->h_error, sizeof(int), cudaHostAllocMapped));
        *p->h_error = 0;
        DRONE_CUDA(cudaHostGetDevicePointer(&p->d_host_error, p->h_error, 0));
        DRONE_CUDA(cudaMalloc(&p->d_error, sizeof(int)));
        DRONE_CUDA(cudaMemsetAsync(p->d_error, 0, sizeof(int), st));
        DRONE_CUDA(cudaMalloc(&p->d_done, 2 * sizeof(unsigned)));
        DRONE_CUDA(cudaMemsetAsync(p->d_done, 0, 2 * sizeof(unsigned), st));
        DRONE_CUDA(cudaMalloc(&t.d_mine, rec_bytes));
        DRONE_CUDA(cudaMalloc(&t.d_all, rec_bytes * P));
        DRONE_CUDA(cudaMalloc(&t.d_status, sizeof(int)));
        // what every rank tells the others: IPC handle, sizes, its two offset tables
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
        DRONE_CUDA(cudaMemcpyAsync(t.d_mine, mine.data(), rec_bytes, cudaMemcpyHostToDevice, st));
        return DRONE_OK;
    };
    if ((rc = local_setup())) {
        xplan_p2p_release(x);
        return rc;
    }

    // first collective: everybody's record
    auto gather = [&]() -> int {
        DRONE_NCCL(ncclAllGather(t.d_mine, t.d_all, rec_bytes, ncclChar, c->comm, st));
        DRONE_CUDA(cudaMemcpyAsync(all.data(), t.d_all, rec_bytes * P, cudaMemcpyDeviceToHost, st));
        DRONE_CUDA(cudaStreamSynchronize(st));
        return DRONE_OK;
    };
    int status = gather();
    char first_message[512] = "";
    if (status == DRONE_OK) status = p2p_connect(x, p, all, rec_bytes);
    if (status != DRONE_OK) snprintf(first_message, sizeof(first_message), "%s", drone_last_error());

    // Closing collective, joined by every rank whatever happened above: nobody may store into a segment before every
    // rank has mapped what it needs, and a rank that failed must not leave the others waiting inside the collective.
    // It carries the status: the smallest (most severe) code of any rank comes back on all of them.
    int agreed = status;
    auto close = [&]() -> int {
        DRONE_CUDA(cudaMemcpyAsync(t.d_status, &status, sizeof(int), cudaMemcpyHostToDevice, st));
        DRONE_NCCL(ncclAllReduce(t.d_status, t.d_status, 1, ncclInt, ncclMin, c->comm, st));
        DRONE_CUDA(cudaMemcpyAsync(&agreed, t.d_status, sizeof(int), cudaMemcpyDeviceToHost, st));
        DRONE_CUDA(cudaStreamSynchronize(st));
        return DRONE_OK;
    };
    const int close_rc = close();
    if (close_rc != DRONE_OK && status == DRONE_OK) {
        status = agreed = close_rc;
        snprintf(first_message, sizeof(first_message), "%s", drone_last_error());
    }
    if (agreed != DRONE_OK) {
        xplan_p2p_release(x);     // unmaps the peers' segments, frees this rank's; the plan keeps its NCCL transport
        if (status != DRONE_OK) return set_error(agreed, "%s", first_message);
        return set_error(agreed, "drone_xplan_enable_p2p: another rank failed to set the transport up (code %d); "
                         "it is off on every rank", agreed);
    }
    return DRONE_OK;
}

}  // extern "C"

namespace drone {

// DRONE_P2P_TIMING=1 in the environment makes every exchange measure its two halves with CUDA events, wait for
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
        fprintf(stderr, "p2p rank %d: push_up %.3f, wait + add_push_down + wait + scatter %.3f ms (n_up %d n_m %d F %d)\n",
                rank, ms[0], ms[1], n_up, n_m, F);
        for (auto &e : ev) cudaEventDestroy(e);
    }
};

static int p2p_check_in_step(drone_p2p *p) {
    if (*(volatile int *)p->h_error != 0)
        return set_error(DRONE_E_STATE,
                         "peer-memory exchange: an earlier call gave up waiting for rank %d (%s flag); the ranks are out of step",
                         *p->h_error % 100, *p->h_error >= 200 ? "down" : "up");
    return DRONE_OK;
}

static bool p2p_rows_as_float4(const float *d_rows, int F, int ld) {
    return (F % 4 == 0) && (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_rows) & 15) == 0);
}

// Upward half, as a copy kernel of its own: my mirror rows go to their owners, whose flags the kernel's last block sets.
int p2p_push_up(drone_xplan *x, const float *d_rows, int F, int ld, cudaStream_t st) {
    drone_p2p *p = x->p2p;
    const int P = x->nranks, n_up = (int)x->up_rows.size();
    const bool vec4 = p2p_rows_as_float4(d_rows, F, ld);
    const int nvec = vec4 ? F / 4 : F;
    if (n_up) {
        const int grid = p2p_grid((long long)n_up * nvec);
        if (vec4) p2p_push_up_kernel<4><<<grid, 256, 0, st>>>(d_rows, ld, p->d_walk, n_up, nvec, p->d_peer_up_recv, p->d_error, p->d_done, p->d_peer_flag_up, p->d_need_down, P, p->epoch);
        else p2p_push_up_kernel<1><<<grid, 256, 0, st>>>(d_rows, ld, p->d_walk, n_up, nvec, p->d_peer_up_recv, p->d_error, p->d_done, p->d_peer_flag_up, p->d_need_down, P, p->epoch);
        DRONE_LAUNCH_CHECK("p2p_push_up_kernel");
    }
    return DRONE_OK;
}

// Upward half done by the caller's kernels: opens the epoch and hands out the routing tables.
int p2p_route_begin(drone_xplan *x, int n_rows, int F, const int2 **route, float *const **peer_rows) {
    *route = nullptr;
    *peer_rows = nullptr;
    if (x->nranks == 1) return DRONE_OK;      // one rank: no mirrors, nothing to send (the caller sees no table)
    drone_p2p *p = x->p2p;
    if (!p) return set_error(DRONE_E_STATE, "peer-memory transport is not enabled on this exchange plan");
    if (n_rows != x->n_local)
        return set_error(DRONE_E_INVALID, "the exchange plan covers %d local rows, the aggregation plan has %d", x->n_local, n_rows);
    if (F > x->max_features)
        return set_error(DRONE_E_TOO_LARGE, "exchange of %d features on a plan made for at most %d", F, x->max_features);
    if (p->push_pending)
        return set_error(DRONE_E_STATE, "an aggregation already sent this plan's mirror rows up: drone_exchange_finish is due");
    const int rc = p2p_check_in_step(p);
    if (rc) return rc;
    ++p->epoch;
    p->push_pending = true;
    *route = p->d_route;
    *peer_rows = p->d_peer_up_recv;
    return DRONE_OK;
}

int p2p_route_publish(drone_xplan *x, cudaStream_t st) {
    drone_p2p *p = x->p2p;
    if (!x->up_rows.empty()) {
        p2p_publish_kernel<<<1, 64, 0, st>>>(p->d_peer_flag_up, p->d_need_down, x->nranks, p->epoch, p->d_error);
        DRONE_LAUNCH_CHECK("p2p_publish_kernel");
    }
    return DRONE_OK;
}

// Downward half: masters wait for their mirrors' rows, add them and store the totals into the mirrors' memory; mirror
// rows wait for the totals and take them.
int exchange_finish_p2p(drone_xplan *x, float *d_rows, int F, int ld, cudaStream_t st) {
    drone_p2p *p = x->p2p;
    const int P = x->nranks;
    const int n_up = (int)x->up_rows.size(), n_m = (int)x->m_rows.size();
    const unsigned epoch = p->epoch;
    p->push_pending = false;
    unsigned *my_flags = reinterpret_cast<unsigned *>(p->segment);
    float *my_up_recv = reinterpret_cast<float *>(p->segment + kFlagBytes);
    float *my_down_recv = reinterpret_cast<float *>(
        p->segment + kFlagBytes + align_up(x->down_rows.size() * (size_t)x->max_features * 4, 256));
    const bool vec4 = p2p_rows_as_float4(d_rows, F, ld);
    const int nvec = vec4 ? F / 4 : F;
    if (n_m) {
        p2p_wait_kernel<<<1, 64, 0, st>>>(my_flags, p->d_need_up, P, epoch, p->d_error, p->d_host_error, 100);
        DRONE_LAUNCH_CHECK("p2p_wait_kernel");
        const int grid = p2p_grid((long long)n_m * nvec);
        if (vec4) p2p_add_push_down_kernel<4><<<grid, 256, 0, st>>>(d_rows, ld, x->d_m_rows, x->d_m_off, p->d_pairs, n_m, nvec, my_up_recv, p->d_peer_down_recv, p->d_error, p->d_done + 1, p->d_peer_flag_down, p->d_need_up, P, epoch);
        else p2p_add_push_down_kernel<1><<<grid, 256, 0, st>>>(d_rows, ld, x->d_m_rows, x->d_m_off, p->d_pairs, n_m, nvec, my_up_recv, p->d_peer_down_recv, p->d_error, p->d_done + 1, p->d_peer_flag_down, p->d_need_up, P, epoch);
        DRONE_LAUNCH_CHECK("p2p_add_push_down_kernel");
    }
    if (n_up) {
        p2p_wait_kernel<<<1, 64, 0, st>>>(my_flags + P, p->d_need_down, P, epoch, p->d_error, p->d_host_error, 200);
        DRONE_LAUNCH_CHECK("p2p_wait_kernel");
        const int grid = p2p_grid((long long)n_up * nvec);
        if (vec4) p2p_scatter_kernel<4><<<grid, 256, 0, st>>>(d_rows, ld, x->d_up_rows, n_up, nvec, my_down_recv, p->d_error);
        else p2p_scatter_kernel<1><<<grid, 256, 0, st>>>(d_rows, ld, x->d_up_rows, n_up, nvec, my_down_recv, p->d_error);
        DRONE_LAUNCH_CHECK("p2p_scatter_kernel");
    }
    return DRONE_OK;
}

// One exchange over peer memory; called by drone_exchange_sum when the plan has the transport enabled.
int exchange_sum_p2p(drone_xplan *x, float *d_rows, int F, int ld, cudaStream_t st) {
    drone_p2p *p = x->p2p;
    if (p->push_pending)
        return set_error(DRONE_E_STATE, "an aggregation already sent this plan's mirror rows up: drone_exchange_finish is due");
    int rc = p2p_check_in_step(p);
    if (rc) return rc;
    ++p->epoch;
    PhaseTimer timer(p2p_timing_enabled(), st);
    timer.mark();
    if ((rc = p2p_push_up(x, d_rows, F, ld, st))) return rc;
    timer.mark();
    if ((rc = exchange_finish_p2p(x, d_rows, F, ld, st))) return rc;
    timer.mark();
    timer.report(x->rank, (int)x->up_rows.size(), (int)x->m_rows.size(), F);
    return DRONE_OK;
}

// One direction of the exchange for elements of `bytes` (8 or 16) per boundary vertex: stores this rank's send list
// into the peers' receive areas, publishes the epoch, waits for the peers' epochs.  *recv_out is where the elements
// sent to this rank lie afterwards (indexed like the receive buffer of the send/recv transport).  up = true starts a
// new epoch; the down move that follows belongs to the same one.
int p2p_move_elements(drone_xplan *x, const void *d_send, size_t bytes, bool up, cudaStream_t st, const void **recv_out) {
    drone_p2p *p = x->p2p;
    if (!p) return set_error(DRONE_E_STATE, "peer-memory transport is not enabled on this exchange plan");
    if (bytes != 8 && bytes != 16)
        return set_error(DRONE_E_INVALID, "peer-memory element move: %zu bytes per element (8 or 16)", bytes);
    if ((size_t)x->max_features * 4 < bytes)
        return set_error(DRONE_E_TOO_LARGE, "peer-memory element move: the plan's receive areas hold %d floats per vertex, "
                         "%zu bytes are needed", x->max_features, bytes);
    if (*(volatile int *)p->h_error != 0)
        return set_error(DRONE_E_STATE,
                         "peer-memory exchange: an earlier call gave up waiting for rank %d (%s flag); the ranks are out of step",
                         *p->h_error % 100, *p->h_error >= 200 ? "down" : "up");
    const int P = x->nranks;
    const int n_up = (int)x->up_rows.size(), n_down = (int)x->down_rows.size();
    if (up) ++p->epoch;
    const unsigned epoch = p->epoch;
    unsigned *my_flags = reinterpret_cast<unsigned *>(p->segment);
    char *my_up_recv = p->segment + kFlagBytes;
    char *my_down_recv = p->segment + kFlagBytes + align_up(x->down_rows.size() * (size_t)x->max_features * 4, 256);
    if (up) {
        if (n_up) {
            const int grid = p2p_grid(n_up);
            if (bytes == 8) p2p_move_elements_kernel<float2, true><<<grid, 256, 0, st>>>((const float2 *)d_send, p->d_walk, n_up, p->d_peer_up_recv, p->d_error, p->d_done, p->d_peer_flag_up, p->d_need_down, P, epoch);
            else p2p_move_elements_kernel<double2, true><<<grid, 256, 0, st>>>((const double2 *)d_send, p->d_walk, n_up, p->d_peer_up_recv, p->d_error, p->d_done, p->d_peer_flag_up, p->d_need_down, P, epoch);
            DRONE_LAUNCH_CHECK("p2p_move_elements_kernel");
        }
        if (n_down) {
            p2p_wait_kernel<<<1, 64, 0, st>>>(my_flags, p->d_need_up, P, epoch, p->d_error, p->d_host_error, 100);
            DRONE_LAUNCH_CHECK("p2p_wait_kernel");
        }
        *recv_out = my_up_recv;
    } else {
        if (n_down) {
            const int grid = p2p_grid(n_down);
            if (bytes == 8) p2p_move_elements_kernel<float2, false><<<grid, 256, 0, st>>>((const float2 *)d_send, p->d_pairs, n_down, p->d_peer_down_recv, p->d_error, p->d_done + 1, p->d_peer_flag_down, p->d_need_up, P, epoch);
            else p2p_move_elements_kernel<double2, false><<<grid, 256, 0, st>>>((const double2 *)d_send, p->d_pairs, n_down, p->d_peer_down_recv, p->d_error, p->d_done + 1, p->d_peer_flag_down, p->d_need_up, P, epoch);
            DRONE_LAUNCH_CHECK("p2p_move_elements_kernel");
        }
        if (n_up) {
            p2p_wait_kernel<<<1, 64, 0, st>>>(my_flags + P, p->d_need_down, P, epoch, p->d_error, p->d_host_error, 200);
            DRONE_LAUNCH_CHECK("p2p_wait_kernel");
        }
        *recv_out = my_down_recv;
    }
    return DRONE_OK;
}

}  // namespace drone
