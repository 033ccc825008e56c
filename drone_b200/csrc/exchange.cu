// EBV vertex-cut exchange: partial sums on mirror rows are added into the master
// row, and the total is written back to every mirror, so that afterwards every
// replica of a vertex holds the global sum.
//
// The reference packs rows in an order produced by atomics and therefore ships
// the global id of every row, plus the per-peer counts, on every call
// (cuda_gcn/src/cuda/cuda_communicate.cu:126-207,276-372).  Here the routing
// tables are turned once into a static plan: for every peer the list of local
// rows that go up (my mirrors it owns) and the list that comes back down (my
// masters it mirrors), both sorted by global vertex id, which both ends can
// compute independently.  A call then moves payload only:
//     gather mirror rows -> all-to-all-v -> add at masters in ascending peer
//     order (and gather the totals) -> all-to-all-v -> scatter into mirror rows.
// The additions have a fixed order, so results are bit-reproducible.
#include "exchange.cuh"

#include <algorithm>
#include <new>

namespace drone {

int exchange_sum_p2p(drone_xplan *x, float *d_rows, int F, int ld, cudaStream_t st);
void xplan_p2p_release(drone_xplan *x);

// buf[i, 0:F] = rows[list[i], 0:F]
// rows[r, 0:nvec] = 0 for every row r that is a mirror (mirror2worker[r] != -1); V = float4 or float.
template <typename V>
__global__ void clear_mirror_rows_kernel(float *__restrict__ rows, int n_rows, int nvec, long long ld,
                                         const int *__restrict__ mirror2worker) {
    const long long total = (long long)n_rows * nvec;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / nvec), j = (int)(i - (long long)r * nvec);
        if (mirror2worker[r] != -1) reinterpret_cast<V *>(rows + (long long)r * ld)[j] = V{};
    }
}

__global__ void gather_rows_kernel(const float *__restrict__ rows, long long ld, const int *__restrict__ list,
                                   int n_list, int F, float *__restrict__ buf) {
    const long long total = (long long)n_list * F;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / F), j = (int)(i - (long long)r * F);
        buf[i] = rows[(long long)list[r] * ld + j];
    }
}

// rows[list[i], 0:F] = buf[i, 0:F]
__global__ void scatter_rows_kernel(float *__restrict__ rows, long long ld, const int *__restrict__ list,
                                    int n_list, int F, const float *__restrict__ buf) {
    const long long total = (long long)n_list * F;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / F), j = (int)(i - (long long)r * F);
        rows[(long long)list[r] * ld + j] = buf[i];
    }
}

// For master row m_rows[i]: rows[row] += recv[m_pos[k]] for k in m_off[i] .. m_off[i+1], in that order.
__global__ void add_at_masters_kernel(float *__restrict__ rows, long long ld, const int *__restrict__ m_rows,
                                      const int *__restrict__ m_off, const int *__restrict__ m_pos, int n_masters,
                                      int F, const float *__restrict__ recv) {
    const long long total = (long long)n_masters * F;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int m = (int)(i / F), j = (int)(i - (long long)m * F);
        float acc = rows[(long long)m_rows[m] * ld + j];
        for (int k = m_off[m]; k < m_off[m + 1]; ++k) acc += recv[(long long)m_pos[k] * F + j];
        rows[(long long)m_rows[m] * ld + j] = acc;
    }
}

static inline int grid_for(long long n) {
    long long g = (n + 255) / 256;
    if (g < 1) g = 1;
    if (g > 148 * 16) g = 148 * 16;
    return (int)g;
}

template <typename T>
static int upload(T **dst, const std::vector<T> &src) {
    DRONE_CUDA(cudaMalloc(dst, sizeof(T) * (src.size() > 0 ? src.size() : 1)));
    if (!src.empty()) DRONE_CUDA(cudaMemcpy(*dst, src.data(), sizeof(T) * src.size(), cudaMemcpyHostToDevice));
    return DRONE_OK;
}

int xplan_ensure_device(drone_xplan *x) {
    int dev = -1;
    DRONE_CUDA(cudaGetDevice(&dev));
    if (x->device == dev) return DRONE_OK;
    if (x->device >= 0)
        return set_error(DRONE_E_STATE, "exchange plan was first used on device %d, now on %d", x->device, dev);
    int rc;
    if ((rc = upload(&x->d_up_rows, x->up_rows))) return rc;
    if ((rc = upload(&x->d_down_rows, x->down_rows))) return rc;
    if ((rc = upload(&x->d_m_rows, x->m_rows))) return rc;
    if ((rc = upload(&x->d_m_off, x->m_off))) return rc;
    if ((rc = upload(&x->d_m_pos, x->m_pos))) return rc;
    const size_t rows = std::max(x->up_rows.size(), x->down_rows.size());
    x->buf_floats = std::max<size_t>(rows * (size_t)x->max_features, 1);
    DRONE_CUDA(cudaMalloc(&x->d_send, sizeof(float) * x->buf_floats));
    DRONE_CUDA(cudaMalloc(&x->d_recv, sizeof(float) * x->buf_floats));
    x->device = dev;
    return DRONE_OK;
}

// One all-to-all-v: send slice q of `send` (rows s_off[q]..s_off[q+1]) to peer q, receive slice q of `recv`.
static int all_to_all_v(const drone_comm *c, const float *send, const std::vector<int> &s_off, float *recv,
                        const std::vector<int> &r_off, int F, cudaStream_t st) {
    DRONE_NCCL(ncclGroupStart());
    for (int q = 0; q < c->nranks; ++q) {
        if (q == c->rank) continue;
        const size_t ns = (size_t)(s_off[q + 1] - s_off[q]) * F, nr = (size_t)(r_off[q + 1] - r_off[q]) * F;
        if (ns) DRONE_NCCL(ncclSend(send + (size_t)s_off[q] * F, ns, ncclFloat, q, c->comm, st));
        if (nr) DRONE_NCCL(ncclRecv(recv + (size_t)r_off[q] * F, nr, ncclFloat, q, c->comm, st));
    }
    DRONE_NCCL(ncclGroupEnd());
    return DRONE_OK;
}

}  // namespace drone

using namespace drone;

extern "C" {

int drone_comm_unique_id(void *id_out, size_t id_bytes) {
    DRONE_REQUIRE(id_out != nullptr, "drone_comm_unique_id: NULL output");
    DRONE_REQUIRE(id_bytes >= sizeof(ncclUniqueId), "drone_comm_unique_id: buffer of %zu bytes, need %zu", id_bytes,
                  sizeof(ncclUniqueId));
    ncclUniqueId id;
    DRONE_NCCL(ncclGetUniqueId(&id));
    memcpy(id_out, &id, sizeof(id));
    return DRONE_OK;
}

int drone_comm_create(drone_comm **out, int rank, int nranks, const void *id, size_t id_bytes) {
    DRONE_REQUIRE(out != nullptr, "drone_comm_create: out is NULL");
    *out = nullptr;
    DRONE_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, "drone_comm_create: rank %d of %d", rank, nranks);
    DRONE_REQUIRE(id != nullptr && id_bytes >= sizeof(ncclUniqueId), "drone_comm_create: bad unique id");
    drone_comm *c = new (std::nothrow) drone_comm();
    if (!c) return set_error(DRONE_E_INVALID, "drone_comm_create: out of host memory");
    c->rank = rank;
    c->nranks = nranks;
    c->owned = true;
    ncclUniqueId nid;
    memcpy(&nid, id, sizeof(nid));
    ncclResult_t r = ncclCommInitRank(&c->comm, nranks, nid, rank);
    if (r != ncclSuccess) {
        delete c;
        return set_error(DRONE_E_NCCL, "ncclCommInitRank failed: %s", ncclGetErrorString(r));
    }
    *out = c;
    return DRONE_OK;
}

int drone_comm_adopt(drone_comm **out, void *nccl_comm, int rank, int nranks) {
    DRONE_REQUIRE(out != nullptr && nccl_comm != nullptr, "drone_comm_adopt: NULL argument");
    DRONE_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, "drone_comm_adopt: rank %d of %d", rank, nranks);
    drone_comm *c = new (std::nothrow) drone_comm();
    if (!c) return set_error(DRONE_E_INVALID, "drone_comm_adopt: out of host memory");
    c->comm = (ncclComm_t)nccl_comm;
    c->rank = rank;
    c->nranks = nranks;
    c->owned = false;
    *out = c;
    return DRONE_OK;
}

int drone_comm_destroy(drone_comm *c) {
    if (!c) return DRONE_OK;
    if (c->owned && c->comm) ncclCommDestroy(c->comm);
    delete c;
    return DRONE_OK;
}

int drone_comm_allreduce_sum(drone_comm *c, void *d_buf, size_t count, int is_double, void *stream) {
    DRONE_REQUIRE(c && d_buf, "drone_comm_allreduce_sum: NULL argument");
    if (c->nranks == 1 || count == 0) return DRONE_OK;
    DRONE_NCCL(ncclAllReduce(d_buf, d_buf, count, is_double ? ncclDouble : ncclFloat, ncclSum, c->comm,
                             (cudaStream_t)stream));
    return DRONE_OK;
}

int drone_comm_bcast(drone_comm *c, float *d_buf, size_t count, int root, void *stream) {
    DRONE_REQUIRE(c && d_buf, "drone_comm_bcast: NULL argument");
    DRONE_REQUIRE(root >= 0 && root < c->nranks, "drone_comm_bcast: root %d of %d ranks", root, c->nranks);
    if (c->nranks == 1 || count == 0) return DRONE_OK;
    DRONE_NCCL(ncclBroadcast(d_buf, d_buf, count, ncclFloat, root, c->comm, (cudaStream_t)stream));
    return DRONE_OK;
}

int drone_comm_reduce_sum(drone_comm *c, float *d_buf, size_t count, int root, void *stream) {
    DRONE_REQUIRE(c && d_buf, "drone_comm_reduce_sum: NULL argument");
    DRONE_REQUIRE(root >= 0 && root < c->nranks, "drone_comm_reduce_sum: root %d of %d ranks", root, c->nranks);
    if (c->nranks == 1 || count == 0) return DRONE_OK;
    DRONE_NCCL(ncclReduce(d_buf, d_buf, count, ncclFloat, ncclSum, root, c->comm, (cudaStream_t)stream));
    return DRONE_OK;
}

int drone_clear_mirror_rows(float *d_rows, int n_rows, int F, int ld, const int *d_mirror2worker, void *stream) {
    DRONE_REQUIRE(n_rows >= 0 && F >= 1 && ld >= F, "drone_clear_mirror_rows: n_rows=%d F=%d ld=%d", n_rows, F, ld);
    if (n_rows == 0) return DRONE_OK;
    DRONE_REQUIRE(d_rows && d_mirror2worker, "drone_clear_mirror_rows: NULL argument");
    const bool vec4 = (F % 4 == 0) && (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_rows) & 15) == 0);
    const long long total = (long long)n_rows * (vec4 ? F / 4 : F);
    const int grid = (int)std::min<long long>((total + 255) / 256, 148 * 16);
    if (vec4) clear_mirror_rows_kernel<float4><<<grid, 256, 0, (cudaStream_t)stream>>>(d_rows, n_rows, F / 4, ld, d_mirror2worker);
    else clear_mirror_rows_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(d_rows, n_rows, F, ld, d_mirror2worker);
    DRONE_LAUNCH_CHECK("clear_mirror_rows_kernel");
    return DRONE_OK;
}

int drone_xplan_create(drone_xplan **out, int rank, int nranks, int n_local, const int *h_local2global,
                       const int *h_mirror2worker, const int *h_master_worker_index, const int *h_master2workers,
                       int max_features) {
    DRONE_REQUIRE(out != nullptr, "drone_xplan_create: out is NULL");
    *out = nullptr;
    DRONE_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, "drone_xplan_create: rank %d of %d", rank, nranks);
    DRONE_REQUIRE(n_local >= 0 && max_features >= 1, "drone_xplan_create: n_local=%d max_features=%d", n_local,
                  max_features);
    DRONE_REQUIRE(n_local == 0 || (h_local2global && h_mirror2worker && h_master_worker_index),
                  "drone_xplan_create: NULL routing table");
    drone_xplan *x = new (std::nothrow) drone_xplan();
    if (!x) return set_error(DRONE_E_INVALID, "drone_xplan_create: out of host memory");
    x->rank = rank;
    x->nranks = nranks;
    x->n_local = n_local;
    x->max_features = max_features;

    // (peer, global id, local row) triples for both directions
    struct Item { int peer, gid, row; };
    std::vector<Item> up, down;
    for (int r = 0; r < n_local; ++r) {
        const int owner = h_mirror2worker[r];
        if (owner != -1) {
            if (owner < 0 || owner >= nranks || owner == rank) {
                delete x;
                return set_error(DRONE_E_INVALID, "drone_xplan_create: row %d is a mirror of worker %d (self is %d of %d)",
                                 r, owner, rank, nranks);
            }
            up.push_back({owner, h_local2global[r], r});
        }
        for (int k = h_master_worker_index[r]; k < h_master_worker_index[r + 1]; ++k) {
            const int q = h_master2workers[k];
            if (q < 0 || q >= nranks || q == rank) {
                delete x;
                return set_error(DRONE_E_INVALID, "drone_xplan_create: master row %d lists mirror worker %d", r, q);
            }
            down.push_back({q, h_local2global[r], r});
        }
    }
    auto by_peer_gid = [](const Item &a, const Item &b) { return a.peer != b.peer ? a.peer < b.peer : a.gid < b.gid; };
    std::sort(up.begin(), up.end(), by_peer_gid);
    std::sort(down.begin(), down.end(), by_peer_gid);
    x->up_off.assign(nranks + 1, 0);
    x->down_off.assign(nranks + 1, 0);
    for (const Item &i : up) { x->up_rows.push_back(i.row); x->up_off[i.peer + 1]++; }
    for (const Item &i : down) { x->down_rows.push_back(i.row); x->down_off[i.peer + 1]++; }
    for (int q = 0; q < nranks; ++q) { x->up_off[q + 1] += x->up_off[q]; x->down_off[q + 1] += x->down_off[q]; }

    // master rows: contributions arrive at position p of the `down`-ordered receive buffer (the up
    // traffic of peer q towards me is ordered exactly like my down list for q)
    std::vector<std::vector<int>> pos_of_row;  // indexed by dense master number
    std::vector<int> master_no(n_local, -1);
    for (size_t p = 0; p < down.size(); ++p) {
        const int r = down[p].row;
        if (master_no[r] < 0) {
            master_no[r] = (int)x->m_rows.size();
            x->m_rows.push_back(r);
            pos_of_row.emplace_back();
        }
        pos_of_row[master_no[r]].push_back((int)p);   // down is sorted by peer: positions ascend with peer
    }
    x->m_off.push_back(0);
    for (auto &v : pos_of_row) {
        for (int p : v) x->m_pos.push_back(p);
        x->m_off.push_back((int)x->m_pos.size());
    }
    *out = x;
    return DRONE_OK;
}

int drone_xplan_destroy(drone_xplan *x) {
    if (!x) return DRONE_OK;
    if (x->device >= 0) {
        int prev = -1;
        cudaGetDevice(&prev);
        cudaSetDevice(x->device);
        xplan_p2p_release(x);
        cudaFree(x->d_up_rows); cudaFree(x->d_down_rows); cudaFree(x->d_m_rows); cudaFree(x->d_m_off);
        cudaFree(x->d_m_pos); cudaFree(x->d_send); cudaFree(x->d_recv);
        if (prev >= 0) cudaSetDevice(prev);
    }
    delete x;
    return DRONE_OK;
}

int drone_xplan_counts(const drone_xplan *x, int *up_rows_per_peer, int *down_rows_per_peer, int *n_master_rows) {
    DRONE_REQUIRE(x != nullptr, "drone_xplan_counts: plan is NULL");
    for (int q = 0; q < x->nranks; ++q) {
        if (up_rows_per_peer) up_rows_per_peer[q] = x->up_off[q + 1] - x->up_off[q];
        if (down_rows_per_peer) down_rows_per_peer[q] = x->down_off[q + 1] - x->down_off[q];
    }
    if (n_master_rows) *n_master_rows = (int)x->m_rows.size();
    return DRONE_OK;
}

int drone_xplan_lists(const drone_xplan *x, int *up_rows, int *down_rows) {
    DRONE_REQUIRE(x != nullptr, "drone_xplan_lists: plan is NULL");
    if (up_rows) std::copy(x->up_rows.begin(), x->up_rows.end(), up_rows);
    if (down_rows) std::copy(x->down_rows.begin(), x->down_rows.end(), down_rows);
    return DRONE_OK;
}

int drone_exchange_finish(drone_xplan *x, float *d_rows, int F, int ld, void *stream) {
    DRONE_REQUIRE(x != nullptr, "drone_exchange_finish: NULL plan");
    DRONE_REQUIRE(F >= 1 && F <= x->max_features, "drone_exchange_finish: F=%d outside 1..%d (max_features of the plan)", F,
                  x->max_features);
    DRONE_REQUIRE(ld >= F, "drone_exchange_finish: ld=%d below F=%d", ld, F);
    if (x->nranks == 1) return DRONE_OK;
    DRONE_REQUIRE(d_rows != nullptr || x->n_local == 0, "drone_exchange_finish: rows is NULL");
    if (!x->p2p || !x->p2p->push_pending)
        return set_error(DRONE_E_STATE, "drone_exchange_finish: no aggregation call has sent this plan's mirror rows up "
                         "(drone_spmm_ex with push_up_to on a plan with the peer-memory transport comes first)");
    return exchange_finish_p2p(x, d_rows, F, ld, (cudaStream_t)stream);
}

int drone_exchange_sum(drone_xplan *x, drone_comm *c, float *d_rows, int F, int ld, void *stream) {
    DRONE_REQUIRE(x && c, "drone_exchange_sum: NULL plan or communicator");
    DRONE_REQUIRE(c->nranks == x->nranks && c->rank == x->rank, "drone_exchange_sum: plan is for rank %d/%d, comm is %d/%d",
                  x->rank, x->nranks, c->rank, c->nranks);
    DRONE_REQUIRE(F >= 1 && F <= x->max_features, "drone_exchange_sum: F=%d outside 1..%d (max_features of the plan)", F,
                  x->max_features);
    DRONE_REQUIRE(ld >= F, "drone_exchange_sum: ld=%d below F=%d", ld, F);
    if (x->nranks == 1) return DRONE_OK;
    DRONE_REQUIRE(d_rows != nullptr || x->n_local == 0, "drone_exchange_sum: rows is NULL");
    int rc = xplan_ensure_device(x);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (x->p2p) return exchange_sum_p2p(x, d_rows, F, ld, st);
    const int n_up = (int)x->up_rows.size(), n_down = (int)x->down_rows.size(), n_m = (int)x->m_rows.size();
    // mirrors -> masters
    if (n_up) {
        gather_rows_kernel<<<grid_for((long long)n_up * F), 256, 0, st>>>(d_rows, ld, x->d_up_rows, n_up, F, x->d_send);
        DRONE_LAUNCH_CHECK("gather_rows_kernel");
    }
    if ((rc = all_to_all_v(c, x->d_send, x->up_off, x->d_recv, x->down_off, F, st))) return rc;
    if (n_m) {
        add_at_masters_kernel<<<grid_for((long long)n_m * F), 256, 0, st>>>(d_rows, ld, x->d_m_rows, x->d_m_off,
                                                                          x->d_m_pos, n_m, F, x->d_recv);
        DRONE_LAUNCH_CHECK("add_at_masters_kernel");
    }
    // masters -> mirrors
    if (n_down) {
        gather_rows_kernel<<<grid_for((long long)n_down * F), 256, 0, st>>>(d_rows, ld, x->d_down_rows, n_down, F,
                                                                          x->d_send);
        DRONE_LAUNCH_CHECK("gather_rows_kernel");
    }
    if ((rc = all_to_all_v(c, x->d_send, x->down_off, x->d_recv, x->up_off, F, st))) return rc;
    if (n_up) {
        scatter_rows_kernel<<<grid_for((long long)n_up * F), 256, 0, st>>>(d_rows, ld, x->d_up_rows, n_up, F, x->d_recv);
        DRONE_LAUNCH_CHECK("scatter_rows_kernel");
    }
    return DRONE_OK;
}

// The same exchange among P plans that live in ONE process on ONE device (each part's rows in its own
// buffer): transfers are device-to-device copies instead of NCCL messages.  Lets a single GPU run the
// multi-part logic end to end.
int drone_exchange_sum_local(int n_parts, drone_xplan **plans, float **d_rows, int F, const int *ld, void *stream) {
    DRONE_REQUIRE(n_parts >= 1 && plans && d_rows && ld, "drone_exchange_sum_local: bad arguments");
    cudaStream_t st = (cudaStream_t)stream;
    for (int p = 0; p < n_parts; ++p) {
        DRONE_REQUIRE(plans[p] && plans[p]->nranks == n_parts && plans[p]->rank == p,
                      "drone_exchange_sum_local: plan %d is not rank %d of %d", p, p, n_parts);
        DRONE_REQUIRE(F >= 1 && F <= plans[p]->max_features && ld[p] >= F, "drone_exchange_sum_local: F=%d, ld=%d", F, ld[p]);
        const int rc = xplan_ensure_device(plans[p]);
        if (rc) return rc;
    }
    for (int phase = 0; phase < 2; ++phase) {
        for (int p = 0; p < n_parts; ++p) {
            drone_xplan *x = plans[p];
            const int *list = phase == 0 ? x->d_up_rows : x->d_down_rows;
            const int n = (int)(phase == 0 ? x->up_rows.size() : x->down_rows.size());
            if (n) {
                gather_rows_kernel<<<grid_for((long long)n * F), 256, 0, st>>>(d_rows[p], ld[p], list, n, F, x->d_send);
                DRONE_LAUNCH_CHECK("gather_rows_kernel");
            }
        }
        for (int p = 0; p < n_parts; ++p)
            for (int q = 0; q < n_parts; ++q) {
                if (p == q) continue;
                const std::vector<int> &s_off = phase == 0 ? plans[p]->up_off : plans[p]->down_off;
                const std::vector<int> &r_off = phase == 0 ? plans[q]->down_off : plans[q]->up_off;
                const size_t ns = (size_t)(s_off[q + 1] - s_off[q]), nr = (size_t)(r_off[p + 1] - r_off[p]);
                if (ns != nr)
                    return set_error(DRONE_E_STATE, "exchange plans disagree: part %d sends %zu rows to %d, which expects %zu",
                                     p, ns, q, nr);
                if (ns)
                    DRONE_CUDA(cudaMemcpyAsync(plans[q]->d_recv + (size_t)r_off[p] * F, plans[p]->d_send + (size_t)s_off[q] * F,
                                               sizeof(float) * ns * F, cudaMemcpyDeviceToDevice, st));
            }
        for (int p = 0; p < n_parts; ++p) {
            drone_xplan *x = plans[p];
            if (phase == 0) {
                const int n_m = (int)x->m_rows.size();
                if (n_m) {
                    add_at_masters_kernel<<<grid_for((long long)n_m * F), 256, 0, st>>>(
                        d_rows[p], ld[p], x->d_m_rows, x->d_m_off, x->d_m_pos, n_m, F, x->d_recv);
                    DRONE_LAUNCH_CHECK("add_at_masters_kernel");
                }
            } else {
                const int n = (int)x->up_rows.size();
                if (n) {
                    scatter_rows_kernel<<<grid_for((long long)n * F), 256, 0, st>>>(d_rows[p], ld[p], x->d_up_rows, n, F,
                                                                                 x->d_recv);
                    DRONE_LAUNCH_CHECK("scatter_rows_kernel");
                }
            }
        }
    }
    return DRONE_OK;
}

}  // extern "C"
