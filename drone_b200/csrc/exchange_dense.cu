// Mirror/master exchange as two dense collectives: reduce-scatter + all-gather over the boundary.
//
// All vertices held by more than one part (the boundary) are listed once, grouped by the part that owns their
// master copy and ascending by global id inside a group; every group is padded to the size of the largest, so the
// list is nranks equal blocks.  A call then is
//     fill:   boundary[pos(v), :] = my row of v for the boundary vertices I hold, 0 elsewhere
//     ncclReduceScatter(sum): block p of the element-wise sum lands on rank p  (mirror -> master, summed)
//     ncclAllGather:          every rank receives all blocks                   (master -> mirror)
//     take:   my row of v = boundary[pos(v), :] for the boundary vertices I hold
// Compared with the point-to-point form (exchange.cu) it moves rows of vertices a rank does not hold, which costs
// bytes when replication is sparse, but it is two library collectives that NVSwitch can reduce in the fabric.
// The summation order inside ncclReduceScatter is NCCL's, so results may differ from the other transports in the
// last bit (they are still the same on every replica).
#include "exchange.cuh"

#include <algorithm>
#include <new>

struct drone_dense_xplan {
    int rank = 0, nranks = 1, n_local = 0, max_features = 0;
    int block_rows = 0;                 // rows per owner block (largest group)
    std::vector<int> rows, pos;         // my boundary rows (local id) and their position in the boundary list
    int device = -1;
    int *d_rows = nullptr, *d_pos = nullptr;
    float *d_boundary = nullptr;        // [nranks * block_rows, max_features]
    float *d_block = nullptr;           // [block_rows, max_features] my reduced block
};

namespace drone {

// boundary[pos[i], :] = rows[list[i], :]   (the buffer was zeroed before)
__global__ void dense_fill_kernel(const float *__restrict__ rows, long long ld, const int *__restrict__ list,
                                  const int *__restrict__ pos, int n, int F, float *__restrict__ boundary) {
    const long long total = (long long)n * F;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / F), j = (int)(i - (long long)r * F);
        boundary[(long long)pos[r] * F + j] = rows[(long long)list[r] * ld + j];
    }
}

// rows[list[i], :] = boundary[pos[i], :]
__global__ void dense_take_kernel(float *__restrict__ rows, long long ld, const int *__restrict__ list,
                                  const int *__restrict__ pos, int n, int F, const float *__restrict__ boundary) {
    const long long total = (long long)n * F;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / F), j = (int)(i - (long long)r * F);
        rows[(long long)list[r] * ld + j] = boundary[(long long)pos[r] * F + j];
    }
}

static inline int dense_grid(long long n) {
    long long g = (n + 255) / 256;
    if (g < 1) g = 1;
    if (g > 148 * 16) g = 148 * 16;
    return (int)g;
}

}  // namespace drone

using namespace drone;

extern "C" {

int drone_dense_xplan_destroy(drone_dense_xplan *x);

int drone_dense_xplan_create(drone_dense_xplan **out, int rank, int nranks, int n_local, const int *h_local2global,
                             int global_v, const int *h_owner, const int *h_replicas, int max_features) {
    DRONE_REQUIRE(out != nullptr, "drone_dense_xplan_create: out is NULL");
    *out = nullptr;
    DRONE_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, "drone_dense_xplan_create: rank %d of %d", rank, nranks);
    DRONE_REQUIRE(n_local >= 0 && global_v > 0 && max_features >= 1, "drone_dense_xplan_create: bad sizes");
    DRONE_REQUIRE(h_owner && h_replicas && (n_local == 0 || h_local2global), "drone_dense_xplan_create: NULL table");
    drone_dense_xplan *x = new (std::nothrow) drone_dense_xplan();
    if (!x) return set_error(DRONE_E_INVALID, "drone_dense_xplan_create: out of host memory");
    x->rank = rank;
    x->nranks = nranks;
    x->n_local = n_local;
    x->max_features = max_features;
    // position of every boundary vertex inside its owner's group (ascending global id)
    std::vector<int> count(nranks, 0), index_in_group((size_t)global_v, -1);
    for (int v = 0; v < global_v; ++v)
        if (h_replicas[v] > 1) {
            const int o = h_owner[v];
            if (o < 0 || o >= nranks) {
                delete x;
                return set_error(DRONE_E_INVALID, "drone_dense_xplan_create: vertex %d has owner %d", v, o);
            }
            index_in_group[v] = count[o]++;
        }
    x->block_rows = std::max(1, *std::max_element(count.begin(), count.end()));
    for (int r = 0; r < n_local; ++r) {
        const int v = h_local2global[r];
        if (v < 0 || v >= global_v) {
            delete x;
            return set_error(DRONE_E_INVALID, "drone_dense_xplan_create: local row %d has global id %d", r, v);
        }
        if (h_replicas[v] > 1) {
            x->rows.push_back(r);
            x->pos.push_back(h_owner[v] * x->block_rows + index_in_group[v]);
        }
    }
    *out = x;
    return DRONE_OK;
}

int drone_dense_xplan_destroy(drone_dense_xplan *x) {
    if (!x) return DRONE_OK;
    if (x->device >= 0) {
        int prev = -1;
        cudaGetDevice(&prev);
        cudaSetDevice(x->device);
        cudaFree(x->d_rows); cudaFree(x->d_pos); cudaFree(x->d_boundary); cudaFree(x->d_block);
        if (prev >= 0) cudaSetDevice(prev);
    }
    delete x;
    return DRONE_OK;
}

// bytes one rank puts on the wire per call and feature: (nranks-1)/nranks of the boundary, twice
long long drone_dense_xplan_boundary_rows(const drone_dense_xplan *x) {
    return x ? (long long)x->nranks * x->block_rows : 0;
}

int drone_exchange_sum_dense(drone_dense_xplan *x, drone_comm *c, float *d_rows, int F, int ld, void *stream) {
    DRONE_REQUIRE(x && c, "drone_exchange_sum_dense: NULL plan or communicator");
    DRONE_REQUIRE(c->nranks == x->nranks && c->rank == x->rank, "drone_exchange_sum_dense: plan is rank %d/%d, comm %d/%d",
                  x->rank, x->nranks, c->rank, c->nranks);
    DRONE_REQUIRE(F >= 1 && F <= x->max_features && ld >= F, "drone_exchange_sum_dense: F=%d (max %d), ld=%d", F,
                  x->max_features, ld);
    if (x->nranks == 1) return DRONE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (x->device < 0) {
        DRONE_CUDA(cudaGetDevice(&x->device));
        const size_t n = x->rows.size();
        DRONE_CUDA(cudaMalloc(&x->d_rows, sizeof(int) * std::max<size_t>(n, 1)));
        DRONE_CUDA(cudaMalloc(&x->d_pos, sizeof(int) * std::max<size_t>(n, 1)));
        if (n) {
            DRONE_CUDA(cudaMemcpy(x->d_rows, x->rows.data(), sizeof(int) * n, cudaMemcpyHostToDevice));
            DRONE_CUDA(cudaMemcpy(x->d_pos, x->pos.data(), sizeof(int) * n, cudaMemcpyHostToDevice));
        }
        const size_t block = (size_t)x->block_rows * x->max_features;
        DRONE_CUDA(cudaMalloc(&x->d_boundary, sizeof(float) * block * x->nranks));
        DRONE_CUDA(cudaMalloc(&x->d_block, sizeof(float) * block));
    }
    const int n = (int)x->rows.size();
    const size_t block_elems = (size_t)x->block_rows * F;
    DRONE_CUDA(cudaMemsetAsync(x->d_boundary, 0, sizeof(float) * block_elems * x->nranks, st));
    if (n) {
        dense_fill_kernel<<<dense_grid((long long)n * F), 256, 0, st>>>(d_rows, ld, x->d_rows, x->d_pos, n, F, x->d_boundary);
        DRONE_LAUNCH_CHECK("dense_fill_kernel");
    }
    DRONE_NCCL(ncclReduceScatter(x->d_boundary, x->d_block, block_elems, ncclFloat, ncclSum, c->comm, st));
    DRONE_NCCL(ncclAllGather(x->d_block, x->d_boundary, block_elems, ncclFloat, c->comm, st));
    if (n) {
        dense_take_kernel<<<dense_grid((long long)n * F), 256, 0, st>>>(d_rows, ld, x->d_rows, x->d_pos, n, F, x->d_boundary);
        DRONE_LAUNCH_CHECK("dense_take_kernel");
    }
    return DRONE_OK;
}

}  // extern "C"
