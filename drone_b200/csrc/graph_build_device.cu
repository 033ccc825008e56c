// One rank's local graph built on the device from its edge list: the numbering and CSR of build_graph
// (cuda_gcn/src/cuda/graph.cu:54-103; twin DRONE/src/cuda/graph.cu), which the reference builds with serial host
// loops over pinned memory.
//
//   local ids   = first-seen order over u0, v0, u1, v1, ...: every vertex takes the smallest position at which it
//                 occurs (atomicMin), the vertices that occur are sorted by that position, the rank is the local id;
//   CSR         = edges sorted by the local id of their source, stably (destinations keep edge-list order), row
//                 pointers from a histogram and a scan.
// Output is identical to drone_graph_build_host.  CUB does the two sorts and the scans.
#include "common.cuh"

#include <cub/cub.cuh>

namespace drone {

static inline int grid_gb(long long n) {
    long long g = (n + 255) / 256;
    if (g < 1) g = 1;
    if (g > 148 * 32) g = 148 * 32;
    return (int)g;
}

__global__ void gb_fill_kernel(int *a, long long n, int value) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) a[i] = value;
}

// first[x] = smallest position 2i (as source) or 2i+1 (as destination); *bad set when an id is out of range
__global__ void gb_first_seen_kernel(const int *__restrict__ u, const int *__restrict__ v, int n_edges, int global_v,
                                     unsigned *first, int *bad) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_edges; i += (long long)gridDim.x * blockDim.x) {
        const int a = u[i], b = v[i];
        if (a < 0 || a >= global_v || b < 0 || b >= global_v) {
            *bad = 1;
            continue;
        }
        atomicMin(first + a, (unsigned)(2 * i));
        atomicMin(first + b, (unsigned)(2 * i + 1));
    }
}

__global__ void gb_flag_present_kernel(const unsigned *__restrict__ first, int global_v, int *flag) {
    for (long long x = blockIdx.x * (long long)blockDim.x + threadIdx.x; x <= global_v; x += (long long)gridDim.x * blockDim.x)
        flag[x] = (x < global_v && first[x] != 0xffffffffu) ? 1 : 0;
}

// the vertices that occur, compacted in id order: keys = first position, vals = vertex id
__global__ void gb_compact_kernel(const unsigned *__restrict__ first, const int *__restrict__ slot, int global_v,
                                  unsigned *keys, int *vals) {
    for (long long x = blockIdx.x * (long long)blockDim.x + threadIdx.x; x < global_v; x += (long long)gridDim.x * blockDim.x)
        if (first[x] != 0xffffffffu) {
            keys[slot[x]] = first[x];
            vals[slot[x]] = (int)x;
        }
}

__global__ void gb_number_kernel(const int *__restrict__ l2g, int n_local, int *g2l) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_local; i += (long long)gridDim.x * blockDim.x)
        g2l[l2g[i]] = (int)i;
}

__global__ void gb_local_edges_kernel(const int *__restrict__ u, const int *__restrict__ v, int n_edges,
                                      const int *__restrict__ g2l, int *lu, int *lv, int *degree) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_edges; i += (long long)gridDim.x * blockDim.x) {
        const int a = g2l[u[i]];
        lu[i] = a;
        lv[i] = g2l[v[i]];
        atomicAdd(degree + a, 1);
    }
}

struct Scratch {
    void *p[10] = {nullptr};
    ~Scratch() { for (void *q : p) cudaFree(q); }
};

}  // namespace drone

using namespace drone;

extern "C" int drone_graph_build_device(int global_v, int n_edges, const int *d_u, const int *d_v, int *d_g2l, int *d_l2g,
                                        int *d_index, int *d_dst, int *n_local_out, void *stream) {
    DRONE_REQUIRE(global_v > 0 && n_edges >= 0, "drone_graph_build_device: bad sizes (V=%d, E=%d)", global_v, n_edges);
    DRONE_REQUIRE(n_edges < (1 << 30), "drone_graph_build_device: %d edges, the position encoding holds 2^30 - 1", n_edges);
    DRONE_REQUIRE(d_g2l && d_l2g && d_index && n_local_out, "drone_graph_build_device: NULL output");
    DRONE_REQUIRE(n_edges == 0 || (d_u && d_v && d_dst), "drone_graph_build_device: NULL edge arrays");
    cudaStream_t st = (cudaStream_t)stream;
    Scratch s;
    unsigned *first = nullptr, *keys = nullptr, *keys_out = nullptr;
    int *flag = nullptr, *slot = nullptr, *vals = nullptr, *bad = nullptr, *lu = nullptr, *lv = nullptr, *lu_out = nullptr;
    DRONE_CUDA(cudaMalloc(&s.p[0], sizeof(unsigned) * (size_t)global_v));
    DRONE_CUDA(cudaMalloc(&s.p[1], sizeof(int) * ((size_t)global_v + 1)));
    DRONE_CUDA(cudaMalloc(&s.p[2], sizeof(int) * ((size_t)global_v + 1)));
    DRONE_CUDA(cudaMalloc(&s.p[3], sizeof(int)));
    first = (unsigned *)s.p[0]; flag = (int *)s.p[1]; slot = (int *)s.p[2]; bad = (int *)s.p[3];
    DRONE_CUDA(cudaMemsetAsync(first, 0xff, sizeof(unsigned) * (size_t)global_v, st));
    DRONE_CUDA(cudaMemsetAsync(bad, 0, sizeof(int), st));
    if (n_edges > 0) {
        gb_first_seen_kernel<<<grid_gb(n_edges), 256, 0, st>>>(d_u, d_v, n_edges, global_v, first, bad);
        DRONE_LAUNCH_CHECK("gb_first_seen_kernel");
    }
    gb_flag_present_kernel<<<grid_gb((long long)global_v + 1), 256, 0, st>>>(first, global_v, flag);
    DRONE_LAUNCH_CHECK("gb_flag_present_kernel");
    size_t tmp_bytes = 0, need = 0;
    DRONE_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, flag, slot, global_v + 1, st));
    const int cap = (int)std::min<long long>(global_v, 2LL * n_edges);
    need = tmp_bytes;
    DRONE_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, keys, keys_out, vals, d_l2g, cap > 0 ? cap : 1, 0, 32, st));
    need = std::max(need, tmp_bytes);
    DRONE_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, lu, lu_out, lv, d_dst, n_edges > 0 ? n_edges : 1, 0, 32, st));
    need = std::max(need, tmp_bytes);
    DRONE_CUDA(cudaMalloc(&s.p[4], need > 0 ? need : 1));
    void *tmp = s.p[4];
    tmp_bytes = need;
    DRONE_CUDA(cub::DeviceScan::ExclusiveSum(tmp, tmp_bytes, flag, slot, global_v + 1, st));
    count_launch();
    int n_local = 0, h_bad = 0;
    DRONE_CUDA(cudaMemcpyAsync(&n_local, slot + global_v, sizeof(int), cudaMemcpyDeviceToHost, st));
    DRONE_CUDA(cudaMemcpyAsync(&h_bad, bad, sizeof(int), cudaMemcpyDeviceToHost, st));
    DRONE_CUDA(cudaStreamSynchronize(st));
    if (h_bad) return set_error(DRONE_E_INVALID, "drone_graph_build_device: an edge names a vertex outside 0..%d", global_v - 1);
    *n_local_out = n_local;
    gb_fill_kernel<<<grid_gb(global_v), 256, 0, st>>>(d_g2l, global_v, -1);
    DRONE_LAUNCH_CHECK("gb_fill_kernel");
    DRONE_CUDA(cudaMemsetAsync(d_index, 0, sizeof(int) * ((size_t)n_local + 1), st));
    if (n_local == 0) {
        DRONE_CUDA(cudaStreamSynchronize(st));
        return DRONE_OK;
    }
    // local ids: the vertices that occur, ordered by where they occur first
    DRONE_CUDA(cudaMalloc(&s.p[5], sizeof(unsigned) * (size_t)n_local));
    DRONE_CUDA(cudaMalloc(&s.p[6], sizeof(unsigned) * (size_t)n_local));
    DRONE_CUDA(cudaMalloc(&s.p[7], sizeof(int) * (size_t)n_local));
    keys = (unsigned *)s.p[5]; keys_out = (unsigned *)s.p[6]; vals = (int *)s.p[7];
    gb_compact_kernel<<<grid_gb(global_v), 256, 0, st>>>(first, slot, global_v, keys, vals);
    DRONE_LAUNCH_CHECK("gb_compact_kernel");
    int end_bit = 1;
    while (end_bit < 32 && (1LL << end_bit) < 2LL * n_edges) ++end_bit;
    tmp_bytes = need;
    DRONE_CUDA(cub::DeviceRadixSort::SortPairs(tmp, tmp_bytes, keys, keys_out, vals, d_l2g, n_local, 0, end_bit, st));
    count_launch();
    gb_number_kernel<<<grid_gb(n_local), 256, 0, st>>>(d_l2g, n_local, d_g2l);
    DRONE_LAUNCH_CHECK("gb_number_kernel");
    // CSR by source, destinations in edge-list order: stable sort of the edges by local source id
    cudaFree(s.p[5]); cudaFree(s.p[6]); cudaFree(s.p[7]);
    s.p[5] = s.p[6] = s.p[7] = nullptr;
    DRONE_CUDA(cudaMalloc(&s.p[5], sizeof(int) * (size_t)n_edges));
    DRONE_CUDA(cudaMalloc(&s.p[6], sizeof(int) * (size_t)n_edges));
    DRONE_CUDA(cudaMalloc(&s.p[7], sizeof(int) * (size_t)n_edges));
    DRONE_CUDA(cudaMalloc(&s.p[8], sizeof(int) * ((size_t)n_local + 1)));
    lu = (int *)s.p[5]; lv = (int *)s.p[6]; lu_out = (int *)s.p[7];
    int *degree = (int *)s.p[8];
    DRONE_CUDA(cudaMemsetAsync(degree, 0, sizeof(int) * ((size_t)n_local + 1), st));
    gb_local_edges_kernel<<<grid_gb(n_edges), 256, 0, st>>>(d_u, d_v, n_edges, d_g2l, lu, lv, degree);
    DRONE_LAUNCH_CHECK("gb_local_edges_kernel");
    tmp_bytes = need;
    DRONE_CUDA(cub::DeviceScan::ExclusiveSum(tmp, tmp_bytes, degree, d_index, n_local + 1, st));
    count_launch();
    end_bit = 1;
    while (end_bit < 31 && (1LL << end_bit) < (long long)n_local) ++end_bit;
    tmp_bytes = need;
    DRONE_CUDA(cub::DeviceRadixSort::SortPairs(tmp, tmp_bytes, lu, lu_out, lv, d_dst, n_edges, 0, end_bit, st));
    count_launch();
    DRONE_CUDA(cudaStreamSynchronize(st));
    return DRONE_OK;
}
