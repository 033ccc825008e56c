// Row-gather ceiling of the device: how fast can SMs fetch randomly chosen rows of a dense fp32 table?
// This is the access pattern of the sparse aggregation's X gathers, without the sparse matrix around it.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o baseline/_build/gather_probe baseline/gather_probe.cu
//   baseline/_build/gather_probe
//
// Not part of the library.  Row indices are drawn on the device, either uniformly over the table or with
// R-MAT-like skew (each index bit is 0 with probability `skew`), and read by the gather kernel like CSR columns.
#include <cstdio>
#include <cuda_runtime.h>

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ULL;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
    return x ^ (x >> 31);
}

// indices[i] = a row id, uniform over `rows` or drawn bit by bit (each bit 0 with probability skew16/65536)
__global__ void make_indices(int *indices, long long n, unsigned long long rows, int bits, unsigned skew16) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        unsigned long long h = mix64(0xABCDEFULL + (unsigned long long)i);
        unsigned long long r;
        if (skew16 == 0) {
            r = __umul64hi(h, rows);
        } else {
            r = 0;
            for (int b = 0; b < bits; ++b) {
                h = mix64(h);
                r = (r << 1) | (((unsigned)(h >> 48)) < skew16 ? 0ULL : 1ULL);
            }
        }
        indices[i] = (int)r;
    }
}

// A warp reads 32 indices, then its 32/G lane groups fetch the rows (G float4 each: G = 8 is a 128-byte row,
// G = 16 a 256-byte row), U fetches in flight per lane -- the loop shape of the aggregation's chunk kernel.
template <int G, int U>
__global__ void __launch_bounds__(256) gather_rows(const float4 *__restrict__ table, const int *__restrict__ indices,
                                                   long long n, float4 *sink) {
    constexpr int RPW = 32 / G;
    const int lane = threadIdx.x & 31, gl = lane & (G - 1), gi = lane / G;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long base = warp * 32; base + 32 <= n; base += warps * 32) {
        const int c = indices[base + lane];
#pragma unroll
        for (int t = 0; t < G; t += U) {
            float4 x[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int r = __shfl_sync(0xffffffffu, c, (t + u) * RPW + gi);
                x[u] = __ldg(table + (long long)r * G + gl);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) { acc.x += x[u].x; acc.y += x[u].y; acc.z += x[u].z; acc.w += x[u].w; }
        }
    }
    if (acc.x == 123.456f) sink[0] = acc;
}

template <int G>
static void run(double gigabytes, double skew) {
    const size_t row_bytes = G * 16;
    unsigned long long rows = (unsigned long long)(gigabytes * 1e9 / row_bytes);
    int bits = 0;
    if (skew > 0) {  // power-of-two table for the bitwise draw
        while ((1ULL << (bits + 1)) <= rows) ++bits;
        rows = 1ULL << bits;
    }
    const long long n = 1LL << 26;   // gathers per launch
    float4 *table = nullptr, *sink = nullptr;
    int *indices = nullptr;
    if (cudaMalloc(&table, rows * row_bytes) != cudaSuccess) { printf("allocation of %.2f GB failed\n", gigabytes); return; }
    cudaMalloc(&sink, 16);
    cudaMalloc(&indices, n * sizeof(int));
    cudaMemset(table, 0, rows * row_bytes);
    make_indices<<<148 * 16, 256>>>(indices, n, rows, bits, (unsigned)(skew * 65536));
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    float ms = 0;
    for (int rep = 0; rep < 3; ++rep) {
        cudaEventRecord(e0);
        gather_rows<G, 8><<<148 * 8, 256>>>(table, indices, n, sink);
        cudaEventRecord(e1);
        cudaEventSynchronize(e1);
        cudaEventElapsedTime(&ms, e0, e1);
    }
    printf("row %3zu B  table %7.2f GB  %-8s  %7.3f ms  %6.2f TB/s\n", row_bytes, rows * row_bytes / 1e9,
           skew > 0 ? "skewed" : "uniform", ms, (double)n * row_bytes / ms / 1e9);
    cudaFree(table);
    cudaFree(sink);
    cudaFree(indices);
}

int main() {
    for (double gb : {0.016, 0.067, 0.134, 0.268, 1.0, 8.6, 32.0}) run<16>(gb, 0.0);
    for (double gb : {0.016, 0.067, 0.134, 0.268, 1.0, 8.6, 32.0}) run<8>(gb, 0.0);
    for (double skew : {0.60, 0.70, 0.76}) { printf("skew %.2f: ", skew); run<16>(0.2685, skew); }
    for (double skew : {0.60, 0.70, 0.76}) { printf("skew %.2f: ", skew); run<8>(8.59, skew); }
    printf("status: %s\n", cudaGetErrorString(cudaGetLastError()));
    return 0;
}
