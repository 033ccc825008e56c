// Shared host-side helpers of the library: status codes, the per-thread error
// message, CUDA call checking and the launch counter.
#pragma once

#include <cuda_runtime.h>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/drone_b200.h"

namespace drone {

// Message of the last failing call on this thread; read by drone_last_error().
char *last_error_buffer();

int set_error(int code, const char *fmt, ...);

extern std::atomic<long long> g_kernel_launches;

inline void count_launch(int n = 1) { g_kernel_launches.fetch_add(n, std::memory_order_relaxed); }

inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Device-side check of a CSR given by the caller (defined with the plan builder): DRONE_E_INVALID naming the first
// bad row pointer or column, DRONE_OK for a well-formed input.  Synchronises `st`.
int validate_csr(const char *who, const int *d_index, const int *d_col, int n_rows, int n_cols, int nnz, cudaStream_t st);

#ifdef __CUDACC__
// (row, column) of a flat element index over rows of `width` elements that advances by a fixed stride: two divisions
// when a thread starts, none per element (a 64-bit division costs more instructions than the copy it indexes).
struct RowColumn {
    int row, col, d_row, d_col, width;
    __device__ RowColumn(long long first, long long stride, int w) : width(w) {
        row = (int)(first / w);
        col = (int)(first - (long long)row * w);
        d_row = (int)(stride / w);
        d_col = (int)(stride - (long long)d_row * w);
    }
    __device__ void advance() {
        row += d_row;
        col += d_col;
        if (col >= width) { col -= width; ++row; }
    }
};
#endif

}  // namespace drone

// Evaluate a CUDA runtime call; on failure record the message and return DRONE_E_CUDA
// from the enclosing function.
#define DRONE_CUDA(call)                                                              \
    do {                                                                              \
        cudaError_t err__ = (call);                                                   \
        if (err__ != cudaSuccess)                                                     \
            return drone::set_error(DRONE_E_CUDA, "%s failed at %s:%d: %s", #call,    \
                                    __FILE__, __LINE__, cudaGetErrorString(err__));   \
    } while (0)

// After a kernel launch: pick up launch-configuration errors without synchronising.
#define DRONE_LAUNCH_CHECK(name)                                                      \
    do {                                                                              \
        cudaError_t err__ = cudaGetLastError();                                       \
        if (err__ != cudaSuccess)                                                     \
            return drone::set_error(DRONE_E_CUDA, "launch of %s failed at %s:%d: %s", \
                                    name, __FILE__, __LINE__,                         \
                                    cudaGetErrorString(err__));                       \
        drone::count_launch();                                                        \
    } while (0)

#define DRONE_REQUIRE(cond, ...)                                       \
    do {                                                               \
        if (!(cond)) return drone::set_error(DRONE_E_INVALID, __VA_ARGS__); \
    } while (0)
