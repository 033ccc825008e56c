// Sparse aggregation kernels:  Y[r,:] = sum_k val[k] * X[col[k],:]  over CSR rows.
//
// The work of one call is split three ways, all decided when the plan was built:
//   1. short rows (at most short_row_limit nonzeros) are stored once more as one
//      contiguous stream with end-of-row flags; a lane group walks about 64
//      entries of it (whole rows), adding a row's nonzeros in CSR order into one
//      accumulator and writing the row at its last entry, so the per-row cost
//      is one store and no warp is spent on a row of two nonzeros;
//   2. long rows: cut into chunks of chunk_nnz nonzeros, one warp per chunk with
//      its 32/G lane groups taking interleaved nonzeros; a row that is a single
//      chunk is written directly, otherwise the chunk sum goes to a partial slot;
//   3. split rows: the partial slots of a row are added in slot order.
// A lane group is G lanes that together hold one dense row: each lane owns VPL
// vectors of VEC floats (float4 when the operands allow 16-byte accesses).
// No atomics are used, so the summation order is fixed by the plan.
//
// The CSR streams (col, val) and the output are touched once and use streaming
// cache hints so that L2 capacity is left to the gathered rows of X.
#include "plan.cuh"

#include <algorithm>
#include <cstdlib>
#include <mutex>

namespace drone {

// L2 cache policies.  Rows of X are gathered many times and should stay resident; the CSR
// streams, the chunk list and the output pass through once and should be the first to go.
__device__ __forceinline__ unsigned long long l2_policy_keep() {
    unsigned long long p;
    asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ unsigned long long l2_policy_stream() {
    unsigned long long p;
    asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ float4 ld_keep(const float4 *ptr, unsigned long long pol) {
    float4 v;
    asm("ld.global.nc.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;"
        : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(ptr), "l"(pol));
    return v;
}
__device__ __forceinline__ float ld_keep(const float *ptr, unsigned long long pol) {
    float v;
    asm("ld.global.nc.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(ptr), "l"(pol));
    return v;
}
__device__ __forceinline__ int ld_stream(const int *ptr, unsigned long long pol) {
    int v;
    asm("ld.global.nc.L1::no_allocate.L2::cache_hint.s32 %0, [%1], %2;" : "=r"(v) : "l"(ptr), "l"(pol));
    return v;
}
__device__ __forceinline__ float ld_stream(const float *ptr, unsigned long long pol) {
    float v;
    asm("ld.global.nc.L1::no_allocate.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(ptr), "l"(pol));
    return v;
}
__device__ __forceinline__ void st_stream(float4 *ptr, const float4 &v, unsigned long long pol) {
    asm volatile("st.global.L2::cache_hint.v4.f32 [%0], {%1,%2,%3,%4}, %5;"
                 :: "l"(ptr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "l"(pol) : "memory");
}
__device__ __forceinline__ void st_stream(float *ptr, const float &v, unsigned long long pol) {
    asm volatile("st.global.L2::cache_hint.f32 [%0], %1, %2;" :: "l"(ptr), "f"(v), "l"(pol) : "memory");
}

template <int VEC> struct Vec;
template <> struct Vec<4> {
    using type = float4;
    static __device__ __forceinline__ float4 zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
    static __device__ __forceinline__ void fma(float4 &a, float v, const float4 &x) {
        a.x = fmaf(v, x.x, a.x);
        a.y = fmaf(v, x.y, a.y);
        a.z = fmaf(v, x.z, a.z);
        a.w = fmaf(v, x.w, a.w);
    }
    static __device__ __forceinline__ void add(float4 &a, const float4 &x) {
        a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
    }
    static __device__ __forceinline__ float4 shfl_xor(const float4 &a, int o) {
        return make_float4(__shfl_xor_sync(0xffffffffu, a.x, o), __shfl_xor_sync(0xffffffffu, a.y, o),
                           __shfl_xor_sync(0xffffffffu, a.z, o), __shfl_xor_sync(0xffffffffu, a.w, o));
    }
};
template <> struct Vec<1> {
    using type = float;
    static __device__ __forceinline__ float zero() { return 0.f; }
    static __device__ __forceinline__ void fma(float &a, float v, const float &x) { a = fmaf(v, x, a); }
    static __device__ __forceinline__ void add(float &a, const float &x) { a += x; }
    static __device__ __forceinline__ float shfl_xor(const float &a, int o) {
        return __shfl_xor_sync(0xffffffffu, a, o);
    }
};

template <int A, int B> struct MinOf { static constexpr int value = A < B ? A : B; };

// ---------------------------------------------------------------------------
// 1. short rows: one lane group walks a range of the short-row stream
//    (about kShortRangeNnz entries, whole rows only) and writes each row when
//    its last entry has been added.  Entries of a row are added in CSR order
//    into one accumulator.
// ---------------------------------------------------------------------------
template <int G, int VPL, int VEC, int U, bool EXACT>
__global__ void __launch_bounds__(256)
spmm_short_stream_kernel(const int *__restrict__ s_range_row, int n_ranges, const int *__restrict__ s_rowptr,
                         const int *__restrict__ s_rows, const int *__restrict__ s_col,
                         const float *__restrict__ s_val, const float *__restrict__ X, long long ldv,
                         float *__restrict__ Y, long long ldy, int nvec) {
    using V = typename Vec<VEC>::type;
    constexpr int RPW = 32 / G;
    constexpr int UU = MinOf<U, G>::value;
    const int lane = threadIdx.x & 31;
    const int gl = lane & (G - 1);
    const int gi = lane / G;
    const long long range = ((blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5) * RPW + gi;
    int ri = 0, k = 0, kend = 0;
    if (range < n_ranges) {
        ri = s_range_row[range];
        const int ri_end = s_range_row[range + 1];
        k = s_rowptr[ri];
        kend = s_rowptr[ri_end];
    }
    int maxlen = kend - k;
#pragma unroll
    for (int o = G; o < 32; o <<= 1) maxlen = max(maxlen, __shfl_xor_sync(0xffffffffu, maxlen, o));

    const V *xb = reinterpret_cast<const V *>(X) + gl;
    const unsigned long long pol_keep = l2_policy_keep(), pol_stream = l2_policy_stream();
    V acc[VPL];
#pragma unroll
    for (int p = 0; p < VPL; ++p) acc[p] = Vec<VEC>::zero();

    unsigned c_next = 0;
    float v_next = 0.f;
    if (k + gl < kend) {
        c_next = (unsigned)ld_stream(s_col + k + gl, pol_stream);
        v_next = ld_stream(s_val + k + gl, pol_stream);
    }
    for (int base = 0; base < maxlen; base += G) {
        const unsigned c = c_next;
        const float v = v_next;
        c_next = 0;
        v_next = 0.f;
        if (k + base + G + gl < kend) {   // next batch, requested before this batch's gathers
            c_next = (unsigned)ld_stream(s_col + k + base + G + gl, pol_stream);
            v_next = ld_stream(s_val + k + base + G + gl, pol_stream);
        }
        const int lim = min(G, maxlen - base);
        for (int j = 0; j < lim; j += UU) {
            unsigned cc[UU];
            float vv[UU];
            V x[UU][VPL];
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                cc[u] = __shfl_sync(0xffffffffu, c, j + u, G);
                vv[u] = __shfl_sync(0xffffffffu, v, j + u, G);
            }
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                const bool live = (k + base + j + u < kend) && !(cc[u] & kPlaceholder);
                const V *xr = xb + (long long)(cc[u] & kColMask) * ldv;
#pragma unroll
                for (int p = 0; p < VPL; ++p)
                    x[u][p] = (live && (EXACT || gl + p * G < nvec)) ? ld_keep(xr + p * G, pol_keep) : Vec<VEC>::zero();
            }
#pragma unroll
            for (int u = 0; u < UU; ++u) {
#pragma unroll
                for (int p = 0; p < VPL; ++p) Vec<VEC>::fma(acc[p], vv[u], x[u][p]);
                if ((cc[u] & kLastInRow) && (k + base + j + u < kend)) {
                    V *yr = reinterpret_cast<V *>(Y + (long long)s_rows[ri] * ldy) + gl;
#pragma unroll
                    for (int p = 0; p < VPL; ++p) {
                        if (EXACT || gl + p * G < nvec) st_stream(yr + p * G, acc[p], pol_stream);
                        acc[p] = Vec<VEC>::zero();
                    }
                    ++ri;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// 2. chunks of long rows: one warp per chunk.  The warp loads 32 (col, val)
//    pairs at a time; its 32/G lane groups take interleaved entries.
// ---------------------------------------------------------------------------
template <int G, int VPL, int VEC, int U, bool EXACT>
__global__ void __launch_bounds__(256)
spmm_chunks_kernel(const Chunk *__restrict__ chunks, int n_chunks, const int *__restrict__ col,
                   const float *__restrict__ val, const float *__restrict__ X, long long ldv,
                   float *__restrict__ Y, long long ldy, float *__restrict__ partials, int nvec) {
    using V = typename Vec<VEC>::type;
    constexpr int RPW = 32 / G;
    constexpr int UU = MinOf<U, G>::value;
    const int lane = threadIdx.x & 31;
    const int gl = lane & (G - 1);
    const int gi = lane / G;
    const long long first_warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long all_warps = ((long long)gridDim.x * blockDim.x) >> 5;
    const V *xb = reinterpret_cast<const V *>(X) + gl;
    const unsigned long long pol_keep = l2_policy_keep(), pol_stream = l2_policy_stream();

    // one chunk per warp when the grid covers the list, several (strided) when the launch is a resident grid
    for (long long warp = first_warp; warp < n_chunks; warp += all_warps) {
    const int4 raw = __ldg(reinterpret_cast<const int4 *>(chunks) + warp);
    const int row = raw.x, k0 = raw.y, len = raw.z, slot = raw.w;

    V acc[VPL];
#pragma unroll
    for (int p = 0; p < VPL; ++p) acc[p] = Vec<VEC>::zero();

    // (col, val) of the next batch are requested before the gathers of the current one are issued, so the
    // dependent chain col -> X row costs one memory latency per batch instead of two
    int c = 0;
    float v = 0.f;
    if (lane < len) {
        c = ld_stream(col + k0 + lane, pol_stream);
        v = ld_stream(val + k0 + lane, pol_stream);
    }
    int base = 0;
    // full batches of 32 entries: no bounds checks
    for (; base + 32 <= len; base += 32) {
        int c_next = 0;
        float v_next = 0.f;
        if (base + 32 + lane < len) {
            c_next = ld_stream(col + k0 + base + 32 + lane, pol_stream);
            v_next = ld_stream(val + k0 + base + 32 + lane, pol_stream);
        }
#pragma unroll
        for (int t = 0; t < G; t += UU) {
            int cc[UU];
            float vv[UU];
            V x[UU][VPL];
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                cc[u] = __shfl_sync(0xffffffffu, c, (t + u) * RPW + gi);
                vv[u] = __shfl_sync(0xffffffffu, v, (t + u) * RPW + gi);
            }
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                const V *xr = xb + (long long)cc[u] * ldv;
#pragma unroll
                for (int p = 0; p < VPL; ++p)
                    x[u][p] = (EXACT || gl + p * G < nvec) ? ld_keep(xr + p * G, pol_keep) : Vec<VEC>::zero();
            }
#pragma unroll
            for (int u = 0; u < UU; ++u)
#pragma unroll
                for (int p = 0; p < VPL; ++p) Vec<VEC>::fma(acc[p], vv[u], x[u][p]);
        }
        c = c_next;
        v = v_next;
    }
    // last, partial batch (entries beyond the chunk were loaded as zeros)
    if (base < len) {
        const int cnt = len - base;
        const int steps = (cnt + RPW - 1) / RPW;  // <= G
        for (int t = 0; t < steps; t += UU) {
            int cc[UU];
            float vv[UU];
            V x[UU][VPL];
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                const int e = (t + u) * RPW + gi;
                cc[u] = __shfl_sync(0xffffffffu, c, e & 31);
                vv[u] = __shfl_sync(0xffffffffu, v, e & 31);
                if (e >= cnt) vv[u] = 0.f;
            }
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                const bool live = (t + u) * RPW + gi < cnt;
                const V *xr = xb + (long long)cc[u] * ldv;
#pragma unroll
                for (int p = 0; p < VPL; ++p)
                    x[u][p] = (live && (EXACT || gl + p * G < nvec)) ? ld_keep(xr + p * G, pol_keep) : Vec<VEC>::zero();
            }
#pragma unroll
            for (int u = 0; u < UU; ++u)
#pragma unroll
                for (int p = 0; p < VPL; ++p) Vec<VEC>::fma(acc[p], vv[u], x[u][p]);
        }
    }
    // combine the lane groups (butterfly: every lane ends with the same total)
#pragma unroll
    for (int o = G; o < 32; o <<= 1)
#pragma unroll
        for (int p = 0; p < VPL; ++p) Vec<VEC>::add(acc[p], Vec<VEC>::shfl_xor(acc[p], o));

    if (gi == 0) {
        V *out = (slot < 0 ? reinterpret_cast<V *>(Y + (long long)row * ldy)
                           : reinterpret_cast<V *>(partials + (long long)slot * nvec * VEC)) + gl;
#pragma unroll
        for (int p = 0; p < VPL; ++p)
            if (EXACT || gl + p * G < nvec) {
                if (slot < 0) st_stream(out + p * G, acc[p], pol_stream); else out[p * G] = acc[p];
            }
    }
    }  // chunks of this warp
}

// ---------------------------------------------------------------------------
// 3. split rows: add the partial slots of a row in slot order.
//    WIDE = false: one warp per split row (eight rows per block), its lane groups take interleaved slots; rows
//    with more than max_slots slots are left to the wide launch.
//    WIDE = true: one block per entry of the plan's list of wide rows, all eight warps share the row and their
//    sums are added in warp order through shared memory.
// ---------------------------------------------------------------------------
template <int G, int VPL, int VEC, bool WIDE>
__global__ void __launch_bounds__(256)
spmm_reduce_partials_kernel(const SplitRow *__restrict__ split, int n_split,
                            const float *__restrict__ partials, float *__restrict__ Y, long long ldy,
                            int nvec, int max_slots) {
    using V = typename Vec<VEC>::type;
    constexpr int RPW = 32 / G;
    extern __shared__ float smem[];  // [8][nvec*VEC] for the wide launch
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    const int gl = lane & (G - 1);
    const int gi = lane / G;
    const long long entry = WIDE ? (long long)blockIdx.x : (long long)blockIdx.x * 8 + w;
    if (entry >= n_split) return;
    const int4 raw = __ldg(reinterpret_cast<const int4 *>(split) + entry);
    const int row = raw.x, slot0 = raw.y, nslots = raw.z;
    if (!WIDE && nslots > max_slots) return;

    V acc[VPL];
#pragma unroll
    for (int p = 0; p < VPL; ++p) acc[p] = Vec<VEC>::zero();
    const int first = WIDE ? w * RPW + gi : gi;
    const int stride = WIDE ? 8 * RPW : RPW;
    for (int sidx = first; sidx < nslots; sidx += stride) {
        const V *pr = reinterpret_cast<const V *>(partials + (long long)(slot0 + sidx) * nvec * VEC);
#pragma unroll
        for (int p = 0; p < VPL; ++p) {
            const int vi = gl + p * G;
            if (vi < nvec) Vec<VEC>::add(acc[p], pr[vi]);
        }
    }
#pragma unroll
    for (int o = G; o < 32; o <<= 1)
#pragma unroll
        for (int p = 0; p < VPL; ++p) Vec<VEC>::add(acc[p], Vec<VEC>::shfl_xor(acc[p], o));

    V *yr = reinterpret_cast<V *>(Y + (long long)row * ldy);
    if (!WIDE) {
        if (gi == 0) {
#pragma unroll
            for (int p = 0; p < VPL; ++p) {
                const int vi = gl + p * G;
                if (vi < nvec) __stcs(yr + vi, acc[p]);
            }
        }
        return;
    }
    V *sm = reinterpret_cast<V *>(smem);
    if (gi == 0) {
#pragma unroll
        for (int p = 0; p < VPL; ++p) {
            const int vi = gl + p * G;
            if (vi < nvec) sm[w * nvec + vi] = acc[p];
        }
    }
    __syncthreads();
    if (w == 0 && gi == 0) {
#pragma unroll
        for (int p = 0; p < VPL; ++p) {
            const int vi = gl + p * G;
            if (vi < nvec) {
                V tot = sm[vi];
                for (int ww = 1; ww < 8; ++ww) Vec<VEC>::add(tot, sm[ww * nvec + vi]);
                __stcs(yr + vi, tot);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// dispatch
// ---------------------------------------------------------------------------
static int tuning_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}

// Grid of the chunk kernel: 16 blocks per SM, every warp striding over the chunk list (DRONE_CHUNK_BLOCKS_PER_SM
// overrides; 0 launches one warp per chunk).  Measured against one warp per chunk, with the short-row kernel running
// beside it on the side stream: R-MAT-20 sym F = 64 0.688 -> 0.618 ms, R-MAT-22 F = 32 1.26 -> 1.09 ms, R-MAT-26 F = 32
// 25.7 -> 23.3 ms, GCN epoch on the Reddit-shaped graph 15.2 -> 15.0 ms.  8 per SM is slightly better on the R-MAT
// graphs (0.609 / 1.07 ms) and worse on the Reddit-shaped one (15.7 ms); 32 per SM loses again (1.11 ms on R-MAT-22).
static int resident_blocks() {
    const int per_sm = tuning_int("DRONE_CHUNK_BLOCKS_PER_SM", 16);
    if (per_sm <= 0) return 0;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return per_sm * sms;
}

struct SpmmArgs {
    const Side *side;
    int n_rows;
    int nvec;
    const float *X;
    long long ldv;   // leading dimension of X in vectors
    float *Y;
    long long ldy;   // leading dimension of Y in floats
    float *partials;
    cudaStream_t st;
    // when set, the short-row kernel is launched on `side_stream` between the two events (fork after what precedes the
    // call on `st`, join before what follows), so that it overlaps the chunk kernels
    cudaStream_t side_stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    int row_class = -1;   // >= 0: only the rows of that class of a plan with row classes
};


// The part of a class-major list with class starts `start` that the call computes.
static inline void class_range(int row_class, int n_classes, const int *start, int *lo, int *count) {
    *lo = row_class < 0 ? 0 : start[row_class];
    *count = (row_class < 0 ? start[n_classes] : start[row_class + 1]) - *lo;
}

template <int G, int VPL, int VEC, int U, bool EXACT>
static int launch_all(const SpmmArgs &a) {
    constexpr int RPW = 32 / G;
    const Side &s = *a.side;
    int range_lo, n_ranges, chunk_lo, n_chunks, split_lo, n_split, wide_lo, n_wide;
    class_range(a.row_class, s.n_classes, s.range_start, &range_lo, &n_ranges);
    class_range(a.row_class, s.n_classes, s.chunk_start, &chunk_lo, &n_chunks);
    class_range(a.row_class, s.n_classes, s.split_start, &split_lo, &n_split);
    class_range(a.row_class, s.n_classes, s.wide_start, &wide_lo, &n_wide);
    const bool overlap = a.side_stream != nullptr && n_ranges > 0 && n_chunks > 0;
    if (n_ranges > 0) {
        cudaStream_t short_stream = a.st;
        if (overlap) {
            DRONE_CUDA(cudaEventRecord(a.fork, a.st));
            DRONE_CUDA(cudaStreamWaitEvent(a.side_stream, a.fork, 0));
            short_stream = a.side_stream;
        }
        const int grid = ceil_div(n_ranges, 8 * RPW);
        spmm_short_stream_kernel<G, VPL, VEC, U, EXACT><<<grid, 256, 0, short_stream>>>(
            s.s_range_row + range_lo, n_ranges, s.s_rowptr, s.s_rows, s.s_col, s.s_val, a.X, a.ldv, a.Y, a.ldy, a.nvec);
        DRONE_LAUNCH_CHECK("spmm_short_stream_kernel");
        if (overlap) DRONE_CUDA(cudaEventRecord(a.join, a.side_stream));
    }
    if (n_chunks > 0) {
        int grid = ceil_div(n_chunks, 8);
        static const int resident = resident_blocks();
        if (resident > 0 && grid > resident) grid = resident;
        spmm_chunks_kernel<G, VPL, VEC, 2 * U, EXACT><<<grid, 256, 0, a.st>>>(
            s.chunks + chunk_lo, n_chunks, s.col, s.val, a.X, a.ldv, a.Y, a.ldy, a.partials, a.nvec);
        DRONE_LAUNCH_CHECK("spmm_chunks_kernel");
    }
    if (n_split > 0) {
        spmm_reduce_partials_kernel<G, VPL, VEC, false><<<ceil_div(n_split, 8), 256, 0, a.st>>>(
            s.split + split_lo, n_split, a.partials, a.Y, a.ldy, a.nvec, kWideSlots);
        DRONE_LAUNCH_CHECK("spmm_reduce_partials_kernel");
        if (n_wide > 0) {
            const size_t smem = sizeof(float) * 8 * (size_t)a.nvec * VEC;
            spmm_reduce_partials_kernel<G, VPL, VEC, true><<<n_wide, 256, smem, a.st>>>(
                s.wide + wide_lo, n_wide, a.partials, a.Y, a.ldy, a.nvec, 0);
            DRONE_LAUNCH_CHECK("spmm_reduce_partials_kernel(wide)");
        }
    }
    if (overlap) DRONE_CUDA(cudaStreamWaitEvent(a.st, a.join, 0));
    return DRONE_OK;
}

template <int G, int VPL, int VEC, int U>
static int launch_exact(const SpmmArgs &a) {
    return a.nvec == G * VPL ? launch_all<G, VPL, VEC, U, true>(a) : launch_all<G, VPL, VEC, U, false>(a);
}

template <int VEC>
static int dispatch_width(const SpmmArgs &a) {
    const int nv = a.nvec;
    if (nv <= 1) return launch_exact<1, 1, VEC, 4>(a);
    if (nv <= 2) return launch_exact<2, 1, VEC, 4>(a);
    if (nv <= 4) return launch_exact<4, 1, VEC, 4>(a);
    if (nv <= 8) return launch_exact<8, 1, VEC, 4>(a);
    if (nv <= 16) return launch_exact<16, 1, VEC, 4>(a);
    if (nv <= 32) return launch_exact<32, 1, VEC, 4>(a);
    if (nv <= 64) return launch_exact<32, 2, VEC, 2>(a);
    if (nv <= 96) return launch_exact<32, 3, VEC, 2>(a);
    if (nv <= 128) return launch_exact<32, 4, VEC, 1>(a);
    if (nv <= 256) return launch_exact<32, 8, VEC, 1>(a);
    if (VEC == 1) {
        if (nv <= 512) return launch_exact<32, 16, 1, 1>(a);
        if (nv <= 1024) return launch_exact<32, 32, 1, 1>(a);
    }
    return set_error(DRONE_E_INVALID, "drone_spmm: feature width %d is above 1024", nv * VEC);
}

static int ensure_scratch(drone_plan *p, size_t bytes) {
    if (bytes <= p->scratch_bytes) return DRONE_OK;
    // grow: frees and reallocates, so earlier calls that use the scratch must have finished
    DRONE_CUDA(cudaDeviceSynchronize());
    cudaFree(p->scratch);
    p->scratch = nullptr;
    p->scratch_bytes = 0;
    DRONE_CUDA(cudaMalloc(&p->scratch, bytes));
    p->scratch_bytes = bytes;
    return DRONE_OK;
}

// Width of the column slices a call is cut into (0 = no slicing).  Gathering a slice of w columns touches only
// n*w*4 bytes of X; when the whole operand does not fit in L2 but a slice does, running the slices one after the
// other turns HBM gathers into L2 gathers at the price of re-reading the CSR stream once per slice.
static int slice_width(const drone_plan *p, int F, bool vec4) {
    const int forced = p->slice_forced;
    if (forced == 0 || !vec4) return 0;
    if (forced > 0) return (forced % 4 == 0 && forced < F && F % forced == 0) ? forced : 0;
    const double l2_budget = 64e6;                      // about half of the 126 MB L2 for the gathered operand
    if ((double)p->n_rows * F * 4 <= l2_budget) return 0;
    for (int w : {128, 64}) {
        if (w < F && F % w == 0 && (double)p->n_rows * w * 4 <= l2_budget) return w;
    }
    return 0;
}

static int spmm_impl(drone_plan *p, int orientation, int F, const float *X, long long ldx, float *Y,
                     long long ldy, cudaStream_t st, int row_class = -1) {
    const Side &s = p->side[orientation];
    if (p->n_rows == 0) return DRONE_OK;
    const bool vec4 = (F % 4 == 0) && (ldx % 4 == 0) && (ldy % 4 == 0) &&
                      ((reinterpret_cast<uintptr_t>(X) & 15) == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0);
    const int slice = slice_width(p, F, vec4);
    const int width = slice > 0 ? slice : F;
    p->last_slice_width = slice;
    if (s.n_partials > 0) {
        const int rc = ensure_scratch(p, sizeof(float) * (size_t)s.n_partials * (size_t)width);
        if (rc) return rc;
    }
    SpmmArgs a;
    a.side = &s;
    a.n_rows = p->n_rows;
    a.ldy = ldy;
    a.partials = p->scratch;
    a.st = st;
    a.side_stream = p->side_stream;
    a.fork = p->fork_event;
    a.join = p->join_event;
    a.row_class = row_class;
    for (int c0 = 0; c0 < F; c0 += width) {
        a.X = X + c0;
        a.Y = Y + c0;
        int rc;
        if (vec4) {
            a.nvec = width / 4;
            a.ldv = ldx / 4;
            rc = dispatch_width<4>(a);
        } else {
            a.nvec = width;
            a.ldv = ldx;
            rc = dispatch_width<1>(a);
        }
        if (rc) return rc;
    }
    return DRONE_OK;
}

}  // namespace drone

using namespace drone;

extern "C" {

int drone_spmm(drone_plan *p, int orientation, int F, const float *d_X, int ldx, float *d_Y, int ldy,
               void *stream) {
    DRONE_REQUIRE(p != nullptr, "drone_spmm: plan is NULL");
    DRONE_REQUIRE(orientation == DRONE_OP_A || orientation == DRONE_OP_AT, "drone_spmm: orientation=%d", orientation);
    DRONE_REQUIRE(p->side[orientation].ready, "drone_spmm: orientation %d was not prepared by drone_plan_create",
                  orientation);
    DRONE_REQUIRE(F >= 1 && F <= 1024, "drone_spmm: feature width F=%d outside 1..1024", F);
    DRONE_REQUIRE(ldx >= F && ldy >= F, "drone_spmm: leading dimensions (ldx=%d, ldy=%d) below F=%d", ldx, ldy, F);
    if (p->n_rows == 0) return DRONE_OK;
    DRONE_REQUIRE(d_X && d_Y, "drone_spmm: NULL operand");
    DRONE_REQUIRE(d_X != d_Y, "drone_spmm: X and Y must not alias");
    int dev = -1;
    DRONE_CUDA(cudaGetDevice(&dev));
    if (dev != p->device) DRONE_CUDA(cudaSetDevice(p->device));
    const int rc = spmm_impl(p, orientation, F, d_X, ldx, d_Y, ldy, (cudaStream_t)stream);
    if (dev != p->device) cudaSetDevice(dev);
    return rc;
}

int drone_spmm_rows(drone_plan *p, int orientation, int row_class, int F, const float *d_X, int ldx, float *d_Y, int ldy,
                    void *stream) {
    DRONE_REQUIRE(p != nullptr, "drone_spmm_rows: plan is NULL");
    DRONE_REQUIRE(orientation == DRONE_OP_A || orientation == DRONE_OP_AT, "drone_spmm_rows: orientation=%d", orientation);
    DRONE_REQUIRE(p->side[orientation].ready, "drone_spmm_rows: orientation %d was not prepared by drone_plan_create",
                  orientation);
    DRONE_REQUIRE(row_class >= 0 && row_class < p->n_classes, "drone_spmm_rows: row_class=%d, the plan has %d classes",
                  row_class, p->n_classes);
    DRONE_REQUIRE(F >= 1 && F <= 1024, "drone_spmm_rows: feature width F=%d outside 1..1024", F);
    DRONE_REQUIRE(ldx >= F && ldy >= F, "drone_spmm_rows: leading dimensions (ldx=%d, ldy=%d) below F=%d", ldx, ldy, F);
    if (p->n_rows == 0) return DRONE_OK;
    DRONE_REQUIRE(d_X && d_Y, "drone_spmm_rows: NULL operand");
    DRONE_REQUIRE(d_X != d_Y, "drone_spmm_rows: X and Y must not alias");
    int dev = -1;
    DRONE_CUDA(cudaGetDevice(&dev));
    if (dev != p->device) DRONE_CUDA(cudaSetDevice(p->device));
    const int rc = spmm_impl(p, orientation, F, d_X, ldx, d_Y, ldy, (cudaStream_t)stream, row_class);
    if (dev != p->device) cudaSetDevice(dev);
    return rc;
}

// Puts the caller's device back on every way out of an entry point that had to switch to the plan's device.
struct DeviceGuard {
    int prev = -1, mine = -1;
    int enter(int device) {
        mine = device;
        DRONE_CUDA(cudaGetDevice(&prev));
        if (prev != mine) DRONE_CUDA(cudaSetDevice(mine));
        return DRONE_OK;
    }
    ~DeviceGuard() { if (prev >= 0 && prev != mine) cudaSetDevice(prev); }
};

static int ensure_staging(drone_plan *p, size_t bytes) {
    if (bytes <= p->stage_bytes) return DRONE_OK;
    DRONE_CUDA(cudaDeviceSynchronize());
    cudaFree(p->stage_x);
    cudaFree(p->stage_y);
    p->stage_x = p->stage_y = nullptr;
    p->stage_bytes = 0;
    DRONE_CUDA(cudaMalloc(&p->stage_x, bytes));
    DRONE_CUDA(cudaMalloc(&p->stage_y, bytes));
    p->stage_bytes = bytes;
    return DRONE_OK;
}

int drone_plan_reserve(drone_plan *p, int max_features, int host_operands) {
    DRONE_REQUIRE(p != nullptr, "drone_plan_reserve: plan is NULL");
    DRONE_REQUIRE(max_features >= 1 && max_features <= 1024, "drone_plan_reserve: max_features=%d outside 1..1024",
                  max_features);
    DeviceGuard guard;
    int rc = guard.enter(p->device);
    if (rc) return rc;
    const size_t slots = (size_t)std::max(p->side[0].n_partials, p->side[1].n_partials);
    if (slots > 0 && (rc = ensure_scratch(p, sizeof(float) * slots * (size_t)max_features))) return rc;
    if (host_operands) {
        if ((rc = ensure_staging(p, sizeof(float) * (size_t)p->n_rows * (size_t)max_features))) return rc;
        if (!p->own_stream) DRONE_CUDA(cudaStreamCreateWithFlags(&p->own_stream, cudaStreamNonBlocking));
    }
    return DRONE_OK;
}

int drone_spmm_host(drone_plan *p, int orientation, int F, const float *h_X, float *h_Y) {
    DRONE_REQUIRE(p != nullptr, "drone_spmm_host: plan is NULL");
    DRONE_REQUIRE(orientation == DRONE_OP_A || orientation == DRONE_OP_AT, "drone_spmm_host: orientation=%d",
                  orientation);
    DRONE_REQUIRE(p->side[orientation].ready, "drone_spmm_host: orientation %d was not prepared", orientation);
    DRONE_REQUIRE(F >= 1 && F <= 1024, "drone_spmm_host: feature width F=%d outside 1..1024", F);
    if (p->n_rows == 0) return DRONE_OK;
    DRONE_REQUIRE(h_X && h_Y, "drone_spmm_host: NULL operand");
    DeviceGuard guard;
    int rc = guard.enter(p->device);
    if (rc) return rc;
    const size_t bytes = sizeof(float) * (size_t)p->n_rows * (size_t)F;
    if ((rc = ensure_staging(p, bytes))) return rc;      // no-op after drone_plan_reserve(.., host_operands = 1)
    if (!p->own_stream) DRONE_CUDA(cudaStreamCreateWithFlags(&p->own_stream, cudaStreamNonBlocking));
    DRONE_CUDA(cudaMemcpyAsync(p->stage_x, h_X, bytes, cudaMemcpyHostToDevice, p->own_stream));
    if ((rc = spmm_impl(p, orientation, F, p->stage_x, F, p->stage_y, F, p->own_stream))) return rc;
    DRONE_CUDA(cudaMemcpyAsync(h_Y, p->stage_y, bytes, cudaMemcpyDeviceToHost, p->own_stream));
    DRONE_CUDA(cudaStreamSynchronize(p->own_stream));
    return DRONE_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Aggregation without any allocation.
//
// Some callers hand every byte of device memory to their own pool when they start, or run on a
// thread that must never wait on the driver's allocator; for them a library call that may reach
// cudaMalloc is unusable.  drone_spmm can reach it (the partial sums of split rows live in a buffer
// that grows on demand).  The entry point below does the same work with the partial sums in a
// fixed array that is part of the library image: DRONE_STATIC_SCRATCH_BYTES on every GPU that loads
// the library, until the process exits.
// ---------------------------------------------------------------------------
namespace drone {

constexpr size_t kStaticScratchFloats = DRONE_STATIC_SCRATCH_BYTES / sizeof(float);

// Partial sums of split rows, [n_partials, F] floats.  In host code this name is only a handle for
// cudaGetSymbolAddress; kernels receive the device address obtained from it.
static __device__ __align__(256) float g_static_partials[kStaticScratchFloats];

static const int kMaxDevices = 64;
static float *g_static_partials_addr[kMaxDevices];   // device address of the array on each device, once known
static std::mutex g_static_partials_mutex;

// Device address of g_static_partials on the CURRENT device (looked up once per device).
static int static_partials_address(int device, float **out) {
    if (device < 0 || device >= kMaxDevices)
        return set_error(DRONE_E_INVALID, "drone_spmm_static_scratch: device ordinal %d is outside 0..%d", device,
                         kMaxDevices - 1);
    std::lock_guard<std::mutex> lock(g_static_partials_mutex);
    if (!g_static_partials_addr[device]) {
        float *addr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress((void **)&addr, g_static_partials);
        if (err != cudaSuccess || !addr)
            return set_error(DRONE_E_CUDA, "drone_spmm_static_scratch: cudaGetSymbolAddress failed on device %d: %s", device,
                             cudaGetErrorString(err));
        g_static_partials_addr[device] = addr;
    }
    *out = g_static_partials_addr[device];
    return DRONE_OK;
}

}  // namespace drone

extern "C" int drone_spmm_static_scratch(drone_plan *p, int orientation, int F, const float *d_X, int ldx, float *d_Y,
                                         int ldy, void *stream) {
    DRONE_REQUIRE(p != nullptr, "drone_spmm_static_scratch: plan is NULL");
    DRONE_REQUIRE(orientation == DRONE_OP_A || orientation == DRONE_OP_AT, "drone_spmm_static_scratch: orientation=%d",
                  orientation);
    const drone::Side &s = p->side[orientation];
    DRONE_REQUIRE(s.ready, "drone_spmm_static_scratch: orientation %d was not prepared by drone_plan_create", orientation);
    DRONE_REQUIRE(F >= 1 && F <= 1024, "drone_spmm_static_scratch: feature width F=%d outside 1..1024", F);
    DRONE_REQUIRE(ldx >= F && ldy >= F, "drone_spmm_static_scratch: leading dimensions (ldx=%d, ldy=%d) below F=%d", ldx,
                  ldy, F);
    if (p->n_rows == 0) return DRONE_OK;
    DRONE_REQUIRE(d_X && d_Y, "drone_spmm_static_scratch: NULL operand");
    DRONE_REQUIRE(d_X != d_Y, "drone_spmm_static_scratch: X and Y must not alias");
    const size_t need = (size_t)s.n_partials * (size_t)F;
    if (need > drone::kStaticScratchFloats)
        return drone::set_error(DRONE_E_TOO_LARGE,
                                "drone_spmm_static_scratch: this plan needs %zu bytes of partial sums at F=%d, the built-in "
                                "scratch holds %zu; use drone_spmm",
                                need * sizeof(float), F, (size_t)DRONE_STATIC_SCRATCH_BYTES);
    int dev = -1;
    DRONE_CUDA(cudaGetDevice(&dev));
    if (dev != p->device) DRONE_CUDA(cudaSetDevice(p->device));
    float *partials = nullptr;
    int rc = drone::static_partials_address(p->device, &partials);
    if (rc == DRONE_OK) {
        drone::SpmmArgs a;
        a.side = &s;
        a.n_rows = p->n_rows;
        a.X = d_X;
        a.Y = d_Y;
        a.ldy = ldy;
        a.partials = partials;
        a.st = (cudaStream_t)stream;
        const bool vec4 = (F % 4 == 0) && (ldx % 4 == 0) && (ldy % 4 == 0) &&
                          ((reinterpret_cast<uintptr_t>(d_X) & 15) == 0) && ((reinterpret_cast<uintptr_t>(d_Y) & 15) == 0);
        if (vec4) {
            a.nvec = F / 4;
            a.ldv = ldx / 4;
            rc = drone::dispatch_width<4>(a);
        } else {
            a.nvec = F;
            a.ldv = ldx;
            rc = drone::dispatch_width<1>(a);
        }
    }
    if (dev != p->device) cudaSetDevice(dev);
    return rc;
}
