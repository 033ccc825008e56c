// Sparse aggregation kernels:  Y[r,:] = sum_k val[k] * X[col[k],:]  over CSR rows.
//
// The work of one call is split three ways, all decided when the plan was built:
//   1. short rows (at most short_row_limit nonzeros): one lane group per row,
//      32/G rows per warp, nonzeros added in CSR order into one accumulator;
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

namespace drone {

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
// 1. short rows: one lane group per row
// ---------------------------------------------------------------------------
template <int G, int VPL, int VEC, int U>
__global__ void __launch_bounds__(256)
spmm_short_rows_kernel(const int *__restrict__ rowptr, const int *__restrict__ col,
                       const float *__restrict__ val, const float *__restrict__ X, long long ldx,
                       float *__restrict__ Y, long long ldy, int n_rows, int nvec, int short_limit) {
    using V = typename Vec<VEC>::type;
    constexpr int RPW = 32 / G;
    constexpr int UU = MinOf<U, G>::value;
    const int lane = threadIdx.x & 31;
    const int gl = lane & (G - 1);
    const int gi = lane / G;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long row = warp * RPW + gi;
    int s = 0, deg = 0;
    const bool in_range = row < n_rows;
    if (in_range) {
        s = rowptr[row];
        deg = rowptr[row + 1] - s;
    }
    const bool mine = in_range && deg <= short_limit;
    if (!mine) deg = 0;
    int maxdeg = deg;
#pragma unroll
    for (int o = G; o < 32; o <<= 1) maxdeg = max(maxdeg, __shfl_xor_sync(0xffffffffu, maxdeg, o));

    V acc[VPL];
#pragma unroll
    for (int p = 0; p < VPL; ++p) acc[p] = Vec<VEC>::zero();

    for (int base = 0; base < maxdeg; base += G) {
        int c = 0;
        float v = 0.f;
        if (base + gl < deg) {
            c = __ldcs(col + s + base + gl);
            v = __ldcs(val + s + base + gl);
        }
        const int lim = min(G, maxdeg - base);
        for (int j = 0; j < lim; j += UU) {
            int cc[UU];
            float vv[UU];
            V x[UU][VPL];
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                cc[u] = __shfl_sync(0xffffffffu, c, j + u, G);
                vv[u] = __shfl_sync(0xffffffffu, v, j + u, G);
            }
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                const bool live = base + j + u < deg;
                const V *xr = reinterpret_cast<const V *>(X + (long long)cc[u] * ldx);
#pragma unroll
                for (int p = 0; p < VPL; ++p) {
                    const int vi = gl + p * G;
                    x[u][p] = (live && vi < nvec) ? __ldg(xr + vi) : Vec<VEC>::zero();
                }
            }
#pragma unroll
            for (int u = 0; u < UU; ++u)
#pragma unroll
                for (int p = 0; p < VPL; ++p) Vec<VEC>::fma(acc[p], vv[u], x[u][p]);
        }
    }
    if (mine) {
        V *yr = reinterpret_cast<V *>(Y + row * ldy);
#pragma unroll
        for (int p = 0; p < VPL; ++p) {
            const int vi = gl + p * G;
            if (vi < nvec) __stcs(yr + vi, acc[p]);
        }
    }
}

// ---------------------------------------------------------------------------
// 2. chunks of long rows: one warp per chunk
// ---------------------------------------------------------------------------
template <int G, int VPL, int VEC, int U>
__global__ void __launch_bounds__(256)
spmm_chunks_kernel(const Chunk *__restrict__ chunks, int n_chunks, const int *__restrict__ col,
                   const float *__restrict__ val, const float *__restrict__ X, long long ldx,
                   float *__restrict__ Y, long long ldy, float *__restrict__ partials, int nvec) {
    using V = typename Vec<VEC>::type;
    constexpr int RPW = 32 / G;
    constexpr int UU = MinOf<U, G>::value;
    const int lane = threadIdx.x & 31;
    const int gl = lane & (G - 1);
    const int gi = lane / G;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    if (warp >= n_chunks) return;
    const int4 raw = __ldg(reinterpret_cast<const int4 *>(chunks) + warp);
    const int row = raw.x, k0 = raw.y, len = raw.z, slot = raw.w;

    V acc[VPL];
#pragma unroll
    for (int p = 0; p < VPL; ++p) acc[p] = Vec<VEC>::zero();

    for (int base = 0; base < len; base += 32) {
        int c = 0;
        float v = 0.f;
        if (base + lane < len) {
            c = __ldcs(col + k0 + base + lane);
            v = __ldcs(val + k0 + base + lane);
        }
        const int cnt = min(32, len - base);
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
                const V *xr = reinterpret_cast<const V *>(X + (long long)cc[u] * ldx);
#pragma unroll
                for (int p = 0; p < VPL; ++p) {
                    const int vi = gl + p * G;
                    x[u][p] = (live && vi < nvec) ? __ldg(xr + vi) : Vec<VEC>::zero();
                }
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
        V *out = slot < 0 ? reinterpret_cast<V *>(Y + (long long)row * ldy)
                          : reinterpret_cast<V *>(partials + (long long)slot * nvec * VEC);
#pragma unroll
        for (int p = 0; p < VPL; ++p) {
            const int vi = gl + p * G;
            if (vi < nvec) {
                if (slot < 0) __stcs(out + vi, acc[p]); else out[vi] = acc[p];
            }
        }
    }
}

// ---------------------------------------------------------------------------
// 3. split rows: add the partial slots of a row in slot order
//    One block per row; lane groups of all its warps take interleaved slots.
//    Rows are filtered by slot count so that rows with few slots run with one
//    warp per block and rows with many slots with eight.
// ---------------------------------------------------------------------------
template <int G, int VPL, int VEC>
__global__ void __launch_bounds__(256)
spmm_reduce_partials_kernel(const SplitRow *__restrict__ split, int n_split,
                            const float *__restrict__ partials, float *__restrict__ Y, long long ldy,
                            int nvec, int min_slots, int max_slots) {
    using V = typename Vec<VEC>::type;
    constexpr int RPW = 32 / G;
    extern __shared__ float smem[];  // [warps][nvec*VEC] when blockDim.x > 32
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    const int nw = blockDim.x >> 5;
    const int gl = lane & (G - 1);
    const int gi = lane / G;
    if ((int)blockIdx.x >= n_split) return;
    const int4 raw = __ldg(reinterpret_cast<const int4 *>(split) + blockIdx.x);
    const int row = raw.x, slot0 = raw.y, nslots = raw.z;
    if (nslots < min_slots || nslots > max_slots) return;

    V acc[VPL];
#pragma unroll
    for (int p = 0; p < VPL; ++p) acc[p] = Vec<VEC>::zero();
    const int stride = nw * RPW;
    for (int sidx = w * RPW + gi; sidx < nslots; sidx += stride) {
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
    if (nw == 1) {
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
                for (int ww = 1; ww < nw; ++ww) Vec<VEC>::add(tot, sm[ww * nvec + vi]);
                __stcs(yr + vi, tot);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// dispatch
// ---------------------------------------------------------------------------
struct SpmmArgs {
    const Side *side;
    int n_rows;
    int nvec;
    int short_limit;
    const float *X;
    long long ldx;
    float *Y;
    long long ldy;
    float *partials;
    cudaStream_t st;
};

static const int kWideSlots = 64;  // split rows above this many slots get eight warps

template <int G, int VPL, int VEC, int U>
static int launch_all(const SpmmArgs &a) {
    constexpr int RPW = 32 / G;
    const Side &s = *a.side;
    if (a.n_rows > 0) {
        const int rows_per_block = 8 * RPW;
        const int grid = ceil_div(a.n_rows, rows_per_block);
        spmm_short_rows_kernel<G, VPL, VEC, U><<<grid, 256, 0, a.st>>>(
            s.rowptr, s.col, s.val, a.X, a.ldx, a.Y, a.ldy, a.n_rows, a.nvec, a.short_limit);
        DRONE_LAUNCH_CHECK("spmm_short_rows_kernel");
    }
    if (s.n_chunks > 0) {
        const int grid = ceil_div(s.n_chunks, 8);
        spmm_chunks_kernel<G, VPL, VEC, U><<<grid, 256, 0, a.st>>>(
            s.chunks, s.n_chunks, s.col, s.val, a.X, a.ldx, a.Y, a.ldy, a.partials, a.nvec);
        DRONE_LAUNCH_CHECK("spmm_chunks_kernel");
    }
    if (s.n_split_rows > 0) {
        spmm_reduce_partials_kernel<G, VPL, VEC><<<s.n_split_rows, 32, 0, a.st>>>(
            s.split, s.n_split_rows, a.partials, a.Y, a.ldy, a.nvec, 0, kWideSlots);
        DRONE_LAUNCH_CHECK("spmm_reduce_partials_kernel");
        if (s.max_nslots > kWideSlots) {
            const size_t smem = sizeof(float) * 8 * (size_t)a.nvec * VEC;
            spmm_reduce_partials_kernel<G, VPL, VEC><<<s.n_split_rows, 256, smem, a.st>>>(
                s.split, s.n_split_rows, a.partials, a.Y, a.ldy, a.nvec, kWideSlots + 1, 0x7fffffff);
            DRONE_LAUNCH_CHECK("spmm_reduce_partials_kernel(wide)");
        }
    }
    return DRONE_OK;
}

template <int VEC>
static int dispatch_width(const SpmmArgs &a) {
    const int nv = a.nvec;
    if (nv <= 1) return launch_all<1, 1, VEC, 4>(a);
    if (nv <= 2) return launch_all<2, 1, VEC, 4>(a);
    if (nv <= 4) return launch_all<4, 1, VEC, 4>(a);
    if (nv <= 8) return launch_all<8, 1, VEC, 4>(a);
    if (nv <= 16) return launch_all<16, 1, VEC, 4>(a);
    if (nv <= 32) return launch_all<32, 1, VEC, 4>(a);
    if (nv <= 64) return launch_all<32, 2, VEC, 4>(a);
    if (nv <= 96) return launch_all<32, 3, VEC, 2>(a);
    if (nv <= 128) return launch_all<32, 4, VEC, 2>(a);
    if (nv <= 256) return launch_all<32, 8, VEC, 1>(a);
    if (VEC == 1) {
        if (nv <= 512) return launch_all<32, 16, 1, 1>(a);
        if (nv <= 1024) return launch_all<32, 32, 1, 1>(a);
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

static int spmm_impl(drone_plan *p, int orientation, int F, const float *X, long long ldx, float *Y,
                     long long ldy, cudaStream_t st) {
    const Side &s = p->side[orientation];
    if (p->n_rows == 0) return DRONE_OK;
    if (s.n_partials > 0) {
        const int rc = ensure_scratch(p, sizeof(float) * (size_t)s.n_partials * (size_t)F);
        if (rc) return rc;
    }
    SpmmArgs a;
    a.side = &s;
    a.n_rows = p->n_rows;
    a.short_limit = p->short_row_limit;
    a.X = X;
    a.ldx = ldx;
    a.Y = Y;
    a.ldy = ldy;
    a.partials = p->scratch;
    a.st = st;
    const bool vec4 = (F % 4 == 0) && (ldx % 4 == 0) && (ldy % 4 == 0) &&
                      ((reinterpret_cast<uintptr_t>(X) & 15) == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0);
    if (vec4) {
        a.nvec = F / 4;
        return dispatch_width<4>(a);
    }
    a.nvec = F;
    return dispatch_width<1>(a);
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

int drone_spmm_host(drone_plan *p, int orientation, int F, const float *h_X, float *h_Y) {
    DRONE_REQUIRE(p != nullptr, "drone_spmm_host: plan is NULL");
    DRONE_REQUIRE(orientation == DRONE_OP_A || orientation == DRONE_OP_AT, "drone_spmm_host: orientation=%d",
                  orientation);
    DRONE_REQUIRE(p->side[orientation].ready, "drone_spmm_host: orientation %d was not prepared", orientation);
    DRONE_REQUIRE(F >= 1 && F <= 1024, "drone_spmm_host: feature width F=%d outside 1..1024", F);
    if (p->n_rows == 0) return DRONE_OK;
    DRONE_REQUIRE(h_X && h_Y, "drone_spmm_host: NULL operand");
    int dev = -1;
    DRONE_CUDA(cudaGetDevice(&dev));
    if (dev != p->device) DRONE_CUDA(cudaSetDevice(p->device));
    const size_t bytes = sizeof(float) * (size_t)p->n_rows * (size_t)F;
    if (bytes > p->stage_bytes) {
        cudaFree(p->stage_x);
        cudaFree(p->stage_y);
        p->stage_x = p->stage_y = nullptr;
        p->stage_bytes = 0;
        DRONE_CUDA(cudaMalloc(&p->stage_x, bytes));
        DRONE_CUDA(cudaMalloc(&p->stage_y, bytes));
        p->stage_bytes = bytes;
    }
    if (!p->own_stream) DRONE_CUDA(cudaStreamCreateWithFlags(&p->own_stream, cudaStreamNonBlocking));
    DRONE_CUDA(cudaMemcpyAsync(p->stage_x, h_X, bytes, cudaMemcpyHostToDevice, p->own_stream));
    const int rc = spmm_impl(p, orientation, F, p->stage_x, F, p->stage_y, F, p->own_stream);
    if (rc) return rc;
    DRONE_CUDA(cudaMemcpyAsync(h_Y, p->stage_y, bytes, cudaMemcpyDeviceToHost, p->own_stream));
    DRONE_CUDA(cudaStreamSynchronize(p->own_stream));
    if (dev != p->device) cudaSetDevice(dev);
    return DRONE_OK;
}

}  // extern "C"
