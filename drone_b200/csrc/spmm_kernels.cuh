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
//      chunk is written directly, otherwise the chunk sum goes to a partial slot.
//      The warps of a resident grid take the chunks from a shared counter, four
//      at a time, so that no warp idles while another still has a queue;
//   3. split rows: the partial slots of a row are added in slot order.
// A lane group is G lanes that together hold one dense row: each lane owns VPL
// vectors of VEC floats (float4 when the operands allow 16-byte accesses).
// No atomics touch the data, so the summation order is fixed by the plan and two
// calls give the same bits whichever warp happens to take which chunk.
//
// Template switches shared by the kernels:
//   UNIT  every stored coefficient counts as 1 (the val stream is not read);
//   HOT   columns carry a tag: a tagged column is a position in the plan's table of
//         hot rows (a compact copy of the most often gathered rows of X, small
//         enough to stay in L2 when X itself is many times larger than L2).
//
// The CSR streams (col, val) and the output are touched once and use streaming
// cache hints so that L2 capacity is left to the gathered rows of X.
//
// This header is compiled into several translation units, one per combination of
// the switches, so that they build side by side.
#pragma once

#include "plan.cuh"

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
    static __device__ __forceinline__ float4 finish(const float4 &a, float scale, int relu) {
        float4 r = make_float4(a.x * scale, a.y * scale, a.z * scale, a.w * scale);
        if (relu) { r.x = fmaxf(r.x, 0.f); r.y = fmaxf(r.y, 0.f); r.z = fmaxf(r.z, 0.f); r.w = fmaxf(r.w, 0.f); }
        return r;
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
    static __device__ __forceinline__ float finish(const float &a, float scale, int relu) {
        const float r = a * scale;
        return relu ? fmaxf(r, 0.f) : r;
    }
};

template <int A, int B> struct MinOf { static constexpr int value = A < B ? A : B; };

// What happens to a finished row before it is stored: Y[r,:] = act(row_scale[r] * sum).  Without a scale array the
// multiplication is skipped, so the plain call stores exactly the sum.
struct Epilogue {
    const float *row_scale = nullptr;   // [n_rows] or NULL
    int relu = 0;                       // 1: negative results are stored as 0
    // Routed rows (the aggregation that also performs the upward half of the mirror/master exchange): route[r] =
    // {peer, row in that peer's receive area} for a row whose total another GPU forms, {-1, ..} otherwise.  A routed
    // row is stored into the peer's memory (rows of route_nvec vectors there; this call writes vectors route_col0 ..)
    // and not into Y.
    const int2 *route = nullptr;        // [n_rows] or NULL
    float *const *peer_rows = nullptr;  // [peers] base of every peer's receive area
    int route_nvec = 0, route_col0 = 0;
};

template <int VEC>
__device__ __forceinline__ typename Vec<VEC>::type finish_row(const typename Vec<VEC>::type &acc, const Epilogue &e,
                                                              float scale) {
    if (e.row_scale == nullptr && !e.relu) return acc;
    return Vec<VEC>::finish(acc, scale, e.relu);
}

// Where a finished row goes: its row of Y, or its place in the owner's receive area (remote: the caller uses a plain
// store, no cache policy of this GPU's L2 on a peer's address).
template <int VEC>
struct RowDestination {
    typename Vec<VEC>::type *ptr;
    bool remote;
};

template <int VEC>
__device__ __forceinline__ RowDestination<VEC> row_destination(const Epilogue &e, float *Y, long long ldy, int row) {
    using V = typename Vec<VEC>::type;
    if (e.route != nullptr) {
        const int2 r = __ldg(e.route + row);
        if (r.x >= 0)
            return {reinterpret_cast<V *>(e.peer_rows[r.x]) + (long long)r.y * e.route_nvec + e.route_col0, true};
    }
    return {reinterpret_cast<V *>(Y + (long long)row * ldy), false};
}

// Where the gathered rows come from.  Without HOT only X is used.
struct Gather {
    const float *X = nullptr;
    long long ldv = 0;                  // leading dimension of X in vectors
    const float *hot = nullptr;         // table of hot rows, [hot_rows, nvec] vectors, dense
    const int *hot_ids = nullptr;       // column of every hot position (all tagged positions, also those beyond hot_rows)
    int hot_rows = 0;                   // tagged positions below this are served from the table
};

// Tagged columns whose position lies beyond the rows the table holds at this call's width are turned back into
// plain columns (one look-up in hot_ids).  Done on the freshly loaded (col) registers of a lane, before they are
// handed around, so that the gathers themselves need no branch and no dependent load.
template <bool HOT>
__device__ __forceinline__ unsigned resolve_column(const Gather &g, unsigned c) {
    if (HOT && (c & kHotTag) && (int)(c & kHotMask) >= g.hot_rows) c = (unsigned)__ldg(g.hot_ids + (c & kHotMask));
    return c;
}

// Address of the row a resolved column stands for: a row of the table for a tagged column, a row of X otherwise.
// Branch-free, so that the gathers of a batch stay independent loads in flight together.  The table is written by
// the fill kernel that precedes the gathering kernels of the same call in stream order, so the read-only load path
// is safe for it as well.
template <int VEC, bool HOT>
__device__ __forceinline__ const typename Vec<VEC>::type *row_address(const Gather &g, unsigned c, int gl, int nvec) {
    using V = typename Vec<VEC>::type;
    if (!HOT) return reinterpret_cast<const V *>(g.X) + (long long)c * g.ldv + gl;
    const bool tagged = (c & kHotTag) != 0;
    const V *base = reinterpret_cast<const V *>(tagged ? g.hot : g.X);
    const long long stride = tagged ? (long long)nvec : g.ldv;
    return base + (long long)(c & kHotMask) * stride + gl;
}

// ---------------------------------------------------------------------------
// 0. table of hot rows: hot[pos, :] = X[hot_ids[pos], :] for pos < hot_rows (dense, nvec vectors per row).
// ---------------------------------------------------------------------------
template <int VEC>
__global__ void __launch_bounds__(256)
spmm_fill_hot_kernel(const int *__restrict__ hot_ids, int hot_rows, const float *__restrict__ X, long long ldv, int nvec,
                     float *__restrict__ hot) {
    using V = typename Vec<VEC>::type;
    const long long total = (long long)hot_rows * nvec;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int pos = (int)(i / nvec), j = (int)(i - (long long)pos * nvec);
        reinterpret_cast<V *>(hot)[i] = __ldg(reinterpret_cast<const V *>(X) + (long long)__ldg(hot_ids + pos) * ldv + j);
    }
}

// ---------------------------------------------------------------------------
// 1. short rows: one lane group walks a range of the short-row stream
//    (about kShortRangeNnz entries, whole rows only) and writes each row when
//    its last entry has been added.  Entries of a row are added in CSR order
//    into one accumulator.
// ---------------------------------------------------------------------------
template <int G, int VPL, int VEC, int U, bool EXACT, bool UNIT, bool HOT>
__global__ void __launch_bounds__(256)
spmm_short_stream_kernel(const int *__restrict__ s_range_row, int n_ranges, const int *__restrict__ s_rowptr,
                         const int *__restrict__ s_rows, const int *__restrict__ s_col,
                         const float *__restrict__ s_val, Gather g, float *__restrict__ Y, long long ldy, int nvec,
                         Epilogue epi) {
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

    const unsigned long long pol_keep = l2_policy_keep(), pol_stream = l2_policy_stream();
    V acc[VPL];
#pragma unroll
    for (int p = 0; p < VPL; ++p) acc[p] = Vec<VEC>::zero();

    unsigned c_next = 0;
    float v_next = UNIT ? 1.f : 0.f;
    if (k + gl < kend) {
        c_next = (unsigned)ld_stream(s_col + k + gl, pol_stream);
        if (!UNIT) v_next = ld_stream(s_val + k + gl, pol_stream);
    }
    for (int base = 0; base < maxlen; base += G) {
        const unsigned c = (c_next & ~kColMask) | resolve_column<HOT>(g, c_next & kColMask);
        const float v = v_next;
        c_next = 0;
        if (!UNIT) v_next = 0.f;
        if (k + base + G + gl < kend) {   // next batch, requested before this batch's gathers
            c_next = (unsigned)ld_stream(s_col + k + base + G + gl, pol_stream);
            if (!UNIT) v_next = ld_stream(s_val + k + base + G + gl, pol_stream);
        }
        const int lim = min(G, maxlen - base);
        for (int j = 0; j < lim; j += UU) {
            unsigned cc[UU];
            float vv[UU];
            V x[UU][VPL];
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                cc[u] = __shfl_sync(0xffffffffu, c, j + u, G);
                vv[u] = UNIT ? 1.f : __shfl_sync(0xffffffffu, v, j + u, G);
            }
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                const bool live = (k + base + j + u < kend) && !(cc[u] & kPlaceholder);
                const V *xr = row_address<VEC, HOT>(g, live ? (cc[u] & kColMask) : 0u, gl, nvec);
#pragma unroll
                for (int p = 0; p < VPL; ++p)
                    x[u][p] = (live && (EXACT || gl + p * G < nvec)) ? ld_keep(xr + p * G, pol_keep)
                                                                    : Vec<VEC>::zero();
            }
#pragma unroll
            for (int u = 0; u < UU; ++u) {
#pragma unroll
                for (int p = 0; p < VPL; ++p) Vec<VEC>::fma(acc[p], vv[u], x[u][p]);
                if ((cc[u] & kLastInRow) && (k + base + j + u < kend)) {
                    const int row = s_rows[ri];
                    const float scale = epi.row_scale ? __ldg(epi.row_scale + row) : 1.f;
                    const RowDestination<VEC> dest = row_destination<VEC>(epi, Y, ldy, row);
                    const bool remote = dest.remote;
                    V *yr = dest.ptr + gl;
#pragma unroll
                    for (int p = 0; p < VPL; ++p) {
                        if (EXACT || gl + p * G < nvec) {
                            const V out = finish_row<VEC>(acc[p], epi, scale);
                            if (remote) yr[p * G] = out;
                            else st_stream(yr + p * G, out, pol_stream);
                        }
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
//    pairs at a time; its 32/G lane groups take interleaved entries.  Warps take
//    chunks from `counter` kChunkGroup at a time (the counter starts at 0; the group size is a compile-time
//    constant on purpose: with a run-time size the compiler produced a tighter loop over the group that ran a
//    quarter slower on the largest graphs); the
//    next group's index is requested while the current group is being worked on,
//    and the first (col, val) batch of the next chunk while the current chunk is.
// ---------------------------------------------------------------------------
constexpr int kChunkGroup = 4;

template <int G, int VPL, int VEC, int U, bool EXACT, bool UNIT, bool HOT>
__global__ void __launch_bounds__(256)
spmm_chunks_kernel(const Chunk *__restrict__ chunks, int n_chunks, const int *__restrict__ col,
                   const float *__restrict__ val, Gather g, float *__restrict__ Y, long long ldy,
                   float *__restrict__ partials, int nvec, Epilogue epi, unsigned *counter) {
    using V = typename Vec<VEC>::type;
    constexpr int RPW = 32 / G;
    constexpr int UU = MinOf<U, G>::value;
    const int lane = threadIdx.x & 31;
    const int gl = lane & (G - 1);
    const int gi = lane / G;
    const unsigned long long pol_keep = l2_policy_keep(), pol_stream = l2_policy_stream();

    unsigned group = 0;
    if (lane == 0) group = atomicAdd(counter, (unsigned)kChunkGroup);
    group = __shfl_sync(0xffffffffu, group, 0);
    while (group < (unsigned)n_chunks) {
        int4 desc = make_int4(0, 0, 0, 0);
        if (lane < kChunkGroup && group + lane < (unsigned)n_chunks)
            desc = __ldg(reinterpret_cast<const int4 *>(chunks) + group + lane);
        const int in_group = min(kChunkGroup, n_chunks - (int)group);
        unsigned next_group = 0;
        if (lane == 0) next_group = atomicAdd(counter, (unsigned)kChunkGroup);   // needed only after this group

        // first batch of the group's first chunk
        int c = 0;
        float v = UNIT ? 1.f : 0.f;
        {
            const int k0 = __shfl_sync(0xffffffffu, desc.y, 0), len = __shfl_sync(0xffffffffu, desc.z, 0);
            if (lane < len) {
                c = ld_stream(col + k0 + lane, pol_stream);
                if (!UNIT) v = ld_stream(val + k0 + lane, pol_stream);
            }
            c = (int)resolve_column<HOT>(g, (unsigned)c);
        }
        for (int j = 0; j < in_group; ++j) {
            const int row = __shfl_sync(0xffffffffu, desc.x, j), k0 = __shfl_sync(0xffffffffu, desc.y, j);
            const int len = __shfl_sync(0xffffffffu, desc.z, j), slot = __shfl_sync(0xffffffffu, desc.w, j);
            // first batch of the chunk after this one, requested now and used when this chunk is done
            int c_ahead = 0;
            float v_ahead = UNIT ? 1.f : 0.f;
            if (j + 1 < in_group) {
                const int nk0 = __shfl_sync(0xffffffffu, desc.y, j + 1), nlen = __shfl_sync(0xffffffffu, desc.z, j + 1);
                if (lane < nlen) {
                    c_ahead = ld_stream(col + nk0 + lane, pol_stream);
                    if (!UNIT) v_ahead = ld_stream(val + nk0 + lane, pol_stream);
                }
            }

            V acc[VPL];
#pragma unroll
            for (int p = 0; p < VPL; ++p) acc[p] = Vec<VEC>::zero();

            int base = 0;
            // full batches of 32 entries: no bounds checks.  (col, val) of the next batch are requested before the
            // gathers of the current one, so the dependent chain col -> X row costs one memory latency per batch
            for (; base + 32 <= len; base += 32) {
                int c_next = 0;
                float v_next = UNIT ? 1.f : 0.f;
                if (base + 32 + lane < len) {
                    c_next = ld_stream(col + k0 + base + 32 + lane, pol_stream);
                    if (!UNIT) v_next = ld_stream(val + k0 + base + 32 + lane, pol_stream);
                }
#pragma unroll
                for (int t = 0; t < G; t += UU) {
                    int cc[UU];
                    float vv[UU];
                    V x[UU][VPL];
#pragma unroll
                    for (int u = 0; u < UU; ++u) {
                        cc[u] = __shfl_sync(0xffffffffu, c, (t + u) * RPW + gi);
                        vv[u] = UNIT ? 1.f : __shfl_sync(0xffffffffu, v, (t + u) * RPW + gi);
                    }
#pragma unroll
                    for (int u = 0; u < UU; ++u) {
                        const V *xr = row_address<VEC, HOT>(g, (unsigned)cc[u], gl, nvec);
#pragma unroll
                        for (int p = 0; p < VPL; ++p)
                            x[u][p] = (EXACT || gl + p * G < nvec) ? ld_keep(xr + p * G, pol_keep)
                                                                   : Vec<VEC>::zero();
                    }
#pragma unroll
                    for (int u = 0; u < UU; ++u)
#pragma unroll
                        for (int p = 0; p < VPL; ++p) Vec<VEC>::fma(acc[p], vv[u], x[u][p]);
                }
                c = (int)resolve_column<HOT>(g, (unsigned)c_next);
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
                        vv[u] = UNIT ? 1.f : __shfl_sync(0xffffffffu, v, e & 31);
                        if (e >= cnt) { vv[u] = 0.f; cc[u] = 0; }
                    }
#pragma unroll
                    for (int u = 0; u < UU; ++u) {
                        const bool live = (t + u) * RPW + gi < cnt;
                        const V *xr = row_address<VEC, HOT>(g, (unsigned)cc[u], gl, nvec);
#pragma unroll
                        for (int p = 0; p < VPL; ++p)
                            x[u][p] = (live && (EXACT || gl + p * G < nvec)) ? ld_keep(xr + p * G, pol_keep)
                                                                            : Vec<VEC>::zero();
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
                if (slot < 0) {
                    const float scale = epi.row_scale ? __ldg(epi.row_scale + row) : 1.f;
                    const RowDestination<VEC> dest = row_destination<VEC>(epi, Y, ldy, row);
                    const bool remote = dest.remote;
                    V *out = dest.ptr + gl;
#pragma unroll
                    for (int p = 0; p < VPL; ++p)
                        if (EXACT || gl + p * G < nvec) {
                            const V tot = finish_row<VEC>(acc[p], epi, scale);
                            if (remote) out[p * G] = tot;
                            else st_stream(out + p * G, tot, pol_stream);
                        }
                } else {
                    V *out = reinterpret_cast<V *>(partials + (long long)slot * nvec * VEC) + gl;
#pragma unroll
                    for (int p = 0; p < VPL; ++p)
                        if (EXACT || gl + p * G < nvec) out[p * G] = acc[p];
                }
            }
            c = (int)resolve_column<HOT>(g, (unsigned)c_ahead);
            v = v_ahead;
        }  // chunks of the group
        group = __shfl_sync(0xffffffffu, next_group, 0);
    }
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
                            int nvec, int max_slots, Epilogue epi) {
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

    const float scale = epi.row_scale ? __ldg(epi.row_scale + row) : 1.f;
    const RowDestination<VEC> dest = row_destination<VEC>(epi, Y, ldy, row);
    const bool remote = dest.remote;
    V *yr = dest.ptr;
    if (!WIDE) {
        if (gi == 0) {
#pragma unroll
            for (int p = 0; p < VPL; ++p) {
                const int vi = gl + p * G;
                if (vi < nvec) {
                    if (remote) yr[vi] = finish_row<VEC>(acc[p], epi, scale);
                    else __stcs(yr + vi, finish_row<VEC>(acc[p], epi, scale));
                }
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
                if (remote) yr[vi] = finish_row<VEC>(tot, epi, scale);
                else __stcs(yr + vi, finish_row<VEC>(tot, epi, scale));
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
    Gather gather;
    float *Y;
    long long ldy;   // leading dimension of Y in floats
    float *partials;
    unsigned *counter;   // chunk counter of the plan (one word, set to 0 in front of every chunk launch)
    Epilogue epi;
    cudaStream_t st;
    // when set, the short-row kernel is launched on `side_stream` between the two events (fork after what precedes the
    // call on `st`, join before what follows), so that it overlaps the chunk kernels
    cudaStream_t side_stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    int row_class = -1;   // >= 0: only the rows of that class of a plan with row classes
    int resident_per_sm = 0;   // 0: as many blocks of the chunk kernel as fit; > 0: at most this many per SM
};

// The part of a class-major list with class starts `start` that the call computes.
static inline void class_range(int row_class, int n_classes, const int *start, int *lo, int *count) {
    *lo = row_class < 0 ? 0 : start[row_class];
    *count = (row_class < 0 ? start[n_classes] : start[row_class + 1]) - *lo;
}

// Blocks of a kernel that one SM holds at a time (asked once per instantiation) times the SM count of the device.
template <typename Kernel>
static int resident_grid(Kernel kernel, int cap_per_sm) {
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, 0) != cudaSuccess) return 0;
    if (cap_per_sm > 0 && per_sm > cap_per_sm) per_sm = cap_per_sm;
    return per_sm * sms;
}

template <int G, int VPL, int VEC, int U, bool EXACT, bool UNIT, bool HOT>
static int launch_all(const SpmmArgs &a) {
    constexpr int RPW = 32 / G;
    const Side &s = *a.side;
    int range_lo, n_ranges, chunk_lo, n_chunks, split_lo, n_split, wide_lo, n_wide;
    class_range(a.row_class, s.n_classes, s.range_start, &range_lo, &n_ranges);
    class_range(a.row_class, s.n_classes, s.chunk_start, &chunk_lo, &n_chunks);
    class_range(a.row_class, s.n_classes, s.split_start, &split_lo, &n_split);
    class_range(a.row_class, s.n_classes, s.wide_start, &wide_lo, &n_wide);
    if (HOT && a.gather.hot_rows > 0) {
        const long long total = (long long)a.gather.hot_rows * a.nvec;
        const int grid = (int)std::min<long long>((total + 255) / 256, 148 * 16);
        spmm_fill_hot_kernel<VEC><<<grid, 256, 0, a.st>>>(a.gather.hot_ids, a.gather.hot_rows, a.gather.X, a.gather.ldv,
                                                         a.nvec, const_cast<float *>(a.gather.hot));
        DRONE_LAUNCH_CHECK("spmm_fill_hot_kernel");
    }
    const bool overlap = a.side_stream != nullptr && n_ranges > 0 && n_chunks > 0;
    if (n_ranges > 0) {
        cudaStream_t short_stream = a.st;
        if (overlap) {
            DRONE_CUDA(cudaEventRecord(a.fork, a.st));
            DRONE_CUDA(cudaStreamWaitEvent(a.side_stream, a.fork, 0));
            short_stream = a.side_stream;
        }
        const int grid = ceil_div(n_ranges, 8 * RPW);
        spmm_short_stream_kernel<G, VPL, VEC, U, EXACT, UNIT, HOT><<<grid, 256, 0, short_stream>>>(
            s.s_range_row + range_lo, n_ranges, s.s_rowptr, s.s_rows, s.s_col, s.s_val, a.gather, a.Y, a.ldy, a.nvec, a.epi);
        DRONE_LAUNCH_CHECK("spmm_short_stream_kernel");
        if (overlap) DRONE_CUDA(cudaEventRecord(a.join, a.side_stream));
    }
    if (n_chunks > 0) {
        auto kernel = spmm_chunks_kernel<G, VPL, VEC, 2 * U, EXACT, UNIT, HOT>;
        static int resident_all = 0;
        if (resident_all == 0) resident_all = resident_grid(kernel, 0);
        int resident = resident_all;
        if (a.resident_per_sm > 0) resident = std::min(resident, a.resident_per_sm * 148);
        int grid = ceil_div(ceil_div(n_chunks, kChunkGroup), 8);
        if (resident > 0 && grid > resident) grid = resident;
        DRONE_CUDA(cudaMemsetAsync(a.counter, 0, sizeof(unsigned), a.st));
        kernel<<<grid, 256, 0, a.st>>>(s.chunks + chunk_lo, n_chunks, s.col, s.val, a.gather, a.Y, a.ldy, a.partials,
                                       a.nvec, a.epi, a.counter);
        DRONE_LAUNCH_CHECK("spmm_chunks_kernel");
    }
    if (n_split > 0) {
        spmm_reduce_partials_kernel<G, VPL, VEC, false><<<ceil_div(n_split, 8), 256, 0, a.st>>>(
            s.split + split_lo, n_split, a.partials, a.Y, a.ldy, a.nvec, kWideSlots, a.epi);
        DRONE_LAUNCH_CHECK("spmm_reduce_partials_kernel");
        if (n_wide > 0) {
            const size_t smem = sizeof(float) * 8 * (size_t)a.nvec * VEC;
            spmm_reduce_partials_kernel<G, VPL, VEC, true><<<n_wide, 256, smem, a.st>>>(
                s.wide + wide_lo, n_wide, a.partials, a.Y, a.ldy, a.nvec, 0, a.epi);
            DRONE_LAUNCH_CHECK("spmm_reduce_partials_kernel(wide)");
        }
    }
    if (overlap) DRONE_CUDA(cudaStreamWaitEvent(a.st, a.join, 0));
    return DRONE_OK;
}

template <int G, int VPL, int VEC, int U, bool UNIT, bool HOT>
static int launch_exact(const SpmmArgs &a) {
    return a.nvec == G * VPL ? launch_all<G, VPL, VEC, U, true, UNIT, HOT>(a) : launch_all<G, VPL, VEC, U, false, UNIT, HOT>(a);
}

// Entry of a translation unit: picks the lane-group shape for the width (nvec vectors of VEC floats per row).
template <int VEC, bool UNIT, bool HOT>
static int dispatch_width(const SpmmArgs &a) {
    const int nv = a.nvec;
    if (nv <= 1) return launch_exact<1, 1, VEC, 4, UNIT, HOT>(a);
    if (nv <= 2) return launch_exact<2, 1, VEC, 4, UNIT, HOT>(a);
    if (nv <= 4) return launch_exact<4, 1, VEC, 4, UNIT, HOT>(a);
    if (nv <= 8) return launch_exact<8, 1, VEC, 4, UNIT, HOT>(a);
    if (nv <= 16) return launch_exact<16, 1, VEC, 4, UNIT, HOT>(a);
    if (nv <= 32) return launch_exact<32, 1, VEC, 4, UNIT, HOT>(a);
    if (nv <= 64) return launch_exact<32, 2, VEC, 2, UNIT, HOT>(a);
    if (nv <= 96) return launch_exact<32, 3, VEC, 2, UNIT, HOT>(a);
    if (nv <= 128) return launch_exact<32, 4, VEC, 1, UNIT, HOT>(a);
    if (nv <= 256) return launch_exact<32, 8, VEC, 1, UNIT, HOT>(a);
    if (VEC == 1) {
        if (nv <= 512) return launch_exact<32, 16, 1, 1, UNIT, HOT>(a);
        if (nv <= 1024) return launch_exact<32, 32, 1, 1, UNIT, HOT>(a);
    }
    return set_error(DRONE_E_INVALID, "drone_spmm: feature width %d is above 1024", nv * VEC);
}

// The four combinations, each defined in a translation unit of its own (spmm_variants_*.cu).
int spmm_dispatch_plain(const SpmmArgs &a, bool vec4);
int spmm_dispatch_unit(const SpmmArgs &a, bool vec4);
int spmm_dispatch_hot(const SpmmArgs &a, bool vec4);
int spmm_dispatch_unit_hot(const SpmmArgs &a, bool vec4);

}  // namespace drone
