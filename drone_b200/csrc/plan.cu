// Plan construction: coefficient kernel, transposed CSR, and the split of rows
// into short rows and fixed-size chunks of long rows.  Everything here runs once
// per graph; none of it is on the per-layer path.
#include "plan.cuh"

#include <cub/cub.cuh>
#include <algorithm>
#include <cstdlib>
#include <new>

namespace drone {

static thread_local char t_error[512];
std::atomic<long long> g_kernel_launches{0};

char *last_error_buffer() { return t_error; }

int set_error(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
    return code;
}

// ---------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------

// values[i] = 1/sqrt(outDeg[u]*inDeg[v]) for edge i = u->v, one warp per source
// row.  The arithmetic follows the reference expression literally
// (cuda_gcn/src/cuda/cuda_kernel.cu:151): the degree product is formed in
// double, narrowed to float for sqrtf, and the reciprocal is a double division
// narrowed to float on the store.
__global__ void csr_values_kernel(const int *__restrict__ index, const int *__restrict__ dst,
                                  const int *__restrict__ in_deg, const int *__restrict__ out_deg,
                                  int n_rows, float *__restrict__ values) {
    const int lane = threadIdx.x & 31;
    const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    for (int u = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; u < n_rows; u += warps_per_grid) {
        const int s = index[u], e = index[u + 1];
        const double od = 1.0 * out_deg[u];
        for (int i = s + lane; i < e; i += 32) {
            const int v = dst[i];
            const float root = sqrtf((float)(od * in_deg[v]));
            values[i] = (float)(1.0 / root);
        }
    }
}

// src[k] = row that owns nonzero k (upper bound search in rowptr).
__global__ void expand_rows_kernel(const int *__restrict__ rowptr, int n_rows, int nnz,
                                   int *__restrict__ src) {
    for (long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x; k < nnz;
         k += (long long)gridDim.x * blockDim.x) {
        int lo = 0, hi = n_rows;  // find the last row with rowptr[row] <= k
        while (hi - lo > 1) {
            const int mid = lo + ((hi - lo) >> 1);
            if (rowptr[mid] <= (int)k) lo = mid; else hi = mid;
        }
        src[k] = lo;
    }
}

__global__ void histogram_kernel(const int *__restrict__ keys, int n, int *__restrict__ counts) {
    for (long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x; k < n;
         k += (long long)gridDim.x * blockDim.x)
        atomicAdd(counts + keys[k], 1);
}

// colT[i] = src[perm[i]], valT[i] = val[perm[i]]
__global__ void gather_transposed_kernel(const int *__restrict__ perm, const int *__restrict__ src,
                                         const float *__restrict__ val, int nnz,
                                         int *__restrict__ col_t, float *__restrict__ val_t) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nnz;
         i += (long long)gridDim.x * blockDim.x) {
        const int p = perm[i];
        col_t[i] = src[p];
        val_t[i] = val[p];
    }
}

__global__ void iota_kernel(int *a, int n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        a[i] = (int)i;
}

// Per row: number of chunks (0 for short rows), number of partial slots, split flag.
__global__ void count_chunks_kernel(const int *__restrict__ rowptr, int n_rows, int short_limit,
                                    int chunk_nnz, int *__restrict__ n_chunks,
                                    int *__restrict__ n_slots, int *__restrict__ is_split,
                                    int *__restrict__ is_long) {
    for (long long r = blockIdx.x * (long long)blockDim.x + threadIdx.x; r <= n_rows;
         r += (long long)gridDim.x * blockDim.x) {
        int c = 0;
        if (r < n_rows) {
            const int deg = rowptr[r + 1] - rowptr[r];
            if (deg > short_limit) c = (deg + chunk_nnz - 1) / chunk_nnz;
        }
        n_chunks[r] = c;
        n_slots[r] = c > 1 ? c : 0;
        is_split[r] = c > 1 ? 1 : 0;
        is_long[r] = c > 0 ? 1 : 0;
    }
}

__global__ void fill_chunks_kernel(const int *__restrict__ rowptr, int n_rows, int chunk_nnz,
                                   const int *__restrict__ chunk_cnt, const int *__restrict__ chunk_off,
                                   const int *__restrict__ slot_off, const int *__restrict__ split_off,
                                   Chunk *__restrict__ chunks, SplitRow *__restrict__ split) {
    for (long long r = blockIdx.x * (long long)blockDim.x + threadIdx.x; r < n_rows;
         r += (long long)gridDim.x * blockDim.x) {
        const int nc = chunk_cnt[r];
        if (nc == 0) continue;
        const int s = rowptr[r], e = rowptr[r + 1];
        const int c0 = chunk_off[r];
        const int p0 = slot_off[r];
        for (int c = 0; c < nc; ++c) {
            Chunk ch;
            ch.row = (int)r;
            ch.k0 = s + c * chunk_nnz;
            ch.len = min(chunk_nnz, e - ch.k0);
            ch.slot = nc > 1 ? p0 + c : -1;
            chunks[c0 + c] = ch;
        }
        if (nc > 1) {
            SplitRow sr;
            sr.row = (int)r;
            sr.slot0 = p0;
            sr.nslots = nc;
            sr.pad = 0;
            split[split_off[r]] = sr;
        }
    }
}

// key[i] = first column of chunk i (tags removed), idx[i] = i
__global__ void chunk_first_column_kernel(const Chunk *__restrict__ chunks, int n_chunks, const int *__restrict__ col,
                                          int *__restrict__ key, int *__restrict__ idx) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_chunks; i += (long long)gridDim.x * blockDim.x) {
        key[i] = (int)((unsigned)col[chunks[i].k0] & kHotMask);
        idx[i] = (int)i;
    }
}

__global__ void permute_chunks_kernel(const Chunk *__restrict__ in, const int *__restrict__ order, int n_chunks,
                                      Chunk *__restrict__ out) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_chunks; i += (long long)gridDim.x * blockDim.x)
        out[i] = in[order[i]];
}

// Per row: 1 if short, and its number of stream entries (a row without nonzeros gets one placeholder).
__global__ void count_short_kernel(const int *__restrict__ rowptr, int n_rows, int short_limit,
                                   int *__restrict__ is_short, int *__restrict__ n_entries) {
    for (long long r = blockIdx.x * (long long)blockDim.x + threadIdx.x; r <= n_rows;
         r += (long long)gridDim.x * blockDim.x) {
        int s = 0, e = 0;
        if (r < n_rows) {
            const int deg = rowptr[r + 1] - rowptr[r];
            if (deg <= short_limit) { s = 1; e = deg > 0 ? deg : 1; }
        }
        is_short[r] = s;
        n_entries[r] = e;
    }
}

__global__ void fill_short_kernel(const int *__restrict__ rowptr, const int *__restrict__ col,
                                  const float *__restrict__ val, int n_rows, int short_limit,
                                  const int *__restrict__ short_off, const int *__restrict__ entry_off,
                                  int *__restrict__ s_rows, int *__restrict__ s_rowptr,
                                  int *__restrict__ s_col, float *__restrict__ s_val) {
    for (long long r = blockIdx.x * (long long)blockDim.x + threadIdx.x; r < n_rows;
         r += (long long)gridDim.x * blockDim.x) {
        const int b = rowptr[r], deg = rowptr[r + 1] - b;
        if (deg > short_limit) continue;
        const int si = short_off[r];
        const int e0 = entry_off[r];
        s_rows[si] = (int)r;
        s_rowptr[si] = e0;
        if (deg == 0) {
            s_col[e0] = (int)(kLastInRow | kPlaceholder);
            s_val[e0] = 0.f;
        } else {
            for (int j = 0; j < deg; ++j) {
                unsigned c = (unsigned)col[b + j];
                if (j == deg - 1) c |= kLastInRow;
                s_col[e0 + j] = (int)c;
                s_val[e0 + j] = val[b + j];
            }
        }
    }
}

// out[i] = first short row in [row_lo, row_hi) whose stream offset is >= first_entry + i * range_nnz, for i < n_ranges
__global__ void short_ranges_kernel(const int *__restrict__ s_rowptr, int row_lo, int row_hi, long long first_entry,
                                    int n_ranges, int range_nnz, int *__restrict__ out) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_ranges;
         i += (long long)gridDim.x * blockDim.x) {
        const long long target = first_entry + i * (long long)range_nnz;
        int lo = row_lo, hi = row_hi;  // first index with s_rowptr[idx] >= target
        while (lo < hi) {
            const int mid = lo + ((hi - lo) >> 1);
            if (s_rowptr[mid] < target) lo = mid + 1; else hi = mid;
        }
        out[i] = lo;
    }
}

// permuted[i] = cnt[order[i]] for i < n, permuted[n] = 0
__global__ void gather_counts_kernel(const int *__restrict__ cnt, const int *__restrict__ order, int n,
                                     int *__restrict__ permuted) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i <= n;
         i += (long long)gridDim.x * blockDim.x)
        permuted[i] = i < n ? cnt[order[i]] : 0;
}

// off[order[i]] = permuted_off[i] for i < n, off[n] = permuted_off[n]
__global__ void scatter_offsets_kernel(const int *__restrict__ permuted_off, const int *__restrict__ order, int n,
                                       int *__restrict__ off) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i <= n;
         i += (long long)gridDim.x * blockDim.x)
        off[i < n ? order[i] : n] = permuted_off[i];
}

__global__ void check_classes_kernel(const int *__restrict__ cls, int n, int n_classes, int *bad) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        if (cls[i] < 0 || cls[i] >= n_classes) *bad = 1;
}

__global__ void max_nslots_kernel(const SplitRow *__restrict__ split, int n, int *out) {
    int m = 0;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        m = max(m, split[i].nslots);
    atomicMax(out, m);
}

// Copies the split rows with more than kWideSlots slots to `wide` (the order does not matter: every row is summed
// on its own); counter[0] ends as their number.  With wide == NULL only counts.
__global__ void select_wide_kernel(const SplitRow *__restrict__ split, int n, SplitRow *wide, int *counter) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const SplitRow r = split[i];
        if (r.nslots > kWideSlots) {
            const int at = atomicAdd(counter, 1);
            if (wide) wide[at] = r;
        }
    }
}

// Input check of a CSR: bad[0] = 1 + position of the first row pointer that is negative, decreasing or above nnz
// (position n_rows + 1 reports rowptr[n_rows] != nnz), bad[1] = 1 + position of the first column outside 0..n_cols-1.
// Both stay 0 for a well-formed input.  Positions are found with atomicMin on (position + 1) stored as unsigned - 1.
__global__ void check_csr_kernel(const int *__restrict__ rowptr, const int *__restrict__ col, int n_rows, int n_cols,
                                 int nnz, unsigned *bad) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long r = blockIdx.x * (long long)blockDim.x + threadIdx.x; r <= n_rows; r += stride) {
        const int a = rowptr[r];
        bool wrong = a < 0 || a > nnz;
        if (r == 0) wrong = wrong || a != 0;
        if (r < n_rows) wrong = wrong || rowptr[r + 1] < a;
        if (r == n_rows) wrong = wrong || a != nnz;
        if (wrong) atomicMin(bad, (unsigned)r);
    }
    for (long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x; k < nnz; k += stride) {
        const int c = col[k];
        if (c < 0 || c >= n_cols) atomicMin(bad + 1, (unsigned)k);
    }
}

// freq[c] = rowptr[c + 1] - rowptr[c]: how often column c occurs in the other orientation's CSR
__global__ void row_lengths_kernel(const int *__restrict__ rowptr, int n, int *__restrict__ freq) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        freq[i] = rowptr[i + 1] - rowptr[i];
}

// position_of[hot_ids[pos]] = pos for pos < n_hot (position_of was filled with -1)
__global__ void scatter_positions_kernel(const int *__restrict__ hot_ids, int n_hot, int *__restrict__ position_of) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_hot; i += (long long)gridDim.x * blockDim.x)
        position_of[hot_ids[i]] = (int)i;
}

// col[k] = kHotTag | position for the columns that have a position in the table of hot rows
__global__ void tag_columns_kernel(int *__restrict__ col, long long nnz, const int *__restrict__ position_of) {
    for (long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x; k < nnz; k += (long long)gridDim.x * blockDim.x) {
        const int pos = __ldg(position_of + col[k]);
        if (pos >= 0) col[k] = (int)(kHotTag | (unsigned)pos);
    }
}

// col[k] = place[col[k]]; stream entries keep their flags, placeholders stay as they are
__global__ void renumber_columns_kernel(int *__restrict__ col, long long n, const int *__restrict__ place, int with_flags) {
    for (long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x; k < n; k += (long long)gridDim.x * blockDim.x) {
        const unsigned c = (unsigned)col[k];
        if (!with_flags) col[k] = __ldg(place + c);
        else if (!(c & kPlaceholder)) col[k] = (int)((c & ~kColMask) | (unsigned)__ldg(place + (c & kColMask)));
    }
}

// plain[k] = the column a possibly tagged entry stands for
__global__ void untag_columns_kernel(const int *__restrict__ col, long long nnz, const int *__restrict__ hot_ids,
                                     int *__restrict__ plain) {
    for (long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x; k < nnz; k += (long long)gridDim.x * blockDim.x) {
        const unsigned c = (unsigned)col[k];
        plain[k] = (c & kHotTag) ? __ldg(hot_ids + (c & kHotMask)) : (int)c;
    }
}

static inline int grid_for(long long n, int block = 256, int cap = 148 * 32) {
    long long g = (n + block - 1) / block;
    if (g < 1) g = 1;
    if (g > cap) g = cap;
    return (int)g;
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------

static int env_int(const char *name, int dflt) {
    const char *s = getenv(name);
    if (!s || !*s) return dflt;
    const int v = atoi(s);
    return v > 0 ? v : dflt;
}

static void free_side(Side &s) {
    cudaFree(s.hot_ids);
    cudaFree(s.col_plain);
    cudaFree(s.rowptr);
    cudaFree(s.col);
    cudaFree(s.val);
    cudaFree(s.chunks);
    cudaFree(s.split);
    cudaFree(s.wide);
    cudaFree(s.s_rows);
    cudaFree(s.s_rowptr);
    cudaFree(s.s_col);
    cudaFree(s.s_val);
    cudaFree(s.s_range_row);
    s = Side();
}

// Build side[DRONE_OP_AT] from side[DRONE_OP_A] (arrays of A must be on the device).
static int build_transpose(drone_plan *p, cudaStream_t st) {
    const Side &a = p->side[DRONE_OP_A];
    Side &t = p->side[DRONE_OP_AT];
    const int n = p->n_rows, nnz = p->nnz;
    DRONE_CUDA(cudaMalloc(&t.rowptr, sizeof(int) * (size_t)(n + 1)));
    DRONE_CUDA(cudaMalloc(&t.col, sizeof(int) * (size_t)(nnz > 0 ? nnz : 1)));
    DRONE_CUDA(cudaMalloc(&t.val, sizeof(float) * (size_t)(nnz > 0 ? nnz : 1)));

    // row pointer of the transpose: histogram of destinations, then exclusive scan
    int *counts = nullptr;
    DRONE_CUDA(cudaMalloc(&counts, sizeof(int) * (size_t)(n + 1)));
    DRONE_CUDA(cudaMemsetAsync(counts, 0, sizeof(int) * (size_t)(n + 1), st));
    if (nnz > 0) {
        histogram_kernel<<<grid_for(nnz), 256, 0, st>>>(a.col, nnz, counts);
        DRONE_LAUNCH_CHECK("histogram_kernel");
    }
    size_t tmp_bytes = 0;
    void *tmp = nullptr;
    DRONE_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, counts, t.rowptr, n + 1, st));
    DRONE_CUDA(cudaMalloc(&tmp, tmp_bytes > 0 ? tmp_bytes : 1));
    DRONE_CUDA(cub::DeviceScan::ExclusiveSum(tmp, tmp_bytes, counts, t.rowptr, n + 1, st));
    count_launch();
    DRONE_CUDA(cudaStreamSynchronize(st));
    cudaFree(tmp);
    cudaFree(counts);

    if (nnz > 0) {
        // stable sort of edge ids by destination: sources stay ascending inside a row
        int *src = nullptr, *keys_alt = nullptr, *perm = nullptr, *perm_alt = nullptr, *keys = nullptr;
        DRONE_CUDA(cudaMalloc(&src, sizeof(int) * (size_t)nnz));
        DRONE_CUDA(cudaMalloc(&keys, sizeof(int) * (size_t)nnz));
        DRONE_CUDA(cudaMalloc(&keys_alt, sizeof(int) * (size_t)nnz));
        DRONE_CUDA(cudaMalloc(&perm, sizeof(int) * (size_t)nnz));
        DRONE_CUDA(cudaMalloc(&perm_alt, sizeof(int) * (size_t)nnz));
        expand_rows_kernel<<<grid_for(nnz), 256, 0, st>>>(a.rowptr, n, nnz, src);
        DRONE_LAUNCH_CHECK("expand_rows_kernel");
        iota_kernel<<<grid_for(nnz), 256, 0, st>>>(perm, nnz);
        DRONE_LAUNCH_CHECK("iota_kernel");
        DRONE_CUDA(cudaMemcpyAsync(keys, a.col, sizeof(int) * (size_t)nnz, cudaMemcpyDeviceToDevice, st));
        int end_bit = 1;
        while (end_bit < 31 && (1LL << end_bit) < (long long)n) ++end_bit;
        cub::DoubleBuffer<int> kb(keys, keys_alt);
        cub::DoubleBuffer<int> vb(perm, perm_alt);
        tmp_bytes = 0;
        DRONE_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, kb, vb, nnz, 0, end_bit, st));
        DRONE_CUDA(cudaMalloc(&tmp, tmp_bytes > 0 ? tmp_bytes : 1));
        DRONE_CUDA(cub::DeviceRadixSort::SortPairs(tmp, tmp_bytes, kb, vb, nnz, 0, end_bit, st));
        count_launch();
        gather_transposed_kernel<<<grid_for(nnz), 256, 0, st>>>(vb.Current(), src, a.val, nnz, t.col, t.val);
        DRONE_LAUNCH_CHECK("gather_transposed_kernel");
        DRONE_CUDA(cudaStreamSynchronize(st));
        cudaFree(tmp);
        cudaFree(src);
        cudaFree(keys);
        cudaFree(keys_alt);
        cudaFree(perm);
        cudaFree(perm_alt);
    }
    return DRONE_OK;
}

static void free_lists(Side &s) {
    cudaFree(s.chunks);
    cudaFree(s.split);
    cudaFree(s.wide);
    cudaFree(s.s_rows);
    cudaFree(s.s_rowptr);
    cudaFree(s.s_col);
    cudaFree(s.s_val);
    cudaFree(s.s_range_row);
    s.chunks = nullptr;
    s.split = s.wide = nullptr;
    s.s_rows = s.s_rowptr = s.s_col = s.s_range_row = nullptr;
    s.s_val = nullptr;
    s.ready = false;
}

// Exclusive scan of n+1 per-row counts into per-row offsets.  With row classes the offsets are class-major: rows are
// numbered in the order `p->row_order` lists them.  starts[c] = offset at which class c begins (starts[n_classes] =
// total).  scratch: 2 arrays of n+1 ints.
static int class_major_scan(const drone_plan *p, const int *cnt, int *off, int *scratch, void *tmp, size_t tmp_bytes,
                            int *starts, cudaStream_t st) {
    const int n = p->n_rows;
    if (!p->row_order) {
        DRONE_CUDA(cub::DeviceScan::ExclusiveSum(tmp, tmp_bytes, cnt, off, n + 1, st));
        count_launch();
        starts[0] = 0;
        DRONE_CUDA(cudaMemcpyAsync(&starts[1], off + n, sizeof(int), cudaMemcpyDeviceToHost, st));
        DRONE_CUDA(cudaStreamSynchronize(st));
        return DRONE_OK;
    }
    int *permuted = scratch, *permuted_off = scratch + (size_t)(n + 1);
    gather_counts_kernel<<<grid_for(n + 1), 256, 0, st>>>(cnt, p->row_order, n, permuted);
    DRONE_LAUNCH_CHECK("gather_counts_kernel");
    DRONE_CUDA(cub::DeviceScan::ExclusiveSum(tmp, tmp_bytes, permuted, permuted_off, n + 1, st));
    count_launch();
    scatter_offsets_kernel<<<grid_for(n + 1), 256, 0, st>>>(permuted_off, p->row_order, n, off);
    DRONE_LAUNCH_CHECK("scatter_offsets_kernel");
    for (int c = 0; c <= p->n_classes; ++c)
        DRONE_CUDA(cudaMemcpyAsync(&starts[c], permuted_off + p->class_start[c], sizeof(int), cudaMemcpyDeviceToHost, st));
    DRONE_CUDA(cudaStreamSynchronize(st));
    return DRONE_OK;
}

// Work lists of one orientation: chunks and split rows of the long rows, the flagged stream of the short rows.
static int build_work_lists(drone_plan *p, Side &s, cudaStream_t st) {
    const int n = p->n_rows;
    const int K = p->n_classes;
    struct Temp {        // freed on every way out
        int *buf = nullptr;
        void *scan = nullptr;
        ~Temp() { cudaFree(buf); cudaFree(scan); }
    } t;
    const size_t stride = (size_t)(n + 1);
    DRONE_CUDA(cudaMalloc(&t.buf, sizeof(int) * stride * 10));  // 10 arrays of n+1 ints: counts x4, offsets x4, scratch x2
    int *buf = t.buf;
    int *cnt[4] = {buf, buf + stride, buf + 2 * stride, buf + 3 * stride};
    int *off[4] = {buf + 4 * stride, buf + 5 * stride, buf + 6 * stride, buf + 7 * stride};
    int *scratch = buf + 8 * stride;
    count_chunks_kernel<<<grid_for(n + 1), 256, 0, st>>>(s.rowptr, n, p->short_row_limit, p->chunk_nnz,
                                                        cnt[0], cnt[1], cnt[2], cnt[3]);
    DRONE_LAUNCH_CHECK("count_chunks_kernel");
    size_t tmp_bytes = 0;
    DRONE_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, cnt[0], off[0], n + 1, st));
    DRONE_CUDA(cudaMalloc(&t.scan, tmp_bytes > 0 ? tmp_bytes : 1));
    void *tmp = t.scan;
    int rc;
    int slot_start[kMaxRowClasses + 1], long_start[kMaxRowClasses + 1];
    if ((rc = class_major_scan(p, cnt[0], off[0], scratch, tmp, tmp_bytes, s.chunk_start, st))) return rc;
    if ((rc = class_major_scan(p, cnt[1], off[1], scratch, tmp, tmp_bytes, slot_start, st))) return rc;
    if ((rc = class_major_scan(p, cnt[2], off[2], scratch, tmp, tmp_bytes, s.split_start, st))) return rc;
    if ((rc = class_major_scan(p, cnt[3], off[3], scratch, tmp, tmp_bytes, long_start, st))) return rc;
    s.n_classes = K;
    s.n_chunks = s.chunk_start[K];
    s.n_partials = slot_start[K];
    s.n_split_rows = s.split_start[K];
    s.n_long_rows = long_start[K];
    s.max_nslots = 0;
    s.n_wide_rows = 0;
    for (int c = 0; c <= K; ++c) s.wide_start[c] = 0;
    if (s.n_chunks > 0) {
        DRONE_CUDA(cudaMalloc(&s.chunks, sizeof(Chunk) * (size_t)s.n_chunks));
        DRONE_CUDA(cudaMalloc(&s.split, sizeof(SplitRow) * (size_t)(s.n_split_rows > 0 ? s.n_split_rows : 1)));
        fill_chunks_kernel<<<grid_for(n), 256, 0, st>>>(s.rowptr, n, p->chunk_nnz, cnt[0], off[0], off[1], off[2],
                                                       s.chunks, s.split);
        DRONE_LAUNCH_CHECK("fill_chunks_kernel");
        if (s.n_split_rows > 0) {
            int *d_max = scratch, *d_count = scratch + 1;
            DRONE_CUDA(cudaMemsetAsync(d_max, 0, 2 * sizeof(int), st));
            max_nslots_kernel<<<grid_for(s.n_split_rows), 256, 0, st>>>(s.split, s.n_split_rows, d_max);
            DRONE_LAUNCH_CHECK("max_nslots_kernel");
            DRONE_CUDA(cudaMemcpyAsync(&s.max_nslots, d_max, sizeof(int), cudaMemcpyDeviceToHost, st));
            // two passes over the classes in turn: count the wide rows, then copy them (class-major as well)
            for (int pass = 0; pass < 2; ++pass) {
                if (pass == 1) {
                    DRONE_CUDA(cudaStreamSynchronize(st));
                    s.n_wide_rows = s.wide_start[K];
                    if (s.n_wide_rows == 0) break;
                    DRONE_CUDA(cudaMalloc(&s.wide, sizeof(SplitRow) * (size_t)s.n_wide_rows));
                    DRONE_CUDA(cudaMemsetAsync(d_count, 0, sizeof(int), st));
                }
                for (int c = 0; c < K; ++c) {
                    const int lo = s.split_start[c], cn = s.split_start[c + 1] - lo;
                    if (cn > 0) {
                        select_wide_kernel<<<grid_for(cn), 256, 0, st>>>(s.split + lo, cn, pass ? s.wide : nullptr, d_count);
                        DRONE_LAUNCH_CHECK("select_wide_kernel");
                    }
                    if (pass == 0)
                        DRONE_CUDA(cudaMemcpyAsync(&s.wide_start[c + 1], d_count, sizeof(int), cudaMemcpyDeviceToHost, st));
                }
            }
        }
        DRONE_CUDA(cudaStreamSynchronize(st));
        // The chunk list ordered by each chunk's first column instead of by row: chunks that start in the same column
        // range are then worked on at about the same time, which keeps more of their gathers in L2 (measured: R-MAT-22
        // F = 32 1.053 -> 0.986 ms, R-MAT-20 symmetrised F = 64 0.645 -> 0.623 ms).  Every chunk writes its own row or
        // its own partial slot, so the order changes no result.  Plans without row classes and without a table of hot
        // rows only: on R-MAT-26 (operand 70 x L2) the row order, which mixes gathers that hit L2 with gathers that go to
        // HBM at all times, is the faster one (21.1 ms against 25.7 ms).  DRONE_CHUNK_ORDER=row / col forces either.
        const char *order = getenv("DRONE_CHUNK_ORDER");
        const bool by_column = order && order[0] == 'c' ? true : order && order[0] == 'r' ? false : s.hot_ids == nullptr;
        if (by_column && K == 1 && s.n_chunks > 1) {
            struct Sort {
                int *key = nullptr, *idx = nullptr, *key2 = nullptr, *idx2 = nullptr;
                Chunk *sorted = nullptr;
                void *tmp = nullptr;
                ~Sort() { cudaFree(key); cudaFree(idx); cudaFree(key2); cudaFree(idx2); cudaFree(tmp); cudaFree(sorted); }
            } o;
            const size_t nb = sizeof(int) * (size_t)s.n_chunks;
            DRONE_CUDA(cudaMalloc(&o.key, nb));
            DRONE_CUDA(cudaMalloc(&o.idx, nb));
            DRONE_CUDA(cudaMalloc(&o.key2, nb));
            DRONE_CUDA(cudaMalloc(&o.idx2, nb));
            DRONE_CUDA(cudaMalloc(&o.sorted, sizeof(Chunk) * (size_t)s.n_chunks));
            chunk_first_column_kernel<<<grid_for(s.n_chunks), 256, 0, st>>>(s.chunks, s.n_chunks, s.col, o.key, o.idx);
            DRONE_LAUNCH_CHECK("chunk_first_column_kernel");
            size_t sort_bytes = 0;
            DRONE_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, o.key, o.key2, o.idx, o.idx2, s.n_chunks, 0, 30, st));
            DRONE_CUDA(cudaMalloc(&o.tmp, sort_bytes > 0 ? sort_bytes : 1));
            DRONE_CUDA(cub::DeviceRadixSort::SortPairs(o.tmp, sort_bytes, o.key, o.key2, o.idx, o.idx2, s.n_chunks, 0, 30, st));
            count_launch();
            permute_chunks_kernel<<<grid_for(s.n_chunks), 256, 0, st>>>(s.chunks, o.idx2, s.n_chunks, o.sorted);
            DRONE_LAUNCH_CHECK("permute_chunks_kernel");
            DRONE_CUDA(cudaMemcpyAsync(s.chunks, o.sorted, sizeof(Chunk) * (size_t)s.n_chunks, cudaMemcpyDeviceToDevice, st));
            DRONE_CUDA(cudaStreamSynchronize(st));
        }
    }
    // stream of the short rows
    count_short_kernel<<<grid_for(n + 1), 256, 0, st>>>(s.rowptr, n, p->short_row_limit, cnt[0], cnt[1]);
    DRONE_LAUNCH_CHECK("count_short_kernel");
    int srow_start[kMaxRowClasses + 1], sent_start[kMaxRowClasses + 1];
    if ((rc = class_major_scan(p, cnt[0], off[0], scratch, tmp, tmp_bytes, srow_start, st))) return rc;
    if ((rc = class_major_scan(p, cnt[1], off[1], scratch, tmp, tmp_bytes, sent_start, st))) return rc;
    s.n_short_rows = srow_start[K];
    s.n_short_entries = sent_start[K];
    s.range_start[0] = 0;
    for (int c = 0; c < K; ++c)
        s.range_start[c + 1] = s.range_start[c] + ceil_div(sent_start[c + 1] - sent_start[c], kShortRangeNnz);
    s.n_short_ranges = s.range_start[K];
    if (s.n_short_rows > 0) {
        DRONE_CUDA(cudaMalloc(&s.s_rows, sizeof(int) * (size_t)s.n_short_rows));
        DRONE_CUDA(cudaMalloc(&s.s_rowptr, sizeof(int) * (size_t)(s.n_short_rows + 1)));
        DRONE_CUDA(cudaMalloc(&s.s_col, sizeof(int) * (size_t)s.n_short_entries));
        DRONE_CUDA(cudaMalloc(&s.s_val, sizeof(float) * (size_t)s.n_short_entries));
        DRONE_CUDA(cudaMalloc(&s.s_range_row, sizeof(int) * (size_t)(s.n_short_ranges + 1)));
        fill_short_kernel<<<grid_for(n), 256, 0, st>>>(s.rowptr, s.col, s.val, n, p->short_row_limit, off[0], off[1],
                                                      s.s_rows, s.s_rowptr, s.s_col, s.s_val);
        DRONE_LAUNCH_CHECK("fill_short_kernel");
        DRONE_CUDA(cudaMemcpyAsync(s.s_rowptr + s.n_short_rows, &s.n_short_entries, sizeof(int),
                                   cudaMemcpyHostToDevice, st));
        // ranges never straddle two classes; entry range_start[c] is also the end of class c-1's last range
        for (int c = 0; c < K; ++c) {
            const int nr = s.range_start[c + 1] - s.range_start[c];
            if (nr > 0) {
                short_ranges_kernel<<<grid_for(nr), 256, 0, st>>>(s.s_rowptr, srow_start[c], srow_start[c + 1],
                                                                 sent_start[c], nr, kShortRangeNnz,
                                                                 s.s_range_row + s.range_start[c]);
                DRONE_LAUNCH_CHECK("short_ranges_kernel");
            }
        }
        for (int c = 1; c <= K; ++c)   // after the kernels in stream order: the closing entry of every class
            DRONE_CUDA(cudaMemcpyAsync(s.s_range_row + s.range_start[c], &srow_start[c], sizeof(int),
                                       cudaMemcpyHostToDevice, st));
        DRONE_CUDA(cudaStreamSynchronize(st));
    }
    s.ready = true;
    return DRONE_OK;
}

// Tags the n_hot most often gathered columns of one orientation: col entries become kHotTag | position, hot_ids
// lists the columns by position (most frequent first, ties by ascending column).  `other_rowptr` is the row pointer of
// the opposite orientation (its row lengths are this orientation's column frequencies) or NULL (then they are counted).
static int tag_hot_columns(drone_plan *p, Side &s, const int *other_rowptr, int n_hot, cudaStream_t st) {
    const int n = p->n_rows;
    const long long nnz = p->nnz;
    struct Temp {
        int *freq = nullptr, *ids = nullptr, *freq_sorted = nullptr, *ids_sorted = nullptr, *position_of = nullptr;
        void *sort = nullptr;
        ~Temp() { cudaFree(freq); cudaFree(ids); cudaFree(freq_sorted); cudaFree(ids_sorted); cudaFree(position_of); cudaFree(sort); }
    } t;
    const size_t bytes = sizeof(int) * (size_t)(n + 1);
    DRONE_CUDA(cudaMalloc(&t.freq, bytes));
    DRONE_CUDA(cudaMalloc(&t.ids, bytes));
    DRONE_CUDA(cudaMalloc(&t.freq_sorted, bytes));
    DRONE_CUDA(cudaMalloc(&t.ids_sorted, bytes));
    DRONE_CUDA(cudaMalloc(&t.position_of, bytes));
    if (other_rowptr) {
        row_lengths_kernel<<<grid_for(n), 256, 0, st>>>(other_rowptr, n, t.freq);
        DRONE_LAUNCH_CHECK("row_lengths_kernel");
    } else {
        DRONE_CUDA(cudaMemsetAsync(t.freq, 0, bytes, st));
        histogram_kernel<<<grid_for(nnz), 256, 0, st>>>(s.col, (int)nnz, t.freq);
        DRONE_LAUNCH_CHECK("histogram_kernel");
    }
    iota_kernel<<<grid_for(n), 256, 0, st>>>(t.ids, n);
    DRONE_LAUNCH_CHECK("iota_kernel");
    size_t tmp_bytes = 0;
    DRONE_CUDA(cub::DeviceRadixSort::SortPairsDescending(nullptr, tmp_bytes, t.freq, t.freq_sorted, t.ids, t.ids_sorted, n, 0, 32, st));
    DRONE_CUDA(cudaMalloc(&t.sort, tmp_bytes > 0 ? tmp_bytes : 1));
    DRONE_CUDA(cub::DeviceRadixSort::SortPairsDescending(t.sort, tmp_bytes, t.freq, t.freq_sorted, t.ids, t.ids_sorted, n, 0, 32, st));
    count_launch();
    DRONE_CUDA(cudaMalloc(&s.hot_ids, sizeof(int) * (size_t)n_hot));
    DRONE_CUDA(cudaMemcpyAsync(s.hot_ids, t.ids_sorted, sizeof(int) * (size_t)n_hot, cudaMemcpyDeviceToDevice, st));
    s.n_hot = n_hot;
    DRONE_CUDA(cudaMemsetAsync(t.position_of, 0xff, bytes, st));
    scatter_positions_kernel<<<grid_for(n_hot), 256, 0, st>>>(s.hot_ids, n_hot, t.position_of);
    DRONE_LAUNCH_CHECK("scatter_positions_kernel");
    tag_columns_kernel<<<grid_for(nnz), 256, 0, st>>>(s.col, nnz, t.position_of);
    DRONE_LAUNCH_CHECK("tag_columns_kernel");
    DRONE_CUDA(cudaStreamSynchronize(st));
    return DRONE_OK;
}

// Checks d_index / d_col before anything indexes with them: a column outside the matrix would otherwise become an
// out-of-bounds access in the histogram of the transpose and in every gather of the aggregation.
int validate_csr(const char *who, const int *d_index, const int *d_col, int n_rows, int n_cols, int nnz, cudaStream_t st) {
    unsigned *d_bad = nullptr;
    unsigned h_bad[2] = {0xffffffffu, 0xffffffffu};
    DRONE_CUDA(cudaMalloc(&d_bad, sizeof(h_bad)));
    cudaError_t err = cudaMemcpyAsync(d_bad, h_bad, sizeof(h_bad), cudaMemcpyHostToDevice, st);
    if (err == cudaSuccess) {
        check_csr_kernel<<<grid_for((long long)(nnz > n_rows ? nnz : n_rows + 1)), 256, 0, st>>>(d_index, d_col, n_rows, n_cols, nnz, d_bad);
        err = cudaGetLastError();
        count_launch();
    }
    if (err == cudaSuccess) err = cudaMemcpyAsync(h_bad, d_bad, sizeof(h_bad), cudaMemcpyDeviceToHost, st);
    if (err == cudaSuccess) err = cudaStreamSynchronize(st);
    cudaFree(d_bad);
    if (err != cudaSuccess) return set_error(DRONE_E_CUDA, "%s: checking the CSR failed: %s", who, cudaGetErrorString(err));
    if (h_bad[0] != 0xffffffffu)
        return set_error(DRONE_E_INVALID, "%s: row pointer %u is not a valid CSR offset (must start at 0, never decrease, "
                         "and end at nnz=%d)", who, h_bad[0], nnz);
    if (h_bad[1] != 0xffffffffu)
        return set_error(DRONE_E_INVALID, "%s: column index at position %u is outside 0..%d", who, h_bad[1], n_cols - 1);
    return DRONE_OK;
}

static int plan_create_impl(drone_plan *p, int n_rows, int nnz, const int *d_index, const int *d_dst,
                            const float *d_values, const int *d_in_degree, const int *d_out_degree,
                            int orientations, cudaStream_t st, bool allow_tags) {
    DRONE_CUDA(cudaGetDevice(&p->device));
    {
        const int rc = validate_csr("drone_plan_create", d_index, d_dst, n_rows, n_rows, nnz, st);
        if (rc) return rc;
    }
    p->n_rows = n_rows;
    p->nnz = nnz;
    p->short_row_limit = env_int("DRONE_SHORT_ROW_LIMIT", 32);
    // Chunks of 256 nonzeros keep the serial work of one warp near ten microseconds;
    // very large graphs take longer chunks so that the chunk list stays below 1% of
    // the CSR stream.
    p->chunk_nnz = env_int("DRONE_CHUNK_NNZ", nnz > (1 << 28) ? 1024 : 256);
    if (p->chunk_nnz < p->short_row_limit) p->chunk_nnz = p->short_row_limit;
    const char *slice = getenv("DRONE_SLICE_WIDTH");       // read per plan, so that one process can hold plans of each kind
    p->slice_forced = (slice && *slice) ? atoi(slice) : -1;

    Side &a = p->side[DRONE_OP_A];
    const size_t nnz_alloc = (size_t)(nnz > 0 ? nnz : 1);
    DRONE_CUDA(cudaMalloc(&a.rowptr, sizeof(int) * (size_t)(n_rows + 1)));
    DRONE_CUDA(cudaMalloc(&a.col, sizeof(int) * nnz_alloc));
    DRONE_CUDA(cudaMalloc(&a.val, sizeof(float) * nnz_alloc));
    DRONE_CUDA(cudaMemcpyAsync(a.rowptr, d_index, sizeof(int) * (size_t)(n_rows + 1), cudaMemcpyDeviceToDevice, st));
    if (nnz > 0) {
        DRONE_CUDA(cudaMemcpyAsync(a.col, d_dst, sizeof(int) * (size_t)nnz, cudaMemcpyDeviceToDevice, st));
        if (d_values) {
            DRONE_CUDA(cudaMemcpyAsync(a.val, d_values, sizeof(float) * (size_t)nnz, cudaMemcpyDeviceToDevice, st));
        } else {
            csr_values_kernel<<<grid_for((long long)n_rows * 32), 256, 0, st>>>(a.rowptr, a.col, d_in_degree,
                                                                              d_out_degree, n_rows, a.val);
            DRONE_LAUNCH_CHECK("csr_values_kernel");
        }
    }
    DRONE_CUDA(cudaStreamSynchronize(st));

    const char *overlap = getenv("DRONE_SPMM_OVERLAP");   // "0" keeps every kernel of a call on the caller's stream
    if (!(overlap && overlap[0] == '0')) {
        DRONE_CUDA(cudaStreamCreateWithFlags(&p->side_stream, cudaStreamNonBlocking));
        DRONE_CUDA(cudaEventCreateWithFlags(&p->fork_event, cudaEventDisableTiming));
        DRONE_CUDA(cudaEventCreateWithFlags(&p->join_event, cudaEventDisableTiming));
    }
    DRONE_CUDA(cudaMalloc(&p->counter, sizeof(unsigned)));
    p->chunk_blocks_per_sm = env_int("DRONE_CHUNK_BLOCKS_PER_SM", 0);
    if (orientations & DRONE_PLAN_AT) {
        const int rc = build_transpose(p, st);
        if (rc) return rc;
    }
    // Table of hot rows: only for graphs whose dense operand is far larger than L2 at the usual widths (at least
    // DRONE_HOT_MIN_ROWS rows, default 2^23: measured on R-MAT graphs with 32 features, the table gains 10 % at 2^26
    // rows and loses 10 % at 2^22, where most gathers hit L2 anyway).  Its size is DRONE_HOT_TABLE_MB (default 64;
    // 0 switches it off); a position is tagged for as many rows as fit at a width of 32 floats, calls with wider rows
    // use a prefix of the positions.
    {
        const char *mb = getenv("DRONE_HOT_TABLE_MB");
        const long long table_mb = (mb && *mb) ? atoll(mb) : 64;
        const int min_rows = env_int("DRONE_HOT_MIN_ROWS", 1 << 23);
        long long n_hot = table_mb * (1LL << 20) / 128;
        if (n_hot > n_rows / 4) n_hot = n_rows / 4;
        if (allow_tags && table_mb > 0 && n_rows >= min_rows && n_rows < (1 << 29) && nnz > 0 && n_hot > 0) {
            Side &t = p->side[DRONE_OP_AT];
            int rc = DRONE_OK;
            if (orientations & DRONE_PLAN_AT) rc = tag_hot_columns(p, t, a.rowptr, (int)n_hot, st);
            if (rc == DRONE_OK && (orientations & DRONE_PLAN_A))
                rc = tag_hot_columns(p, a, (orientations & DRONE_PLAN_AT) ? t.rowptr : nullptr, (int)n_hot, st);
            if (rc) return rc;
            p->hot_table_bytes = (size_t)table_mb << 20;
            DRONE_CUDA(cudaMalloc(&p->hot_table, p->hot_table_bytes));
        }
    }
    if (orientations & DRONE_PLAN_AT) {
        const int rc = build_work_lists(p, p->side[DRONE_OP_AT], st);
        if (rc) return rc;
    }
    if (orientations & DRONE_PLAN_A) {
        int rc = build_work_lists(p, a, st);
        if (rc) return rc;
    } else {
        free_side(a);
    }
    return DRONE_OK;
}

}  // namespace drone

namespace drone {
int plan_order_columns_by_frequency(drone_plan *p, int orientation, const int *d_other_rowptr, int **d_place_out, void *stream) {
    cudaStream_t st = (cudaStream_t)stream;
    Side &s = p->side[orientation];
    if (!s.ready || s.hot_ids) return set_error(DRONE_E_STATE, "plan_order_columns_by_frequency: orientation not prepared, or tagged");
    const int n = p->n_rows;
    struct Temp {
        int *freq = nullptr, *ids = nullptr, *freq_sorted = nullptr, *ids_sorted = nullptr, *place = nullptr;
        void *sort = nullptr;
        ~Temp() { cudaFree(freq); cudaFree(ids); cudaFree(freq_sorted); cudaFree(ids_sorted); cudaFree(place); cudaFree(sort); }
    } t;
    const size_t bytes = sizeof(int) * (size_t)(n + 1);
    DRONE_CUDA(cudaMalloc(&t.freq, bytes));
    DRONE_CUDA(cudaMalloc(&t.ids, bytes));
    DRONE_CUDA(cudaMalloc(&t.freq_sorted, bytes));
    DRONE_CUDA(cudaMalloc(&t.ids_sorted, bytes));
    DRONE_CUDA(cudaMalloc(&t.place, bytes));
    row_lengths_kernel<<<grid_for(n), 256, 0, st>>>(d_other_rowptr, n, t.freq);
    DRONE_LAUNCH_CHECK("row_lengths_kernel");
    iota_kernel<<<grid_for(n), 256, 0, st>>>(t.ids, n);
    DRONE_LAUNCH_CHECK("iota_kernel");
    size_t tmp_bytes = 0;
    DRONE_CUDA(cub::DeviceRadixSort::SortPairsDescending(nullptr, tmp_bytes, t.freq, t.freq_sorted, t.ids, t.ids_sorted, n, 0, 32, st));
    DRONE_CUDA(cudaMalloc(&t.sort, tmp_bytes > 0 ? tmp_bytes : 1));
    DRONE_CUDA(cub::DeviceRadixSort::SortPairsDescending(t.sort, tmp_bytes, t.freq, t.freq_sorted, t.ids, t.ids_sorted, n, 0, 32, st));
    count_launch();
    scatter_positions_kernel<<<grid_for(n), 256, 0, st>>>(t.ids_sorted, n, t.place);
    DRONE_LAUNCH_CHECK("scatter_positions_kernel");
    if (p->nnz > 0) {
        renumber_columns_kernel<<<grid_for(p->nnz), 256, 0, st>>>(s.col, p->nnz, t.place, 0);
        DRONE_LAUNCH_CHECK("renumber_columns_kernel");
    }
    if (s.n_short_entries > 0) {
        renumber_columns_kernel<<<grid_for(s.n_short_entries), 256, 0, st>>>(s.s_col, s.n_short_entries, t.place, 1);
        DRONE_LAUNCH_CHECK("renumber_columns_kernel");
    }
    DRONE_CUDA(cudaStreamSynchronize(st));
    *d_place_out = t.place;
    t.place = nullptr;
    return DRONE_OK;
}
}  // namespace drone

using namespace drone;

extern "C" int drone_plan_destroy(drone_plan *p);
static int plan_create_checked(drone_plan **out, int n_rows, int nnz, const int *d_index, const int *d_dst,
                               const float *d_values, const int *d_in_degree, const int *d_out_degree,
                               int orientations, void *stream, bool allow_tags) {
    DRONE_REQUIRE(out != nullptr, "drone_plan_create: out is NULL");
    *out = nullptr;
    DRONE_REQUIRE(n_rows >= 0 && nnz >= 0, "drone_plan_create: negative size (n_rows=%d, nnz=%d)", n_rows, nnz);
    DRONE_REQUIRE(n_rows < (1 << 30), "drone_plan_create: n_rows=%d is above the 2^30-1 limit of the column encoding", n_rows);
    DRONE_REQUIRE(d_index != nullptr, "drone_plan_create: d_index is NULL");
    DRONE_REQUIRE(nnz == 0 || d_dst != nullptr, "drone_plan_create: d_dst is NULL with nnz=%d", nnz);
    DRONE_REQUIRE(nnz == 0 || d_values != nullptr || (d_in_degree && d_out_degree),
                  "drone_plan_create: need d_values or both degree arrays");
    DRONE_REQUIRE((orientations & DRONE_PLAN_BOTH) != 0 && (orientations & ~DRONE_PLAN_BOTH) == 0,
                  "drone_plan_create: orientations=%d is not a combination of DRONE_PLAN_A/AT", orientations);
    drone_plan *p = new (std::nothrow) drone_plan();
    if (!p) return set_error(DRONE_E_INVALID, "drone_plan_create: out of host memory");
    const int rc = plan_create_impl(p, n_rows, nnz, d_index, d_dst, d_values, d_in_degree, d_out_degree,
                                    orientations, (cudaStream_t)stream, allow_tags);
    if (rc != DRONE_OK) {
        drone_plan_destroy(p);
        return rc;
    }
    *out = p;
    return DRONE_OK;
}


namespace drone {
int plan_create_untagged(drone_plan **out, int n_rows, int nnz, const int *d_index, const int *d_dst, const float *d_values,
                         const int *d_in_degree, const int *d_out_degree, int orientations, void *stream) {
    return plan_create_checked(out, n_rows, nnz, d_index, d_dst, d_values, d_in_degree, d_out_degree, orientations,
                               stream, false);
}
}  // namespace drone

extern "C" {

int drone_version(void) { return 1001; }

const char *drone_last_error(void) { return last_error_buffer(); }

long long drone_kernel_launch_count(void) { return g_kernel_launches.load(); }

int drone_compute_csr_values(const int *d_index, const int *d_dst, const int *d_in_degree,
                             const int *d_out_degree, int n_rows, float *d_values, void *stream) {
    DRONE_REQUIRE(n_rows >= 0, "drone_compute_csr_values: n_rows=%d is negative", n_rows);
    if (n_rows == 0) return DRONE_OK;
    DRONE_REQUIRE(d_index && d_dst && d_in_degree && d_out_degree && d_values,
                  "drone_compute_csr_values: NULL pointer argument");
    csr_values_kernel<<<grid_for((long long)n_rows * 32), 256, 0, (cudaStream_t)stream>>>(
        d_index, d_dst, d_in_degree, d_out_degree, n_rows, d_values);
    DRONE_LAUNCH_CHECK("csr_values_kernel");
    return DRONE_OK;
}

int drone_plan_create(drone_plan **out, int n_rows, int nnz, const int *d_index, const int *d_dst,
                      const float *d_values, const int *d_in_degree, const int *d_out_degree,
                      int orientations, void *stream) {
    return plan_create_checked(out, n_rows, nnz, d_index, d_dst, d_values, d_in_degree, d_out_degree, orientations,
                               stream, true);
}

int drone_plan_destroy(drone_plan *p) {
    if (!p) return DRONE_OK;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(p->device);
    free_side(p->side[0]);
    free_side(p->side[1]);
    cudaFree(p->row_order);
    cudaFree(p->counter);
    cudaFree(p->hot_table);
    cudaFree(p->pad_x);
    cudaFree(p->pad_y);
    cudaFree(p->scratch);
    cudaFree(p->stage_x);
    cudaFree(p->stage_y);
    for (int s = 0; s < 2; ++s) {
        cudaFree(p->queue_x[s]);
        cudaFree(p->queue_y[s]);
        for (cudaEvent_t e : {p->queue_in[s], p->queue_done[s], p->queue_out[s]})
            if (e) cudaEventDestroy(e);
    }
    if (p->out_stream) cudaStreamDestroy(p->out_stream);
    if (p->own_stream) cudaStreamDestroy(p->own_stream);
    if (p->copy_stream) cudaStreamDestroy(p->copy_stream);
    for (cudaEvent_t e : p->half_loaded)
        if (e) cudaEventDestroy(e);
    if (p->side_stream) cudaStreamDestroy(p->side_stream);
    if (p->fork_event) cudaEventDestroy(p->fork_event);
    if (p->join_event) cudaEventDestroy(p->join_event);
    if (prev >= 0) cudaSetDevice(prev);
    delete p;
    return DRONE_OK;
}

int drone_plan_set_row_classes(drone_plan *p, const int *d_row_class, int n_classes, void *stream) {
    DRONE_REQUIRE(p != nullptr, "drone_plan_set_row_classes: plan is NULL");
    DRONE_REQUIRE(n_classes >= 1 && n_classes <= kMaxRowClasses, "drone_plan_set_row_classes: n_classes=%d outside 1..%d",
                  n_classes, kMaxRowClasses);
    DRONE_REQUIRE(n_classes == 1 || d_row_class != nullptr, "drone_plan_set_row_classes: d_row_class is NULL");
    struct Restore {      // the caller's device comes back on every way out
        int prev = -1, mine = -1;
        ~Restore() { if (prev >= 0 && prev != mine) cudaSetDevice(prev); }
    } dev;
    struct Temp {         // scratch of this call
        int *keys_out = nullptr, *rows = nullptr, *counts = nullptr, *order = nullptr;
        void *sort = nullptr;
        ~Temp() { cudaFree(keys_out); cudaFree(rows); cudaFree(counts); cudaFree(order); cudaFree(sort); }
    } t;
    cudaStream_t st = (cudaStream_t)stream;
    DRONE_CUDA(cudaGetDevice(&dev.prev));
    dev.mine = p->device;
    if (dev.prev != p->device) DRONE_CUDA(cudaSetDevice(p->device));
    const int n = p->n_rows;
    int h_counts[kMaxRowClasses] = {0};
    const bool classes = n_classes > 1 && n > 0;
    if (classes) {        // everything that can fail on the input happens before the plan is touched
        DRONE_CUDA(cudaMalloc(&t.keys_out, sizeof(int) * (size_t)n));
        DRONE_CUDA(cudaMalloc(&t.rows, sizeof(int) * (size_t)n));
        DRONE_CUDA(cudaMalloc(&t.order, sizeof(int) * (size_t)n));
        DRONE_CUDA(cudaMalloc(&t.counts, sizeof(int) * (kMaxRowClasses + 1)));
        DRONE_CUDA(cudaMemsetAsync(t.counts, 0, sizeof(int) * (kMaxRowClasses + 1), st));
        check_classes_kernel<<<grid_for(n), 256, 0, st>>>(d_row_class, n, n_classes, t.counts + kMaxRowClasses);
        DRONE_LAUNCH_CHECK("check_classes_kernel");
        int bad = 0;
        DRONE_CUDA(cudaMemcpyAsync(&bad, t.counts + kMaxRowClasses, sizeof(int), cudaMemcpyDeviceToHost, st));
        DRONE_CUDA(cudaStreamSynchronize(st));
        if (bad) return set_error(DRONE_E_INVALID, "drone_plan_set_row_classes: a row has a class outside 0..%d", n_classes - 1);
        histogram_kernel<<<grid_for(n), 256, 0, st>>>(d_row_class, n, t.counts);
        DRONE_LAUNCH_CHECK("histogram_kernel");
        iota_kernel<<<grid_for(n), 256, 0, st>>>(t.rows, n);
        DRONE_LAUNCH_CHECK("iota_kernel");
        int end_bit = 1;
        while ((1 << end_bit) < n_classes) ++end_bit;
        size_t tmp_bytes = 0;
        // stable: rows stay ascending inside a class
        DRONE_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, d_row_class, t.keys_out, t.rows, t.order, n, 0, end_bit, st));
        DRONE_CUDA(cudaMalloc(&t.sort, tmp_bytes > 0 ? tmp_bytes : 1));
        DRONE_CUDA(cub::DeviceRadixSort::SortPairs(t.sort, tmp_bytes, d_row_class, t.keys_out, t.rows, t.order, n, 0, end_bit, st));
        count_launch();
        DRONE_CUDA(cudaMemcpyAsync(h_counts, t.counts, sizeof(int) * kMaxRowClasses, cudaMemcpyDeviceToHost, st));
        DRONE_CUDA(cudaStreamSynchronize(st));
    }
    DRONE_CUDA(cudaDeviceSynchronize());   // calls that still read the lists must have finished
    cudaFree(p->row_order);
    p->row_order = nullptr;
    p->n_classes = 1;
    p->class_start[0] = 0;
    p->class_start[1] = n;
    if (classes) {
        p->row_order = t.order;
        t.order = nullptr;
        p->n_classes = n_classes;
        for (int c = 0; c < n_classes; ++c) p->class_start[c + 1] = p->class_start[c] + h_counts[c];
    }
    int rc = DRONE_OK;
    for (int o = 0; o < 2 && rc == DRONE_OK; ++o) {
        Side &s = p->side[o];
        if (!s.rowptr) continue;
        free_lists(s);
        rc = build_work_lists(p, s, st);
    }
    return rc;
}

int drone_plan_get_stats(const drone_plan *p, drone_plan_stats *out) {
    DRONE_REQUIRE(p && out, "drone_plan_get_stats: NULL argument");
    memset(out, 0, sizeof(*out));
    out->n_rows = p->n_rows;
    out->nnz = p->nnz;
    out->short_row_limit = p->short_row_limit;
    out->chunk_nnz = p->chunk_nnz;
    for (int o = 0; o < 2; ++o) {
        out->n_long_rows[o] = p->side[o].n_long_rows;
        out->n_chunks[o] = p->side[o].n_chunks;
        out->n_split_rows[o] = p->side[o].n_split_rows;
        out->n_partials[o] = p->side[o].n_partials;
    }
    out->scratch_bytes = (long long)p->scratch_bytes;
    out->last_slice_width = p->last_slice_width;
    out->hot_rows_tagged = std::max(p->side[0].n_hot, p->side[1].n_hot);
    return DRONE_OK;
}

int drone_plan_get_csr(const drone_plan *p, int orientation, const int **d_rowptr, const int **d_col,
                       const float **d_val) {
    DRONE_REQUIRE(p != nullptr, "drone_plan_get_csr: plan is NULL");
    DRONE_REQUIRE(orientation == DRONE_OP_A || orientation == DRONE_OP_AT,
                  "drone_plan_get_csr: orientation=%d", orientation);
    Side &s = const_cast<drone_plan *>(p)->side[orientation];
    DRONE_REQUIRE(s.ready, "drone_plan_get_csr: orientation %d was not prepared by drone_plan_create", orientation);
    if (s.hot_ids && !s.col_plain && p->nnz > 0) {   // tagged plan: the caller gets an untagged copy, made once
        int prev = -1;
        DRONE_CUDA(cudaGetDevice(&prev));
        if (prev != p->device) DRONE_CUDA(cudaSetDevice(p->device));
        cudaError_t err = cudaMalloc(&s.col_plain, sizeof(int) * (size_t)p->nnz);
        if (err == cudaSuccess) {
            untag_columns_kernel<<<grid_for(p->nnz), 256>>>(s.col, p->nnz, s.hot_ids, s.col_plain);
            err = cudaDeviceSynchronize();
            count_launch();
        }
        if (prev != p->device) cudaSetDevice(prev);
        if (err != cudaSuccess) return set_error(DRONE_E_CUDA, "drone_plan_get_csr: %s", cudaGetErrorString(err));
    }
    if (d_rowptr) *d_rowptr = s.rowptr;
    if (d_col) *d_col = s.col_plain ? s.col_plain : s.col;
    if (d_val) *d_val = s.val;
    return DRONE_OK;
}

int drone_host_alloc(void **out, size_t bytes) {
    DRONE_REQUIRE(out != nullptr, "drone_host_alloc: out is NULL");
    DRONE_CUDA(cudaHostAlloc(out, bytes > 0 ? bytes : 1, cudaHostAllocDefault));
    return DRONE_OK;
}

int drone_host_free(void *ptr) {
    if (ptr) DRONE_CUDA(cudaFreeHost(ptr));
    return DRONE_OK;
}

}  // extern "C"
