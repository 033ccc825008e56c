// Host side of the aggregation: argument checks, column slicing, the choice of kernel variant and the entry points
// of the C ABI.  The kernels are in spmm_kernels.cuh, compiled once per variant in spmm_variants_*.cu.
#include "spmm_kernels.cuh"
#include "exchange.cuh"

#include <algorithm>
#include <cstdlib>
#include <mutex>

namespace drone {

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

// in_scale[i] = 1/sqrt(inDegree[i]), out_scale[i] = 1/sqrt(outDegree[i]) (0 for a degree of 0): the two factors of the
// reference's edge coefficient 1/sqrt(outDegree[u] * inDegree[v]).
__global__ void degree_scales_kernel(const int *__restrict__ in_deg, const int *__restrict__ out_deg, int n,
                                     float *__restrict__ in_scale, float *__restrict__ out_scale) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    in_scale[i] = in_deg[i] > 0 ? (float)(1.0 / sqrt((double)in_deg[i])) : 0.f;
    out_scale[i] = out_deg[i] > 0 ? (float)(1.0 / sqrt((double)out_deg[i])) : 0.f;
}

// padded[r, 0:F] = X[r, 0:F], padded[r, F:Fp] = 0          (Fp = F rounded up to a multiple of 4)
__global__ void pad_rows_kernel(const float *__restrict__ X, long long ldx, int n_rows, int F, int Fp,
                                float *__restrict__ padded) {
    const long long total = (long long)n_rows * Fp;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / Fp), j = (int)(i - (long long)r * Fp);
        padded[i] = j < F ? __ldg(X + (long long)r * ldx + j) : 0.f;
    }
}

// Y[row, 0:F] = padded[row, 0:F] for the rows of `rows` (rows == NULL: rows 0..n_rows-1)
__global__ void unpad_rows_kernel(const float *__restrict__ padded, int Fp, const int *__restrict__ rows, int n_rows, int F,
                                  float *__restrict__ Y, long long ldy) {
    const long long total = (long long)n_rows * F;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int k = (int)(i / F), j = (int)(i - (long long)k * F);
        const int r = rows ? __ldg(rows + k) : k;
        Y[(long long)r * ldy + j] = __ldcs(padded + (long long)r * Fp + j);
    }
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
    if (p->hot_table) return 0;                         // tagged plan: the hot rows are kept in L2 by their table
    const double l2_budget = 64e6;                      // about half of the 126 MB L2 for the gathered operand
    if ((double)p->n_rows * F * 4 <= l2_budget) return 0;
    for (int w : {128, 64}) {
        if (w < F && F % w == 0 && (double)p->n_rows * w * 4 <= l2_budget) return w;
    }
    return 0;
}

// What a call may ask for beyond the plain product (drone_spmm_opts of the C ABI, already checked).
struct CallOptions {
    int row_class = -1;
    bool unit_values = false;
    Epilogue epi;
    drone_xplan *push_up_to = nullptr;   // the call also sends the mirror rows of Y to their owners
};

static bool operands_allow_vec4(int F, long long ldx, long long ldy, const float *X, const float *Y) {
    return (F % 4 == 0) && (ldx % 4 == 0) && (ldy % 4 == 0) && ((reinterpret_cast<uintptr_t>(X) & 15) == 0) &&
           ((reinterpret_cast<uintptr_t>(Y) & 15) == 0);
}

// One launch sequence over columns [0, width) of the operands a.gather.X / a.Y point at.
static int run_variant(const drone_plan *p, const Side &s, SpmmArgs &a, bool vec4, int width, bool unit_values) {
    if (vec4) {
        a.nvec = width / 4;
    } else {
        a.nvec = width;
    }
    const bool tagged = s.hot_ids != nullptr;
    if (tagged) {
        // rows of the table at this width; positions beyond it fall back to X through hot_ids
        const long long fit = (long long)(p->hot_table_bytes / (sizeof(float) * (size_t)width));
        a.gather.hot = p->hot_table;
        a.gather.hot_ids = s.hot_ids;
        a.gather.hot_rows = (int)std::min<long long>(fit, s.n_hot);
        return unit_values ? spmm_dispatch_unit_hot(a, vec4) : spmm_dispatch_hot(a, vec4);
    }
    return unit_values ? spmm_dispatch_unit(a, vec4) : spmm_dispatch_plain(a, vec4);
}

static int spmm_impl(drone_plan *p, int orientation, int F, const float *X, long long ldx, float *Y,
                     long long ldy, cudaStream_t st, const CallOptions &opt = CallOptions()) {
    const Side &s = p->side[orientation];
    if (p->n_rows == 0) return DRONE_OK;
    bool vec4 = operands_allow_vec4(F, ldx, ldy, X, Y);
    // Rows that cannot be read as float4 where they lie: with padded staging reserved, work on padded copies.
    const int Fp = (F + 3) & ~3;
    const bool padded = !vec4 && p->pad_x != nullptr && Fp <= p->pad_width && F >= 5;
    float *const caller_Y = Y;
    const long long caller_ldy = ldy;
    const int caller_F = F;
    if (padded) {
        const long long total = (long long)p->n_rows * Fp;
        pad_rows_kernel<<<(int)std::min<long long>((total + 255) / 256, 148 * 16), 256, 0, st>>>(X, ldx, p->n_rows, F, Fp, p->pad_x);
        DRONE_LAUNCH_CHECK("pad_rows_kernel");
        X = p->pad_x;
        Y = p->pad_y;
        ldx = ldy = F = Fp;
        vec4 = true;
    }
    // The upward half of the exchange inside this call: the kernels store mirror rows into their owners' memory
    // (rows read as float4 where they lie), or the copy kernel sends them afterwards (any other layout).
    bool routed = false, send_after = false;
    const int2 *route = nullptr;
    float *const *peer_rows = nullptr;
    if (opt.push_up_to) {
        const int rc = p2p_route_begin(opt.push_up_to, p->n_rows, F, &route, &peer_rows);
        if (rc) return rc;
        routed = route != nullptr && vec4 && !padded;
        send_after = route != nullptr && !routed;
    }
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
    a.counter = p->counter;
    a.epi = opt.epi;
    a.st = st;
    a.side_stream = p->side_stream;
    a.fork = p->fork_event;
    a.join = p->join_event;
    a.row_class = opt.row_class;
    a.resident_per_sm = p->chunk_blocks_per_sm;
    a.gather.ldv = vec4 ? ldx / 4 : ldx;
    if (routed) {
        a.epi.route = route;
        a.epi.peer_rows = peer_rows;
        a.epi.route_nvec = F / 4;
    }
    for (int c0 = 0; c0 < F; c0 += width) {
        a.gather.X = X + c0;
        a.Y = Y + c0;
        a.epi.route_col0 = c0 / 4;
        const int rc = run_variant(p, s, a, vec4, width, opt.unit_values);
        if (rc) return rc;
    }
    if (routed) {
        const int rc = p2p_route_publish(opt.push_up_to, st);
        if (rc) return rc;
    }
    if (padded) {
        const int *rows = nullptr;
        int n_out = p->n_rows;
        if (opt.row_class >= 0 && p->row_order) {      // only the rows this call computed
            rows = p->row_order + p->class_start[opt.row_class];
            n_out = p->class_start[opt.row_class + 1] - p->class_start[opt.row_class];
        }
        if (n_out > 0) {
            const long long total = (long long)n_out * caller_F;
            unpad_rows_kernel<<<(int)std::min<long long>((total + 255) / 256, 148 * 16), 256, 0, st>>>(
                p->pad_y, Fp, rows, n_out, caller_F, caller_Y, caller_ldy);
            DRONE_LAUNCH_CHECK("unpad_rows_kernel");
        }
    }
    if (send_after) return p2p_push_up(opt.push_up_to, caller_Y, caller_F, (int)caller_ldy, st);
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

int drone_spmm_ex(drone_plan *p, int orientation, int F, const float *d_X, int ldx, float *d_Y, int ldy,
                  const drone_spmm_opts *opts, void *stream) {
    DRONE_REQUIRE(p != nullptr, "drone_spmm_ex: plan is NULL");
    DRONE_REQUIRE(orientation == DRONE_OP_A || orientation == DRONE_OP_AT, "drone_spmm_ex: orientation=%d", orientation);
    DRONE_REQUIRE(p->side[orientation].ready, "drone_spmm_ex: orientation %d was not prepared by drone_plan_create",
                  orientation);
    DRONE_REQUIRE(F >= 1 && F <= 1024, "drone_spmm_ex: feature width F=%d outside 1..1024", F);
    DRONE_REQUIRE(ldx >= F && ldy >= F, "drone_spmm_ex: leading dimensions (ldx=%d, ldy=%d) below F=%d", ldx, ldy, F);
    CallOptions opt;
    if (opts) {
        DRONE_REQUIRE(opts->epilogue == DRONE_EPILOGUE_NONE || opts->epilogue == DRONE_EPILOGUE_RELU,
                      "drone_spmm_ex: epilogue=%d is not a DRONE_EPILOGUE_* value", opts->epilogue);
        DRONE_REQUIRE(opts->row_class >= -1 && opts->row_class < p->n_classes,
                      "drone_spmm_ex: row_class=%d, the plan has %d classes", opts->row_class, p->n_classes);
        DRONE_REQUIRE(opts->unit_values == 0 || opts->unit_values == 1, "drone_spmm_ex: unit_values=%d is not 0 or 1",
                      opts->unit_values);
        opt.row_class = opts->row_class;
        opt.unit_values = opts->unit_values == 1;
        opt.epi.relu = opts->epilogue == DRONE_EPILOGUE_RELU;
        opt.epi.row_scale = opts->d_row_scale;
        opt.push_up_to = opts->push_up_to;
        DRONE_REQUIRE(!(opt.push_up_to && opt.epi.relu),
                      "drone_spmm_ex: DRONE_EPILOGUE_RELU cannot be combined with push_up_to (the sum over the replicas comes first)");
    }
    if (p->n_rows == 0) {
        if (opt.push_up_to) {      // a rank without rows still takes part in the exchange that follows
            const int2 *route = nullptr;
            float *const *peer_rows = nullptr;
            return p2p_route_begin(opt.push_up_to, 0, F, &route, &peer_rows);
        }
        return DRONE_OK;
    }
    DRONE_REQUIRE(d_X && d_Y, "drone_spmm_ex: NULL operand");
    DRONE_REQUIRE(d_X != d_Y, "drone_spmm_ex: X and Y must not alias");
    DeviceGuard guard;
    int rc = guard.enter(p->device);
    if (rc) return rc;
    return spmm_impl(p, orientation, F, d_X, ldx, d_Y, ldy, (cudaStream_t)stream, opt);
}

int drone_degree_scales(const int *d_in_degree, const int *d_out_degree, int n_rows, float *d_in_scale, float *d_out_scale,
                        void *stream) {
    DRONE_REQUIRE(n_rows >= 0, "drone_degree_scales: n_rows=%d is negative", n_rows);
    if (n_rows == 0) return DRONE_OK;
    DRONE_REQUIRE(d_in_degree && d_out_degree && d_in_scale && d_out_scale, "drone_degree_scales: NULL argument");
    degree_scales_kernel<<<ceil_div(n_rows, 256), 256, 0, (cudaStream_t)stream>>>(d_in_degree, d_out_degree, n_rows,
                                                                                 d_in_scale, d_out_scale);
    DRONE_LAUNCH_CHECK("degree_scales_kernel");
    return DRONE_OK;
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
    CallOptions opt;
    opt.row_class = row_class;
    const int rc = spmm_impl(p, orientation, F, d_X, ldx, d_Y, ldy, (cudaStream_t)stream, opt);
    if (dev != p->device) cudaSetDevice(dev);
    return rc;
}

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

// Pinned host operands of at least 64 columns (a multiple of 8): the call can run as two column halves, the
// second half's host-to-device copy and the first half's result going over PCIe at the same time, in opposite
// directions.  DRONE_HOST_PIPELINE=0 keeps the copy - compute - copy sequence.
static bool host_call_can_be_pipelined(const drone_plan *p, int F, const float *h_X, const float *h_Y) {
    static const bool enabled = [] {
        const char *v = getenv("DRONE_HOST_PIPELINE");
        return !(v && v[0] == '0');
    }();
    (void)p;
    if (!enabled || F < 64 || F % 8 != 0) return false;
    for (const void *ptr : {(const void *)h_X, (const void *)h_Y}) {
        cudaPointerAttributes attr;
        if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        if (attr.type != cudaMemoryTypeHost) return false;
    }
    void *mapped = nullptr;      // the kernels store into Y through its device alias: it must be mapped memory
    if (cudaHostGetDevicePointer(&mapped, const_cast<float *>(h_Y), 0) != cudaSuccess || mapped == nullptr) {
        cudaGetLastError();
        return false;
    }
    return (reinterpret_cast<uintptr_t>(h_X) & 15) == 0 && (reinterpret_cast<uintptr_t>(mapped) & 15) == 0;
}

// The two halves: half h of X is copied (strided, the DMA engine reads 4·F/2 bytes of every host row) into the
// plan's staging on the copy stream; the aggregation of that half starts when it has landed and stores its result
// rows straight into the caller's pinned Y (the kernels' stores go out over PCIe as they are issued), while the copy
// engine is already bringing the other half of X in.
static int spmm_host_pipelined(drone_plan *p, int orientation, int F, const float *h_X, float *h_Y) {
    if (!p->copy_stream) DRONE_CUDA(cudaStreamCreateWithFlags(&p->copy_stream, cudaStreamNonBlocking));
    for (cudaEvent_t &e : p->half_loaded)
        if (!e) DRONE_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    float *d_Y = nullptr;
    DRONE_CUDA(cudaHostGetDevicePointer((void **)&d_Y, h_Y, 0));
    const int w = F / 2;
    const size_t pitch = sizeof(float) * (size_t)F;
    for (int h = 0; h < 2; ++h) {
        DRONE_CUDA(cudaMemcpy2DAsync(p->stage_x + h * w, pitch, h_X + h * w, pitch, sizeof(float) * (size_t)w, (size_t)p->n_rows,
                                     cudaMemcpyHostToDevice, p->copy_stream));
        DRONE_CUDA(cudaEventRecord(p->half_loaded[h], p->copy_stream));
    }
    for (int h = 0; h < 2; ++h) {
        DRONE_CUDA(cudaStreamWaitEvent(p->own_stream, p->half_loaded[h], 0));
        const int rc = spmm_impl(p, orientation, w, p->stage_x + h * w, F, d_Y + h * w, F, p->own_stream);
        if (rc) return rc;
    }
    DRONE_CUDA(cudaStreamSynchronize(p->own_stream));
    return DRONE_OK;
}

int drone_plan_reserve(drone_plan *p, int max_features, int what) {
    DRONE_REQUIRE(p != nullptr, "drone_plan_reserve: plan is NULL");
    DRONE_REQUIRE(max_features >= 1 && max_features <= 1024, "drone_plan_reserve: max_features=%d outside 1..1024",
                  max_features);
    DeviceGuard guard;
    int rc = guard.enter(p->device);
    if (rc) return rc;
    const size_t slots = (size_t)std::max(p->side[0].n_partials, p->side[1].n_partials);
    if (slots > 0 && (rc = ensure_scratch(p, sizeof(float) * slots * (size_t)max_features))) return rc;
    DRONE_REQUIRE((what & ~(DRONE_RESERVE_HOST_OPERANDS | DRONE_RESERVE_PADDED_ROWS)) == 0,
                  "drone_plan_reserve: what=%d is not a combination of DRONE_RESERVE_* flags", what);
    if (what & DRONE_RESERVE_HOST_OPERANDS) {
        if ((rc = ensure_staging(p, sizeof(float) * (size_t)p->n_rows * (size_t)max_features))) return rc;
        if (!p->own_stream) DRONE_CUDA(cudaStreamCreateWithFlags(&p->own_stream, cudaStreamNonBlocking));
    }
    if ((what & DRONE_RESERVE_PADDED_ROWS) && p->n_rows > 0) {
        const int width = (max_features + 3) & ~3;
        if (width > p->pad_width) {
            DRONE_CUDA(cudaDeviceSynchronize());
            cudaFree(p->pad_x);
            cudaFree(p->pad_y);
            p->pad_x = p->pad_y = nullptr;
            p->pad_width = 0;
            const size_t bytes = sizeof(float) * (size_t)p->n_rows * (size_t)width;
            DRONE_CUDA(cudaMalloc(&p->pad_x, bytes));
            DRONE_CUDA(cudaMalloc(&p->pad_y, bytes));
            p->pad_width = width;
        }
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
    if (host_call_can_be_pipelined(p, F, h_X, h_Y)) return spmm_host_pipelined(p, orientation, F, h_X, h_Y);
    DRONE_CUDA(cudaMemcpyAsync(p->stage_x, h_X, bytes, cudaMemcpyHostToDevice, p->own_stream));
    if ((rc = spmm_impl(p, orientation, F, p->stage_x, F, p->stage_y, F, p->own_stream))) return rc;
    DRONE_CUDA(cudaMemcpyAsync(h_Y, p->stage_y, bytes, cudaMemcpyDeviceToHost, p->own_stream));
    DRONE_CUDA(cudaStreamSynchronize(p->own_stream));
    return DRONE_OK;
}

// Queue of host-operand calls.  Slot s = call number mod 2 owns one pair of staging buffers; three streams carry
// the three stages of a call (copy in, aggregation, copy out), chained by events, so that call k's operands come in
// while call k-1 is aggregated and call k-2's result goes out: PCIe is busy in both directions at once.
static int ensure_queue(drone_plan *p, size_t bytes) {
    if (!p->own_stream) DRONE_CUDA(cudaStreamCreateWithFlags(&p->own_stream, cudaStreamNonBlocking));
    if (!p->copy_stream) DRONE_CUDA(cudaStreamCreateWithFlags(&p->copy_stream, cudaStreamNonBlocking));
    if (!p->out_stream) DRONE_CUDA(cudaStreamCreateWithFlags(&p->out_stream, cudaStreamNonBlocking));
    for (int s = 0; s < 2; ++s)
        for (cudaEvent_t *e : {&p->queue_in[s], &p->queue_done[s], &p->queue_out[s]})
            if (!*e) DRONE_CUDA(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
    if (bytes <= p->queue_bytes) return DRONE_OK;
    DRONE_CUDA(cudaDeviceSynchronize());      // calls in flight use the buffers about to be replaced
    for (int s = 0; s < 2; ++s) {
        cudaFree(p->queue_x[s]);
        cudaFree(p->queue_y[s]);
        p->queue_x[s] = p->queue_y[s] = nullptr;
    }
    p->queue_bytes = 0;
    for (int s = 0; s < 2; ++s) {
        DRONE_CUDA(cudaMalloc(&p->queue_x[s], bytes));
        DRONE_CUDA(cudaMalloc(&p->queue_y[s], bytes));
    }
    p->queue_bytes = bytes;
    return DRONE_OK;
}

int drone_spmm_host_submit(drone_plan *p, int orientation, int F, const float *h_X, float *h_Y, long long *ticket) {
    DRONE_REQUIRE(p != nullptr, "drone_spmm_host_submit: plan is NULL");
    DRONE_REQUIRE(orientation == DRONE_OP_A || orientation == DRONE_OP_AT, "drone_spmm_host_submit: orientation=%d",
                  orientation);
    DRONE_REQUIRE(p->side[orientation].ready, "drone_spmm_host_submit: orientation %d was not prepared", orientation);
    DRONE_REQUIRE(F >= 1 && F <= 1024, "drone_spmm_host_submit: feature width F=%d outside 1..1024", F);
    DRONE_REQUIRE(ticket != nullptr, "drone_spmm_host_submit: ticket is NULL");
    DRONE_REQUIRE(p->n_rows == 0 || (h_X && h_Y), "drone_spmm_host_submit: NULL operand");
    DeviceGuard guard;
    int rc = guard.enter(p->device);
    if (rc) return rc;
    const long long k = p->submitted;
    const int s = (int)(k & 1);
    if (p->n_rows > 0) {
        const size_t bytes = sizeof(float) * (size_t)p->n_rows * (size_t)F;
        if ((rc = ensure_queue(p, bytes))) return rc;
        // the slot's previous call (k - 2) must have left it: its result copied out, hence its operands consumed
        if (k >= 2) DRONE_CUDA(cudaEventSynchronize(p->queue_out[s]));
        DRONE_CUDA(cudaMemcpyAsync(p->queue_x[s], h_X, bytes, cudaMemcpyHostToDevice, p->copy_stream));
        DRONE_CUDA(cudaEventRecord(p->queue_in[s], p->copy_stream));
        DRONE_CUDA(cudaStreamWaitEvent(p->own_stream, p->queue_in[s], 0));
        if ((rc = spmm_impl(p, orientation, F, p->queue_x[s], F, p->queue_y[s], F, p->own_stream))) return rc;
        DRONE_CUDA(cudaEventRecord(p->queue_done[s], p->own_stream));
        DRONE_CUDA(cudaStreamWaitEvent(p->out_stream, p->queue_done[s], 0));
        DRONE_CUDA(cudaMemcpyAsync(h_Y, p->queue_y[s], bytes, cudaMemcpyDeviceToHost, p->out_stream));
        DRONE_CUDA(cudaEventRecord(p->queue_out[s], p->out_stream));
    }
    *ticket = k;
    p->submitted = k + 1;
    return DRONE_OK;
}

int drone_spmm_host_wait(drone_plan *p, long long ticket) {
    DRONE_REQUIRE(p != nullptr, "drone_spmm_host_wait: plan is NULL");
    DRONE_REQUIRE(ticket >= 0 && ticket < p->submitted, "drone_spmm_host_wait: ticket %lld was not issued (%lld calls so far)",
                  ticket, p->submitted);
    if (p->n_rows == 0 || ticket + 2 < p->submitted) return DRONE_OK;     // a later submit on the slot waited for it
    DeviceGuard guard;
    const int rc = guard.enter(p->device);
    if (rc) return rc;
    DRONE_CUDA(cudaEventSynchronize(p->queue_out[ticket & 1]));
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
    const size_t need = (size_t)s.n_partials * (size_t)((F + 3) & ~3);   // the width the kernels may run at (padded rows)
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
        // same route as drone_spmm (padded staging when the plan has it, no column slices), with the partial sums in
        // the built-in array: the plan's own scratch pointer is swapped for the duration of the call
        float *const plan_scratch = p->scratch;
        const size_t plan_scratch_bytes = p->scratch_bytes;
        const int plan_slices = p->slice_forced;
        p->scratch = partials;
        p->scratch_bytes = DRONE_STATIC_SCRATCH_BYTES;
        p->slice_forced = 0;
        rc = drone::spmm_impl(p, orientation, F, d_X, ldx, d_Y, ldy, (cudaStream_t)stream);
        p->scratch = plan_scratch;
        p->scratch_bytes = plan_scratch_bytes;
        p->slice_forced = plan_slices;
    }
    if (dev != p->device) cudaSetDevice(dev);
    return rc;
}
