// ttb_api.cu -- the extern "C" layer: argument checking, view resolution,
// kernel dispatch, per-device workspaces and the host-buffer entry point.
//
// Mirrors the contract of tinytensor::cuda::batched_matmul_runner
// (tinytensor/tensor/backend/cuda/matmul.cu:26-78): rank-3 operands of one dtype
// on one device, result contiguous [B,N,M].  Differences, all deliberate:
//  * strided views are consumed as they are (the reference clones them first,
//    matmul.cu:40-41);
//  * lhs.size(0) == rhs.size(0) is checked (the reference reads B from lhs only,
//    matmul.cu:30);
//  * errors come back as status codes instead of assert/exit.
// There is no CPU fallback anywhere in this library.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "tma_desc.cuh"

namespace ttb {

namespace {
thread_local char g_err[512] = "";
thread_local int g_last_variant = 0;
thread_local long long g_launches = 0;

struct Options {
    int force_variant = TTB_VARIANT_AUTO;
    int tf32_terms = 2;  // 2 = hybrid split (TF32 + two bf16 corrections), 3 = 3xTF32, 1 = one TF32 pass
    int k_chunk = 0;
    int splitk = 1;
    int two_cta = -1;  // -1 = choose by shape
    int streamk = -1;  // -1 = when whole tiles would leave SMs idle, 0 = never, 1 = whenever possible
    int mask_big = 0;
    int tc_profile = 0;
    int tc_debug = 0;
    int conv_columns_mb = 2048;  // budget of conv2d's unrolled-columns workspace
    int int_tensor = 1;          // i32 products may use the int8 tensor-core kernel
    int peer_tma = 1;            // fused all-gather: epilogue tensor stores reach the peers (0: forwarding warps)
    int a_tmem = 0;              // f32 hybrid split: correction MMAs read their A operands from tensor memory
    int extra_conv = 1;          // f32 pair form: warps 2-3 convert 5/8 of every B tile
    int sk_pair = -1;            // f32 tensor-core kernel: paired stream-K (-1 automatic, 0 never, 1 whenever possible)
    int pieces = -1;             // f32 tensor-core kernel: piece schedule (-1 automatic, 0 never, n parts per tile)
};
Options g_opt;

constexpr int kMaxDevices = 64;
constexpr int kMaxStreamKSets = 8;
constexpr int kExtraSlots = 3;
constexpr int kHostChunks = 8;  // pipeline depth of the host-buffer entry point
struct StreamKSet {
    cudaStream_t stream;
    float *partials;
    unsigned int *flags;
};
// A cached scratch buffer.  `captured` records that it was handed to a launch while its stream
// was being captured: a CUDA graph may then hold the pointer for as long as the process lives.
struct Workspace {
    cudaStream_t stream;
    int slot;
    void *ptr;
    size_t bytes;
    bool captured;
};
constexpr int kProfCtas = 256;
constexpr size_t kProfBytes = kProfCtas * 8 * sizeof(long long);
struct DeviceState {
    bool init = false;
    int sms = 0;
    DeviceStatus *status = nullptr;
    std::vector<Workspace> ws;   // cached scratch buffers, one per (stream, slot)
    std::vector<void *> retired; // outgrown buffers a captured graph may still write through
    long long *prof = nullptr;  // kProfCtas x 8 wait-cycle counters of the tcgen05 kernel
    StreamKSet sk[kMaxStreamKSets];
    int sk_count = 0;
    void *stage[3] = {nullptr, nullptr, nullptr};
    cudaStream_t hs[3] = {nullptr, nullptr, nullptr};  // host-buffer entry point: upload, product, download
    cudaEvent_t hev[2 * kHostChunks] = {};
    bool hs_init = false;
    size_t stage_bytes[3] = {0, 0, 0};
    std::mutex host_mu;  // the host-buffer entry point owns the staging buffers and streams for a whole call
};
DeviceState g_dev[kMaxDevices];
std::atomic<bool> g_dev_ready[kMaxDevices];  // set once a device's state is initialised: the per-call fast path
std::mutex g_mu;
}  // namespace

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what) {
    set_error("%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
    return e == cudaErrorMemoryAllocation ? TTB_ENOMEM : TTB_ECUDA;
}

void note_launch(int variant, int count) {
    if (variant >= 0) g_last_variant = variant;
    g_launches += count;
}

size_t dtype_size(int dtype) {
    switch (dtype) {
        case TTB_U8: return 1;
        case TTB_I16: return 2;
        case TTB_I32: return 4;
        case TTB_I64: return 8;
        case TTB_F32: return 4;
        case TTB_F64: return 8;
        default: return 0;
    }
}

static int device_state(int device, DeviceState **out) {
    if (device >= 0 && device < kMaxDevices && g_dev_ready[device].load(std::memory_order_acquire)) {
        *out = &g_dev[device];  // every call after the first: no driver query, no lock
        return TTB_OK;
    }
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceCount");
    if (device < 0 || device >= n || device >= kMaxDevices) {
        set_error("device id %d out of range (have %d)", device, n);
        return TTB_EDEVICE;
    }
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState &d = g_dev[device];
    if (!d.init) {
        e = cudaSetDevice(device);
        if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
        e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
        e = cudaMalloc(&d.status, sizeof(DeviceStatus));
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(status)");
        e = cudaMemset(d.status, 0, sizeof(DeviceStatus));
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemset(status)");
        e = cudaMalloc(&d.prof, kProfBytes);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(profile)");
        e = cudaMemset(d.prof, 0, kProfBytes);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemset(profile)");
        d.init = true;
    }
    g_dev_ready[device].store(true, std::memory_order_release);
    *out = &d;
    return TTB_OK;
}

int device_status_ptr(int device, DeviceStatus **out) {
    DeviceState *d;
    int rc = device_state(device, &d);
    if (rc != TTB_OK) return rc;
    *out = d->status;
    return TTB_OK;
}

long long *profile_ptr(int device) {
    if (!g_opt.tc_profile) return nullptr;
    DeviceState *d;
    if (device_state(device, &d) != TTB_OK) return nullptr;
    return d->prof;
}

int profile_level() { return g_opt.tc_profile; }

size_t conv_columns_budget() { return static_cast<size_t>(g_opt.conv_columns_mb) << 20; }

int sm_count(int device, int *out) {
    DeviceState *d;
    int rc = device_state(device, &d);
    if (rc != TTB_OK) return rc;
    *out = d->sms;
    return TTB_OK;
}

// Stream-K workspace of the f32 tensor-core kernel: partial-sum slots and ready flags, one
// set per (device, stream) so that launches on different streams never share one.  A flag is
// raised by the unit that wrote partial sums and lowered by the unit that read them, so every
// flag is 0 again when a kernel ends and nothing has to be cleared between launches.
int streamk_workspace(int device, cudaStream_t stream, float **partials, unsigned int **flags) {
    DeviceState *d;
    int rc = device_state(device, &d);
    if (rc != TTB_OK) return rc;
    std::lock_guard<std::mutex> lk(g_mu);
    for (int i = 0; i < d->sk_count; ++i) {
        if (d->sk[i].stream == stream) {
            *partials = d->sk[i].partials;
            *flags = d->sk[i].flags;
            return TTB_OK;
        }
    }
    if (d->sk_count == kMaxStreamKSets) {
        set_error("stream-K workspaces for %d streams are in use on device %d", kMaxStreamKSets, device);
        return TTB_ELIMIT;
    }
    StreamKSet s{};
    s.stream = stream;
    // 32 x 128 fp32 slots, two per epilogue warp (at most 8 warps per SM's CTA): the contiguous
    // cut uses the first of each pair, the piece schedule both in turn.  Behind the slot flags,
    // kStreamKTickets arrival counters for the piece schedule (one per tile, CTA and warp).
    const size_t slots = static_cast<size_t>(d->sms) * 8 * 2;
    cudaError_t e = cudaMalloc(&s.partials, slots * 32 * 128 * sizeof(float));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(stream-K partials)");
    e = cudaMalloc(&s.flags, (slots + kStreamKTickets) * sizeof(unsigned int));
    if (e != cudaSuccess) {
        cudaFree(s.partials);
        return cuda_fail(e, "cudaMalloc(stream-K flags)");
    }
    e = cudaMemset(s.flags, 0, (slots + kStreamKTickets) * sizeof(unsigned int));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemset(stream-K flags)");
    d->sk[d->sk_count++] = s;
    *partials = s.partials;
    *flags = s.flags;
    return TTB_OK;
}

// Cached scratch buffers, one per (device, stream, slot), grown on demand.  Slot 0: split-K
// partial sums of the CUDA-core kernels; 1: conv2d's unrolled columns; 2: conv2d's
// weight-gradient partials; 3: conv2d's padded weights (the products conv2d runs may use slot 0
// at the same time, hence separate slots).  Keyed by stream so that calls on different streams
// of one device never share partial sums; calls on ONE stream are ordered by the stream.
// Growing replaces the buffer: cudaFree synchronises the device, so kernels that still use the
// old one have finished -- except launches recorded into a CUDA graph, which run again later.
// Hence a buffer that was handed out during a stream capture is retired (kept allocated) instead
// of freed, and growing DURING a capture is refused: run the call once before capturing.
int workspace_slot(int device, cudaStream_t stream, int slot, size_t bytes, void **out) {
    DeviceState *d;
    int rc = device_state(device, &d);
    if (rc != TTB_OK) return rc;
    if (slot < 0 || slot > kExtraSlots) {
        set_error("workspace slot %d out of range", slot);
        return TTB_EINVAL;
    }
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaError_t e = cudaStreamIsCapturing(stream, &cap);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamIsCapturing");
    const bool capturing = cap != cudaStreamCaptureStatusNone;
    std::lock_guard<std::mutex> lk(g_mu);
    Workspace *w = nullptr;
    for (auto &x : d->ws) {
        if (x.stream == stream && x.slot == slot) w = &x;
    }
    if (w == nullptr) {
        d->ws.push_back(Workspace{stream, slot, nullptr, 0, false});
        w = &d->ws.back();
    }
    if (w->bytes < bytes) {
        if (capturing) {
            set_error("a %zu-byte workspace is needed but only %zu bytes are cached for this stream: device memory "
                      "cannot be allocated while the stream is being captured; make the same call once before the capture",
                      bytes, w->bytes);
            return TTB_EUNSUPPORTED;
        }
        if (w->ptr != nullptr) {
            if (w->captured) {
                d->retired.push_back(w->ptr);
            } else {
                cudaFree(w->ptr);
            }
        }
        w->ptr = nullptr;
        w->bytes = 0;
        w->captured = false;
        const size_t want = slot == 0 ? bytes + (bytes >> 2) : bytes;
        e = cudaMalloc(&w->ptr, want);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(workspace)");
        w->bytes = want;
    }
    if (capturing) w->captured = true;
    *out = w->ptr;
    return TTB_OK;
}

int workspace_get(int device, cudaStream_t stream, size_t bytes, void **out) {
    return workspace_slot(device, stream, 0, bytes, out);
}

static int stage_get(DeviceState *d, int which, size_t bytes, void **out) {
    if (d->stage_bytes[which] < bytes) {
        if (d->stage[which]) cudaFree(d->stage[which]);
        d->stage[which] = nullptr;
        d->stage_bytes[which] = 0;
        cudaError_t e = cudaMalloc(&d->stage[which], bytes);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(staging)");
        d->stage_bytes[which] = bytes;
    }
    *out = d->stage[which];
    return TTB_OK;
}

// Streams and events of the host-buffer entry point's pipeline (created once per device).
static int host_streams(DeviceState *d) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (d->hs_init) return TTB_OK;
    for (int i = 0; i < 3; ++i) {
        cudaError_t e = cudaStreamCreateWithFlags(&d->hs[i], cudaStreamNonBlocking);
        if (e != cudaSuccess) return cuda_fail(e, "cudaStreamCreateWithFlags");
    }
    for (int i = 0; i < 2 * kHostChunks; ++i) {
        cudaError_t e = cudaEventCreateWithFlags(&d->hev[i], cudaEventDisableTiming);
        if (e != cudaSuccess) return cuda_fail(e, "cudaEventCreateWithFlags");
    }
    d->hs_init = true;
    return TTB_OK;
}

// Number of elements the view spans in its storage, from its first element.
static int64_t view_span(const ttb_view *v) {
    int64_t last = 0;
    for (int i = 0; i < 3; ++i) last += (v->size[i] - 1) * v->stride[i];
    return last + 1;
}

static int check_view(const ttb_view *v, const char *name) {
    if (!v || !v->data) {
        set_error("%s: null view or data pointer", name);
        return TTB_EINVAL;
    }
    if (v->offset < 0) {
        set_error("%s: negative offset %lld", name, static_cast<long long>(v->offset));
        return TTB_EINVAL;
    }
    for (int i = 0; i < 3; ++i) {
        if (v->size[i] < 1) {
            set_error("%s: size[%d] = %lld, must be >= 1", name, i, static_cast<long long>(v->size[i]));
            return TTB_ESHAPE;
        }
        if (v->stride[i] < 0) {
            set_error("%s: negative stride[%d] = %lld", name, i, static_cast<long long>(v->stride[i]));
            return TTB_EINVAL;
        }
        if (v->size[i] > (1LL << 31) - 1) {
            set_error("%s: size[%d] = %lld exceeds 2^31-1", name, i, static_cast<long long>(v->size[i]));
            return TTB_ESHAPE;
        }
    }
    return TTB_OK;
}

static int resolve(const ttb_view *lhs, const ttb_view *rhs, void *out, int64_t out_offset,
                   const int64_t out_stride[3], int dtype, int device, void *stream, Problem *p) {
    const size_t es = dtype_size(dtype);
    if (dtype == TTB_BOOL8) {
        set_error("matmul is not defined for bool8");
        return TTB_EDTYPE;
    }
    if (es == 0) {
        set_error("unknown dtype %d", dtype);
        return TTB_EDTYPE;
    }
    int rc = check_view(lhs, "lhs");
    if (rc != TTB_OK) return rc;
    rc = check_view(rhs, "rhs");
    if (rc != TTB_OK) return rc;
    if (!out) {
        set_error("out: null pointer");
        return TTB_EINVAL;
    }
    if (lhs->size[0] != rhs->size[0]) {
        set_error("batch sizes differ: lhs %lld vs rhs %lld", static_cast<long long>(lhs->size[0]),
                  static_cast<long long>(rhs->size[0]));
        return TTB_ESHAPE;
    }
    if (lhs->size[2] != rhs->size[1]) {
        set_error("inner dims differ: lhs[.,.,%lld] vs rhs[.,%lld,.]", static_cast<long long>(lhs->size[2]),
                  static_cast<long long>(rhs->size[1]));
        return TTB_ESHAPE;
    }
    p->B = lhs->size[0];
    p->N = lhs->size[1];
    p->K = lhs->size[2];
    p->M = rhs->size[2];
    // The reference holds element counts in `int` (tinytensor/tensor/shape.cpp:33).
    const long double out_elems = static_cast<long double>(p->B) * p->N * p->M;
    if (out_elems > 9.0e18L) {
        set_error("result too large");
        return TTB_ESHAPE;
    }
    p->a = static_cast<const char *>(lhs->data) + lhs->offset * es;
    p->b = static_cast<const char *>(rhs->data) + rhs->offset * es;
    p->a_sb = lhs->stride[0];
    p->a_si = lhs->stride[1];
    p->a_sk = lhs->stride[2];
    p->b_sb = rhs->stride[0];
    p->b_sk = rhs->stride[1];
    p->b_sj = rhs->stride[2];
    if (out_stride) {
        if (out_offset < 0 || out_stride[0] < 0 || out_stride[1] < 0 || out_stride[2] < 0) {
            set_error("out: negative offset or stride");
            return TTB_EINVAL;
        }
        p->c = static_cast<char *>(out) + out_offset * es;
        p->c_sb = out_stride[0];
        p->c_si = out_stride[1];
        p->c_sj = out_stride[2];
    } else {
        p->c = out;
        p->c_sb = p->N * p->M;
        p->c_si = p->M;
        p->c_sj = 1;
    }
    p->dtype = dtype;
    p->device = device;
    p->stream = static_cast<cudaStream_t>(stream);
    return TTB_OK;
}

static F32Options f32_options(bool two_cta) {
    F32Options o;
    o.terms = g_opt.tf32_terms;
    o.k_chunk = g_opt.k_chunk;
    o.two_cta = two_cta ? 1 : 0;
    o.mask_big = g_opt.mask_big;
    o.dbg = g_opt.tc_debug;
    o.streamk = g_opt.streamk;
    o.peer_tma = g_opt.peer_tma;
    o.a_tmem = g_opt.a_tmem;
    o.extra_conv = g_opt.extra_conv;
    o.pieces = g_opt.pieces;
    o.sk_pair = g_opt.sk_pair;
    return o;
}

// Same checks and view resolution for entry points defined in other translation units.
int resolve_problem(const ttb_view *lhs, const ttb_view *rhs, void *out, int dtype, int device, void *stream,
                    Problem *p) {
    return resolve(lhs, rhs, out, 0, nullptr, dtype, device, stream, p);
}

static int dispatch(const Problem &p);
int dispatch_problem(const Problem &p) { return dispatch(p); }

static int dispatch(const Problem &p) {
    DeviceState *d;
    int rc = device_state(p.device, &d);
    if (rc != TTB_OK) return rc;
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != p.device) {
        // The reference selects the device before every launch (kernel_launch.cuh:20).
        cudaError_t e = cudaSetDevice(p.device);
        if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    }
    const int force = g_opt.force_variant;
    char why[160] = "";
    switch (force) {
        case TTB_VARIANT_SIMT: return launch_simt(p, false);
        case TTB_VARIANT_SIMT_SPLITK: return launch_simt(p, true);
        case TTB_VARIANT_TCGEN05_3XTF32:
        case TTB_VARIANT_TCGEN05_2CTA:
            if (p.dtype != TTB_F32 || !f32_tcgen05_eligible(p, why, sizeof(why))) {
                set_error("forced tcgen05 variant cannot take this call: %s",
                          p.dtype != TTB_F32 ? "dtype is not f32" : why);
                return TTB_EUNSUPPORTED;
            }
            return launch_f32_tcgen05(p, f32_options(force == TTB_VARIANT_TCGEN05_2CTA));
        case TTB_VARIANT_DMMA_F64:
            if (p.dtype != TTB_F64 || !f64_dmma_eligible(p)) {
                set_error("forced DMMA variant cannot take this call");
                return TTB_EUNSUPPORTED;
            }
            return launch_f64_dmma(p);
        case TTB_VARIANT_TCGEN05_I8LIMB:
            if (!i32_tcgen05_eligible(p, why, sizeof(why))) {
                set_error("forced int8-plane tcgen05 variant cannot take this call: %s", why);
                return TTB_EUNSUPPORTED;
            }
            return launch_i32_tcgen05(p, g_opt.two_cta, g_opt.tc_debug);
        default: break;
    }
    // Automatic dispatch.
    if (p.dtype == TTB_F32) {
        // Tensor cores pay off once the product has enough work per output tile;
        // skinny outputs (a dim <= 16) are bandwidth-bound and go to the SIMT kernel.
        const bool big = p.N > 16 && p.M > 16 && p.K >= 16 &&
                         static_cast<double>(p.N) * p.M * p.K * p.B >= 128.0 * 128.0 * 64.0;
        if (big && f32_tcgen05_eligible(p, why, sizeof(why))) {
            // CTA pairs (256x256 tiles) halve shared-memory and L2 traffic per flop; they
            // pay off once the output is more than one 128-wide tile in both dims and there
            // are enough pair tiles to occupy a good part of the GPU.
            // Fewer pair tiles are fine when K is long: stream-K then deals the K blocks out over
            // all pairs (16 or more each).
            const long long pair_tiles = ((p.N + 255) / 256) * ((p.M + 255) / 256) * p.B;
            const long long kb = (p.K + 31) / 32;
            const bool enough = pair_tiles >= 24 || (g_opt.streamk != 0 && kb >= 64 && pair_tiles * kb / (d->sms / 2) >= 16);
            const bool pair = g_opt.two_cta < 0 ? (p.N > 128 && p.M > 128 && enough) : g_opt.two_cta != 0;
            return launch_f32_tcgen05(p, f32_options(pair));
        }
        return launch_simt(p, g_opt.splitk != 0, true);
    }
    if (p.dtype == TTB_F64) {
        if (p.N > 16 && p.M > 16 && p.K > 16 && f64_dmma_eligible(p)) return launch_f64_dmma(p);
        return launch_simt(p, g_opt.splitk != 0, true);
    }
    if (p.dtype == TTB_I32 && g_opt.int_tensor != 0) {
        // Ten int8 tensor-core products of byte planes beat the 32-bit multiply-add pipe once
        // the 128 x 128 tiles are reasonably full and there is some K to amortise the epilogue.
        const bool big = p.N >= 64 && p.M >= 64 && p.K >= 64 &&
                         static_cast<double>(p.N) * p.M * p.K * p.B >= 256.0 * 256.0 * 256.0;
        if (big && i32_tcgen05_eligible(p, why, sizeof(why))) return launch_i32_tcgen05(p, g_opt.two_cta, g_opt.tc_debug);
    }
    return launch_simt(p, g_opt.splitk != 0, true);
}

}  // namespace ttb

using namespace ttb;

extern "C" {

TTB_API int ttb_batched_matmul(const ttb_view *lhs, const ttb_view *rhs, void *out, int dtype, int device_id,
                               void *stream) {
    Problem p{};
    int rc = resolve(lhs, rhs, out, 0, nullptr, dtype, device_id, stream, &p);
    if (rc != TTB_OK) return rc;
    return dispatch(p);
}

TTB_API int ttb_batched_matmul_strided_out(const ttb_view *lhs, const ttb_view *rhs, void *out,
                                           int64_t out_offset, const int64_t out_stride[3], int dtype,
                                           int device_id, void *stream) {
    if (!out_stride) {
        set_error("out_stride: null pointer");
        return TTB_EINVAL;
    }
    Problem p{};
    int rc = resolve(lhs, rhs, out, out_offset, out_stride, dtype, device_id, stream, &p);
    if (rc != TTB_OK) return rc;
    return dispatch(p);
}

TTB_API int ttb_batched_matmul_fused(const ttb_view *lhs, const ttb_view *rhs, void *out, int64_t out_offset,
                                     const int64_t out_stride[3], const ttb_view *addend, int activation,
                                     int dtype, int device_id, void *stream) {
    Problem p{};
    int rc = resolve(lhs, rhs, out, out_offset, out_stride, dtype, device_id, stream, &p);
    if (rc != TTB_OK) return rc;
    if (activation != TTB_ACT_NONE && activation != TTB_ACT_RELU) {
        set_error("unknown activation %d", activation);
        return TTB_EINVAL;
    }
    if (activation == TTB_ACT_RELU && dtype != TTB_F32 && dtype != TTB_F64) {
        set_error("relu in the epilogue needs a floating-point dtype");
        return TTB_EDTYPE;
    }
    if (addend) {
        rc = check_view(addend, "addend");
        if (rc != TTB_OK) return rc;
        if (addend->size[0] != p.B || addend->size[1] != p.N || addend->size[2] != p.M) {
            set_error("addend is [%lld,%lld,%lld], the product is [%lld,%lld,%lld]",
                      static_cast<long long>(addend->size[0]), static_cast<long long>(addend->size[1]),
                      static_cast<long long>(addend->size[2]), static_cast<long long>(p.B),
                      static_cast<long long>(p.N), static_cast<long long>(p.M));
            return TTB_ESHAPE;
        }
        p.d = static_cast<const char *>(addend->data) + addend->offset * dtype_size(dtype);
        p.d_sb = addend->stride[0];
        p.d_si = addend->stride[1];
        p.d_sj = addend->stride[2];
    }
    p.act = activation;
    return dispatch(p);
}

TTB_API int ttb_matmul_allgather(const ttb_view *lhs, const ttb_view *rhs, void *out, int64_t out_offset,
                                 const int64_t out_stride[3], void *const *peer_out, int n_peers, int dtype,
                                 int device_id, void *stream) {
    if (!out_stride || n_peers < 0 || (n_peers > 0 && !peer_out)) {
        set_error("ttb_matmul_allgather: null out_stride / peer_out or negative n_peers");
        return TTB_EINVAL;
    }
    Problem p{};
    int rc = resolve(lhs, rhs, out, out_offset, out_stride, dtype, device_id, stream, &p);
    if (rc != TTB_OK) return rc;
    if (n_peers == 0) return dispatch(p);
    char why[160] = "";
    if (p.dtype != TTB_F32 || !f32_tcgen05_eligible(p, why, sizeof(why))) {
        set_error("ttb_matmul_allgather: the fused exchange exists for the f32 tensor-core kernel only (%s)",
                  p.dtype != TTB_F32 ? "dtype is not f32" : why);
        return TTB_EUNSUPPORTED;
    }
    // Argument checks first: they need no device.
    void *peers[16];
    if (n_peers > 15) {
        set_error("ttb_matmul_allgather: at most 15 peers, got %d", n_peers);
        return TTB_ELIMIT;
    }
    for (int i = 0; i < n_peers; ++i) {
        if (!peer_out[i]) {
            set_error("ttb_matmul_allgather: peer_out[%d] is null", i);
            return TTB_EINVAL;
        }
        peers[i] = static_cast<char *>(peer_out[i]) + out_offset * 4;
        // The kernel picks vector (16-byte) or scalar stores from THIS GPU's C and then uses the
        // same kind for every peer: a peer buffer aligned differently would fault in the kernel.
        if ((reinterpret_cast<uintptr_t>(peers[i]) & 15) != (reinterpret_cast<uintptr_t>(p.c) & 15)) {
            set_error("ttb_matmul_allgather: peer_out[%d] (%p) is not aligned like out (%p) modulo 16 bytes", i,
                      peers[i], p.c);
            return TTB_EINVAL;
        }
    }
    DeviceState *d;
    rc = device_state(p.device, &d);
    if (rc != TTB_OK) return rc;
    cudaError_t e = cudaSetDevice(p.device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    const long long pair_tiles = ((p.N + 255) / 256) * ((p.M + 255) / 256) * p.B;
    const bool pair = g_opt.two_cta < 0 ? (p.N > 128 && p.M > 128 && pair_tiles >= 24) : g_opt.two_cta != 0;
    return launch_f32_tcgen05(p, f32_options(pair), n_peers, peers);
}

TTB_API int ttb_matmul_allgather_multicast(const ttb_view *lhs, const ttb_view *rhs, void *out, int64_t out_offset,
                                           const int64_t out_stride[3], void *multicast_out, int dtype, int device_id,
                                           void *stream) {
    if (!out_stride || !multicast_out) {
        set_error("ttb_matmul_allgather_multicast: null out_stride / multicast_out");
        return TTB_EINVAL;
    }
    Problem p{};
    int rc = resolve(lhs, rhs, out, out_offset, out_stride, dtype, device_id, stream, &p);
    if (rc != TTB_OK) return rc;
    char why[160] = "";
    if (p.dtype != TTB_F32 || !f32_tcgen05_eligible(p, why, sizeof(why))) {
        set_error("ttb_matmul_allgather_multicast: the fused exchange exists for the f32 tensor-core kernel only (%s)",
                  p.dtype != TTB_F32 ? "dtype is not f32" : why);
        return TTB_EUNSUPPORTED;
    }
    DeviceState *d;
    rc = device_state(p.device, &d);
    if (rc != TTB_OK) return rc;
    cudaError_t e = cudaSetDevice(p.device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    const long long pair_tiles = ((p.N + 255) / 256) * ((p.M + 255) / 256) * p.B;
    const bool pair = g_opt.two_cta < 0 ? (p.N > 128 && p.M > 128 && pair_tiles >= 24) : g_opt.two_cta != 0;
    return launch_f32_tcgen05(p, f32_options(pair), 0, nullptr, static_cast<char *>(multicast_out) + out_offset * 4);
}

TTB_API int ttb_batched_matmul_host(const ttb_view *lhs, const ttb_view *rhs, void *out, int dtype,
                                    int device_id) {
    Problem p{};
    int rc = resolve(lhs, rhs, out, 0, nullptr, dtype, device_id, nullptr, &p);
    if (rc != TTB_OK) return rc;
    DeviceState *d;
    rc = device_state(device_id, &d);
    if (rc != TTB_OK) return rc;
    // One call at a time per device: the staging buffers, the three streams and their events are
    // shared, so a second host thread waits here until the first call has synchronised.
    std::lock_guard<std::mutex> host_lock(d->host_mu);
    cudaError_t e = cudaSetDevice(device_id);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    const size_t es = dtype_size(dtype);
    const size_t a_bytes = static_cast<size_t>(view_span(lhs)) * es;
    const size_t b_bytes = static_cast<size_t>(view_span(rhs)) * es;
    const size_t c_bytes = static_cast<size_t>(p.B) * p.N * p.M * es;
    void *da, *db, *dc;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if ((rc = stage_get(d, 0, a_bytes, &da)) != TTB_OK) return rc;
        if ((rc = stage_get(d, 1, b_bytes, &db)) != TTB_OK) return rc;
        if ((rc = stage_get(d, 2, c_bytes, &dc)) != TTB_OK) return rc;
    }
    // Only the span each view touches travels; strides are kept, so the device
    // side consumes the same (possibly permuted) view.
    const char *ha = static_cast<const char *>(p.a), *hb = static_cast<const char *>(p.b);
    p.a = da;
    p.b = db;
    p.c = dc;

    // Large products are pipelined in chunks so that the upload of chunk j+1, the product of
    // chunk j and the download of chunk j-1 overlap (PCIe is full duplex, the copy engines
    // run beside the SMs):
    //  * B == 1, lhs rows contiguous: chunks of output rows.  rhs goes up first, then blocks of
    //    lhs rows; each block's product is a block of rows of C, downloaded as soon as it is
    //    done.  Every copy is one contiguous span.
    //  * B == 1, only rhs rows contiguous: chunks of output columns, the same with the roles
    //    exchanged (the column blocks of rhs and C are 2-D copies).
    //  * B >= 4, batch-major operands: chunks of batches.
    // Anything else, and small products, take the plain path: copy, multiply, copy.
    const double work = 2.0 * static_cast<double>(p.B) * p.N * p.K * p.M;
    const int64_t a_one = (lhs->size[1] - 1) * lhs->stride[1] + (lhs->size[2] - 1) * lhs->stride[2] + 1;
    const int64_t b_one = (rhs->size[1] - 1) * rhs->stride[1] + (rhs->size[2] - 1) * rhs->stride[2] + 1;
    const bool by_rows = p.B == 1 && lhs->stride[2] == 1 && lhs->stride[1] >= p.K && p.N >= 1024 && work >= 4e10;
    const bool by_cols = !by_rows && p.B == 1 && rhs->stride[2] == 1 && rhs->stride[1] >= p.M && p.M >= 1024 &&
                         work >= 4e10;
    const bool by_batch = !by_rows && !by_cols && p.B >= 4 && lhs->stride[0] >= a_one && rhs->stride[0] >= b_one &&
                          work >= 4e10;
    if (by_rows || by_cols || by_batch) {
        rc = host_streams(d);
        if (rc != TTB_OK) return rc;
        cudaStream_t s_up = d->hs[0], s_mm = d->hs[1], s_down = d->hs[2];
        const int64_t extent = by_rows ? p.N : by_cols ? p.M : p.B;
        int nch = by_batch ? static_cast<int>(extent / 2) : static_cast<int>(extent / 1024);
        if (nch > kHostChunks) nch = kHostChunks;
        if (nch < 2) nch = 2;
        // chunk edges: multiples of 128 rows or columns / whole batches
        const int64_t gran = by_batch ? 1 : 128;
        const int64_t per = ((extent + nch - 1) / nch + gran - 1) / gran * gran;
        if (by_cols) {
            e = cudaMemcpyAsync(da, ha, a_bytes, cudaMemcpyHostToDevice, s_up);
            if (e != cudaSuccess) return cuda_fail(e, "H2D lhs");
        }
        if (by_rows) {
            e = cudaMemcpyAsync(db, hb, b_bytes, cudaMemcpyHostToDevice, s_up);
            if (e != cudaSuccess) return cuda_fail(e, "H2D rhs");
        }
        const Problem full = p;
        for (int c = 0; c < nch; ++c) {
            const int64_t x0 = c * per, x1 = (x0 + per < extent) ? x0 + per : extent;
            if (x0 >= extent) break;
            Problem q = full;
            q.stream = s_mm;
            if (by_rows) {
                const size_t a_off = static_cast<size_t>(x0 * lhs->stride[1]) * es;
                const size_t a_len = static_cast<size_t>((x1 - x0 - 1) * lhs->stride[1] + p.K) * es;
                e = cudaMemcpyAsync(static_cast<char *>(da) + a_off, ha + a_off, a_len, cudaMemcpyHostToDevice, s_up);
                if (e != cudaSuccess) return cuda_fail(e, "H2D lhs rows");
                q.a = static_cast<char *>(da) + a_off;
                q.c = static_cast<char *>(dc) + static_cast<size_t>(x0) * p.M * es;
                q.N = x1 - x0;
            } else if (by_cols) {
                const size_t pitch = static_cast<size_t>(rhs->stride[1]) * es;
                e = cudaMemcpy2DAsync(static_cast<char *>(db) + x0 * es, pitch, hb + x0 * es, pitch,
                                      static_cast<size_t>(x1 - x0) * es, static_cast<size_t>(p.K),
                                      cudaMemcpyHostToDevice, s_up);
                if (e != cudaSuccess) return cuda_fail(e, "H2D rhs block");
                q.b = static_cast<char *>(db) + x0 * es;
                q.c = static_cast<char *>(dc) + x0 * es;
                q.M = x1 - x0;
            } else {
                const size_t a_off = static_cast<size_t>(x0 * lhs->stride[0]) * es;
                const size_t b_off = static_cast<size_t>(x0 * rhs->stride[0]) * es;
                const size_t a_len = static_cast<size_t>((x1 - x0 - 1) * lhs->stride[0] + a_one) * es;
                const size_t b_len = static_cast<size_t>((x1 - x0 - 1) * rhs->stride[0] + b_one) * es;
                e = cudaMemcpyAsync(static_cast<char *>(da) + a_off, ha + a_off, a_len, cudaMemcpyHostToDevice, s_up);
                if (e != cudaSuccess) return cuda_fail(e, "H2D lhs batches");
                e = cudaMemcpyAsync(static_cast<char *>(db) + b_off, hb + b_off, b_len, cudaMemcpyHostToDevice, s_up);
                if (e != cudaSuccess) return cuda_fail(e, "H2D rhs batches");
                q.a = static_cast<char *>(da) + a_off;
                q.b = static_cast<char *>(db) + b_off;
                q.c = static_cast<char *>(dc) + static_cast<size_t>(x0) * p.N * p.M * es;
                q.B = x1 - x0;
            }
            e = cudaEventRecord(d->hev[2 * c], s_up);
            if (e != cudaSuccess) return cuda_fail(e, "cudaEventRecord");
            e = cudaStreamWaitEvent(s_mm, d->hev[2 * c], 0);
            if (e != cudaSuccess) return cuda_fail(e, "cudaStreamWaitEvent");
            rc = dispatch(q);
            if (rc != TTB_OK) {
                cudaDeviceSynchronize();
                return rc;
            }
            e = cudaEventRecord(d->hev[2 * c + 1], s_mm);
            if (e != cudaSuccess) return cuda_fail(e, "cudaEventRecord");
            e = cudaStreamWaitEvent(s_down, d->hev[2 * c + 1], 0);
            if (e != cudaSuccess) return cuda_fail(e, "cudaStreamWaitEvent");
            if (by_rows) {
                const size_t off = static_cast<size_t>(x0) * p.M * es;
                e = cudaMemcpyAsync(static_cast<char *>(out) + off, static_cast<char *>(dc) + off,
                                    static_cast<size_t>(x1 - x0) * p.M * es, cudaMemcpyDeviceToHost, s_down);
            } else if (by_cols) {
                const size_t pitch = static_cast<size_t>(p.M) * es;
                e = cudaMemcpy2DAsync(static_cast<char *>(out) + x0 * es, pitch, static_cast<char *>(dc) + x0 * es, pitch,
                                      static_cast<size_t>(x1 - x0) * es, static_cast<size_t>(p.N),
                                      cudaMemcpyDeviceToHost, s_down);
            } else {
                const size_t off = static_cast<size_t>(x0) * p.N * p.M * es;
                e = cudaMemcpyAsync(static_cast<char *>(out) + off, static_cast<char *>(dc) + off,
                                    static_cast<size_t>(x1 - x0) * p.N * p.M * es, cudaMemcpyDeviceToHost, s_down);
            }
            if (e != cudaSuccess) return cuda_fail(e, "D2H out block");
        }
        for (int i = 0; i < 3; ++i) {
            e = cudaStreamSynchronize(d->hs[i]);
            if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
        }
        return TTB_OK;
    }

    e = cudaMemcpyAsync(da, ha, a_bytes, cudaMemcpyHostToDevice, nullptr);
    if (e != cudaSuccess) return cuda_fail(e, "H2D lhs");
    e = cudaMemcpyAsync(db, hb, b_bytes, cudaMemcpyHostToDevice, nullptr);
    if (e != cudaSuccess) return cuda_fail(e, "H2D rhs");
    rc = dispatch(p);
    if (rc != TTB_OK) return rc;
    e = cudaMemcpyAsync(out, dc, c_bytes, cudaMemcpyDeviceToHost, nullptr);
    if (e != cudaSuccess) return cuda_fail(e, "D2H out");
    e = cudaStreamSynchronize(nullptr);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
    return TTB_OK;
}

TTB_API int ttb_partition(int64_t B, int64_t N, int64_t K, int64_t M, int world, int rank, int64_t col_align,
                          int64_t *begin, int64_t *end) {
    if (!begin || !end || world < 1 || rank < 0 || rank >= world) {
        set_error("ttb_partition: bad world/rank or null output");
        return TTB_EINVAL;
    }
    if (B < 1 || N < 1 || K < 1 || M < 1) {
        set_error("ttb_partition: sizes must be >= 1");
        return TTB_ESHAPE;
    }
    if (col_align < 1) col_align = 1;
    if (B > 1) {
        // Contiguous batch ranges, sizes differing by at most one.
        const int64_t base = B / world, rem = B % world;
        const int64_t b0 = rank * base + (rank < rem ? rank : rem);
        *begin = b0;
        *end = b0 + base + (rank < rem ? 1 : 0);
        return 0;
    }
    // Column blocks in units of col_align columns.
    const int64_t units = (M + col_align - 1) / col_align;
    const int64_t base = units / world, rem = units % world;
    const int64_t u0 = rank * base + (rank < rem ? rank : rem);
    const int64_t u1 = u0 + base + (rank < rem ? 1 : 0);
    int64_t c0 = u0 * col_align, c1 = u1 * col_align;
    if (c0 > M) c0 = M;
    if (c1 > M) c1 = M;
    *begin = c0;
    *end = c1;
    return 1;
}

TTB_API const char *ttb_last_error(void) { return g_err; }
TTB_API int ttb_last_variant(void) { return g_last_variant; }
TTB_API int64_t ttb_launch_count(void) { return g_launches; }

TTB_API const char *ttb_variant_name(int variant) {
    switch (variant) {
        case TTB_VARIANT_AUTO: return "auto";
        case TTB_VARIANT_SIMT: return "simt";
        case TTB_VARIANT_TCGEN05_3XTF32: return "tcgen05_3xtf32";
        case TTB_VARIANT_DMMA_F64: return "dmma_f64";
        case TTB_VARIANT_SIMT_SPLITK: return "simt_splitk";
        case TTB_VARIANT_TCGEN05_2CTA: return "tcgen05_3xtf32_2cta";
        case TTB_VARIANT_TCGEN05_I8LIMB: return "tcgen05_i8_byte_planes";
        case TTB_VARIANT_SIMT_SKINNY: return "simt_skinny";
        default: return "unknown";
    }
}

TTB_API int ttb_set_option(const char *key, int64_t value) {
    if (!key) {
        set_error("ttb_set_option: null key");
        return TTB_EINVAL;
    }
    if (!strcmp(key, "force_variant")) {
        if (value < 0 || value > TTB_VARIANT_TCGEN05_I8LIMB) {
            set_error("force_variant: %lld is not a variant", static_cast<long long>(value));
            return TTB_EINVAL;
        }
        g_opt.force_variant = static_cast<int>(value);
        return TTB_OK;
    }
    if (!strcmp(key, "tf32_terms")) {
        if (value < 1 || value > 3) {
            set_error("tf32_terms must be 1, 2 or 3");
            return TTB_EINVAL;
        }
        g_opt.tf32_terms = static_cast<int>(value);
        return TTB_OK;
    }
    if (!strcmp(key, "k_chunk")) {
        if (value < -1 || value > (1 << 20)) {
            set_error("k_chunk out of range");
            return TTB_EINVAL;
        }
        g_opt.k_chunk = static_cast<int>(value);
        return TTB_OK;
    }
    if (!strcmp(key, "splitk")) {
        g_opt.splitk = value != 0;
        return TTB_OK;
    }
    if (!strcmp(key, "two_cta")) {
        if (value < -1 || value > 1) {
            set_error("two_cta must be -1 (by shape), 0 or 1");
            return TTB_EINVAL;
        }
        g_opt.two_cta = static_cast<int>(value);
        return TTB_OK;
    }
    if (!strcmp(key, "mask_big")) {
        g_opt.mask_big = value != 0;
        return TTB_OK;
    }
    if (!strcmp(key, "tc_profile")) {
        g_opt.tc_profile = value == 2 ? 2 : (value != 0 ? 1 : 0);
        return TTB_OK;
    }
    if (!strcmp(key, "streamk")) {
        if (value < -1 || value > 1) {
            set_error("streamk must be -1 (automatic), 0 or 1");
            return TTB_EINVAL;
        }
        g_opt.streamk = static_cast<int>(value);
        return TTB_OK;
    }
    if (!strcmp(key, "tc_debug")) {
        g_opt.tc_debug = static_cast<int>(value);
        return TTB_OK;
    }
    if (!strcmp(key, "int_tensor")) {
        g_opt.int_tensor = value != 0;
        return TTB_OK;
    }
    if (!strcmp(key, "a_tmem")) {
        g_opt.a_tmem = value != 0;
        return TTB_OK;
    }
    if (!strcmp(key, "sk_pair")) {
        if (value < -1 || value > 1) {
            set_error("sk_pair takes -1 (automatic), 0 or 1");
            return TTB_EINVAL;
        }
        g_opt.sk_pair = static_cast<int>(value);
        return TTB_OK;
    }
    if (!strcmp(key, "pieces")) {
        if (value < -1 || value > 64) {
            set_error("pieces out of range (-1 automatic, 0 never, up to 64 parts per tile)");
            return TTB_EINVAL;
        }
        g_opt.pieces = static_cast<int>(value);
        return TTB_OK;
    }
    if (!strcmp(key, "extra_conv")) {
        g_opt.extra_conv = value != 0;
        return TTB_OK;
    }
    if (!strcmp(key, "peer_tma")) {
        g_opt.peer_tma = value != 0;
        return TTB_OK;
    }
    if (!strcmp(key, "conv_columns_mb")) {
        if (value < 1 || value > 65536) {
            set_error("conv_columns_mb must be 1..65536");
            return TTB_EINVAL;
        }
        g_opt.conv_columns_mb = static_cast<int>(value);
        return TTB_OK;
    }
    set_error("unknown option '%s'", key);
    return TTB_EINVAL;
}

TTB_API int64_t ttb_get_option(const char *key) {
    if (!key) return TTB_EINVAL;
    if (!strcmp(key, "force_variant")) return g_opt.force_variant;
    if (!strcmp(key, "tf32_terms")) return g_opt.tf32_terms;
    if (!strcmp(key, "k_chunk")) return g_opt.k_chunk;
    if (!strcmp(key, "splitk")) return g_opt.splitk;
    if (!strcmp(key, "two_cta")) return g_opt.two_cta;
    if (!strcmp(key, "mask_big")) return g_opt.mask_big;
    if (!strcmp(key, "tc_profile")) return g_opt.tc_profile;
    if (!strcmp(key, "streamk")) return g_opt.streamk;
    if (!strcmp(key, "conv_columns_mb")) return g_opt.conv_columns_mb;
    if (!strcmp(key, "int_tensor")) return g_opt.int_tensor;
    if (!strcmp(key, "peer_tma")) return g_opt.peer_tma;
    if (!strcmp(key, "a_tmem")) return g_opt.a_tmem;
    if (!strcmp(key, "extra_conv")) return g_opt.extra_conv;
    if (!strcmp(key, "pieces")) return g_opt.pieces;
    if (!strcmp(key, "sk_pair")) return g_opt.sk_pair;
    set_error("unknown option '%s'", key);
    return TTB_EINVAL;
}

TTB_API int ttb_device_count(void) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceCount");
    return n;
}

TTB_API int ttb_check_device(int device_id) {
    DeviceState *d;
    int rc = device_state(device_id, &d);
    if (rc != TTB_OK) return rc;
    cudaError_t e = cudaSetDevice(device_id);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSynchronize");
    DeviceStatus h{};
    e = cudaMemcpy(&h, d->status, sizeof(h), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(status)");
    if (h.error != 0) {
        cudaMemset(d->status, 0, sizeof(DeviceStatus));
        // A kernel that gave up may have left stream-K flags raised or tickets drawn: clear them all.
        for (int i = 0; i < d->sk_count; ++i)
            cudaMemset(d->sk[i].flags, 0, (static_cast<size_t>(d->sms) * 16 + kStreamKTickets) * sizeof(unsigned int));
        set_error("device %d: a bounded wait inside a kernel gave up (code %u, detail %u)", device_id, h.error,
                  h.detail);
        return TTB_ETIMEOUT;
    }
    return TTB_OK;
}

TTB_API int ttb_tc_profile(int device_id, int64_t *out, int ctas) {
    DeviceState *d;
    int rc = device_state(device_id, &d);
    if (rc != TTB_OK) return rc;
    if (!out || ctas < 1 || ctas > kProfCtas) {
        set_error("ttb_tc_profile: need an output array for 1..%d CTAs", kProfCtas);
        return TTB_EINVAL;
    }
    cudaError_t e = cudaSetDevice(device_id);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSynchronize");
    e = cudaMemcpy(out, d->prof, static_cast<size_t>(ctas) * 8 * sizeof(long long), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(profile)");
    return TTB_OK;
}

TTB_API void ttb_tensor_map_cache_stats(uint64_t *hits, uint64_t *misses) { tensor_map_cache_stats(hits, misses); }

TTB_API int ttb_measure_fp64_tensor_peak(int device_id, double *tflops) {
    if (!tflops) {
        set_error("ttb_measure_fp64_tensor_peak: null output");
        return TTB_EINVAL;
    }
    return measure_fp64_tensor_peak(device_id, tflops);
}

TTB_API int ttb_view_tma_eligible(const ttb_view *v, int dtype, int operand) {
    if (!v || (operand != 0 && operand != 1)) return 0;
    const size_t es = dtype_size(dtype);
    if (es == 0) return 0;
    for (int i = 0; i < 3; ++i)
        if (v->size[i] < 1 || v->stride[i] < 0) return 0;
    // Matrix dims of the view: (rows, cols) = (size[1], size[2]).  For lhs the
    // K dim is cols, for rhs it is rows; eligibility is symmetric in that.
    const uintptr_t base = reinterpret_cast<uintptr_t>(v->data) + static_cast<uintptr_t>(v->offset) * es;
    if (base % 16 != 0) return 0;
    const int64_t s1 = v->stride[1], s2 = v->stride[2];
    const int64_t n1 = v->size[1], n2 = v->size[2];
    auto ok_outer = [&](int64_t stride, int64_t n) { return n == 1 || (stride > 0 && (stride * es) % 16 == 0); };
    const bool inner2 = (s2 == 1 || n2 == 1) && ok_outer(s1, n1);
    const bool inner1 = (s1 == 1 || n1 == 1) && ok_outer(s2, n2);
    if (!inner1 && !inner2) return 0;
    if (v->size[0] > 1 && v->stride[0] != 0 && (v->stride[0] * es) % 16 != 0) return 0;
    return 1;
}

TTB_API int ttb_version(void) { return 100; }

}  // extern "C"
