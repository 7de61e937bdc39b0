// common.cuh -- types shared by the C ABI layer and the kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ttb.h"

namespace ttb {

// One batched product, fully resolved: element pointers already include the
// view offsets, strides are in elements.
// lhs[b,i,k] = a[b*a_sb + i*a_si + k*a_sk]
// rhs[b,k,j] = b[b*b_sb + k*b_sk + j*b_sj]
// out[b,i,j] = c[b*c_sb + i*c_si + j*c_sj]
struct Problem {
    const void *a;
    const void *b;
    void *c;
    int64_t B, N, K, M;
    int64_t a_sb, a_si, a_sk;
    int64_t b_sb, b_sk, b_sj;
    int64_t c_sb, c_si, c_sj;
    int dtype;
    int device;
    cudaStream_t stream;
    // Fused epilogue: out = act(lhs.rhs + addend).  `addend` is a [B,N,M] view of the same dtype
    // whose strides may be 0 (a bias row or column broadcast) or may describe `c` itself
    // (accumulation into the output); nullptr = none.  Element pointer includes the offset.
    const void *d = nullptr;
    int64_t d_sb = 0, d_si = 0, d_sj = 0;
    int act = 0;  // TTB_ACT_NONE / TTB_ACT_RELU
};

// The same, as the kernels take it.
struct Epilogue {
    const void *d;
    long long d_sb, d_si, d_sj;
    int act;
};
inline Epilogue epilogue_of(const Problem &p) { return Epilogue{p.d, p.d_sb, p.d_si, p.d_sj, p.act}; }

// Error word written by kernels whose bounded waits gave up.  One per device,
// in ordinary global memory owned by the library.
struct DeviceStatus {
    unsigned int error;     // 0 = fine; otherwise a code naming the wait that gave up
    unsigned int detail;    // stage / tile that was being waited for
};

enum DeviceErrorCode : unsigned int {
    kErrNone = 0,
    kErrProducerWait = 1,
    kErrConverterWait = 2,
    kErrMmaWait = 3,
    kErrEpilogueWait = 4,
    kErrAccEmptyWait = 5,
    kErrForwardWait = 6,
    kErrStreamKWait = 7
};

void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);
void note_launch(int variant, int count);

// Returns the device-resident status word of `device` (allocated on first use).
int device_status_ptr(int device, DeviceStatus **out);
int sm_count(int device, int *out);
// Device buffer for the tcgen05 kernel's wait-cycle counters, or nullptr when the
// "tc_profile" option is off.
long long *profile_ptr(int device);
int profile_level();  // 0 off, 1 all counters, 2 the CTA lifetimes only (no clock reads inside the loops)
// Stream-K workspace (partial-sum slots, ready flags) of (device, stream).
int streamk_workspace(int device, cudaStream_t stream, float **partials, unsigned int **flags);
// The flags array holds 2 x 8 x SMs slot flags followed by this many arrival counters.
constexpr int kStreamKTickets = 65536;

// Per-dtype launchers.  Each returns a ttb_status.
// allow_skinny: products with one tiny dim may take the streaming kernels (automatic dispatch).
int launch_simt(const Problem &p, bool allow_splitk, bool allow_skinny = false);
struct F32Options {
    int terms = 2;      // 2 = hybrid split (TF32 big.big + two bf16 correction products, default);
                        // 3 = classic 3xTF32; 1 = one TF32 pass (test only)
    int k_chunk = 0;    // K blocks accumulated in TMEM before folding into registers (0 = all)
    int two_cta = 0;    // use CTA pairs (cta_group::2)
    int mask_big = 0;   // converters also rewrite the raw tile with its masked big part (test only)
    int dbg = 0;        // timing experiments (wrong results when non-zero)
    int streamk = -1;   // K blocks dealt out evenly over the SMs: -1 automatic, 0 never, 1 whenever possible
    int peer_tma = 1;   // fused all-gather: peers are reached by the epilogue's bulk tensor stores when possible
    int a_tmem = 0;     // hybrid split: A operands of the correction MMAs in tensor memory
    int extra_conv = 1; // pair form: the two spare warps of the producer warpgroup convert too
    int sk_pair = -1;   // paired stream-K (odd units walk their range backwards, tickets): -1 = with a fused
                        // all-gather that the epilogue sends, 0 = never, 1 = whenever stream-K allows
    int pieces = -1;    // piece schedule (every tile's K cut into this many parts, dealt out round-robin):
                        // -1 = four parts when an all-gather is fused into the product, 0 = never
};
// n_peers > 0 fuses an all-gather into the product: every finished tile is also stored into
// peer_c[i] (peer-mapped pointers to the other GPUs' C, same layout as p.c).
// mc_c: an NVLink multicast address of C (all-gather through the switch); excludes peer_c.
int launch_f32_tcgen05(const Problem &p, const F32Options &opt, int n_peers = 0, void *const *peer_c = nullptr,
                       void *mc_c = nullptr);
bool f32_tcgen05_eligible(const Problem &p, char *why, int why_len);
// two_cta: -1 = pick CTA pairs by shape, 0 = never, 1 = always.
int launch_i32_tcgen05(const Problem &p, int two_cta = -1, int dbg = 0);
bool i32_tcgen05_eligible(const Problem &p, char *why, int why_len);
int launch_f64_dmma(const Problem &p);
int measure_fp64_tensor_peak(int device, double *tflops);
bool f64_dmma_eligible(const Problem &p);

size_t dtype_size(int dtype);

}  // namespace ttb
