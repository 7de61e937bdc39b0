// gemm_f32_tcgen05.cu -- f32 batched GEMM on the 5th-generation tensor cores of sm_100a.
//
// C[b] = A[b] . B[b] in fp32-class accuracy from split operands.  kind::tf32 reads an fp32
// word and ignores its low 13 mantissa bits, so every operand x splits as x = big + small
// with big = x truncated to TF32 (which the tensor core derives by itself from the raw word)
// and small = x - big (exact in fp32).  Then A.B = big_A.big_B + small_A.B + big_A.small_B
// up to a term below 2^-20 relative.  Two ways to add the two correction terms:
//   hybrid (default, "tf32_terms" = 2): the converters write bf16(small) and bf16(x) tiles and
//       the corrections run as bf16 MMAs (kind::f16): small_A.bf16(B) + bf16(A).small_B.
//       A correction is ~2^-11 of the product, so bf16's 8 bits leave ~2^-19; a bf16 MMA costs
//       half the tensor cycles and half the shared-memory reads of a TF32 one.
//   3xTF32 ("tf32_terms" = 3): the converters write fp32 `small` tiles (rounded to nearest
//       TF32) and the corrections run as TF32 MMAs: small_A.big_B + big_A.small_B.
//
// The tensor core's fp32 accumulator does not round to nearest: summing all of a long K
// inside TMEM loses accuracy in proportion to K.  K is therefore cut into chunks (default
// 8 K-blocks = 256 elements); each chunk is accumulated in TMEM from zero and the chunk
// sums are added in fp32 registers (round-to-nearest) by the epilogue warps.
//
// Replaces matmul_kernel<float> of the reference
// (tinytensor/tensor/backend/cuda/kernel/matmul.cuh:27-151), a 64x64x8 CUDA-core
// kernel that needs contiguous operands.
//
// One CTA (persistent, static round-robin over tiles), roles by aligned warpgroup:
//   warp 0       TMA producer: cp.async.bulk.tensor loads of the raw fp32 A and B tiles
//                through tensor maps built from the operand's own strides (K-major or
//                MN-major, so transposed views need no copy);
//   warp 1       MMA issuer: one thread issues the tcgen05.mma instructions of a K block,
//                accumulating in TMEM: in the hybrid form the two corrections first, a
//                tcgen05.commit that releases the correction slot, then the TF32 product of the
//                raw tiles and the commit that releases the raw slot -- the converters' round
//                trip (slot free -> convert -> converted -> issue) runs behind the TF32 product.
//                A commit reaches the barrier of both CTAs of a pair (its multicast form).
//   warps 2-3    pair form: convert 5/8 of every B tile; or, in the fallback form of the fused
//                all-gather, forward finished tiles to the peer GPUs' C; idle in the one-CTA form.
//   epilogue WG  (one per 128 accumulator columns): tcgen05.ld each chunk sum, add into
//                registers, store C after the last chunk.  Two TMEM accumulators, so the
//                read-out of chunk i overlaps the MMAs of chunk i+1.
//   last WG(s)   (one in the pair form, two in the one-CTA form)
//                converters: read the raw tile from shared memory, write the correction
//                operands (bf16 tiles in their own swizzled layout, or fp32 `small` tiles at
//                the same offsets), fence.proxy.async, signal.
// Two forms: CG = 1, a 128x128 tile per CTA; CG = 2, a 256x256 tile per CTA pair
// (cta_group::2): each CTA loads 128 rows of A and 128 columns of B and owns 128 rows of
// the accumulator, which halves shared-memory and L2 traffic per flop.  No load carries a
// multicast qualifier; each CTA fetches its own tiles.
// All waits are bounded: a wait that gives up writes an error word and the CTA unwinds
// (TMEM freed) instead of hanging.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdio>
#include <cstring>

#include <mutex>

#include "common.cuh"
#include "ptx.cuh"
#include "tma_desc.cuh"

namespace ttb {
namespace {

using namespace ptx;

constexpr int BM = 128;              // lhs rows per CTA
constexpr int BNC = 128;             // rhs columns loaded per CTA
constexpr int BK = 32;               // fp32 per K block = 128 bytes = one swizzle row
constexpr int UMMA_K = 8;            // K of one tcgen05.mma kind::tf32
constexpr int STAGES = 4;             // raw ring: tiles as TMA delivers them (deep: hides load latency)
constexpr int SMALL_STAGES = 2;       // small ring: written by the converters just ahead of the MMAs
constexpr int TILE_BYTES = BM * BK * 4;        // 16 KiB: one operand tile
constexpr int RAW_BYTES = 2 * TILE_BYTES;      // raw A + raw B
constexpr int STAGE_BYTES = RAW_BYTES;         // one slot of either ring
constexpr int SMALL_RING_OFFSET = STAGES * STAGE_BYTES;
constexpr int OUT_STAGING_OFFSET = (STAGES + SMALL_STAGES) * STAGE_BYTES;  // epilogue store staging
constexpr int OUT_STAGING_WARP_BYTES = 32 * 128;  // 32 rows x 32 fp32 per epilogue warp
constexpr int OUT_STAGING_BYTES = 8 * OUT_STAGING_WARP_BYTES;              // up to 8 epilogue warps
constexpr int SMEM_BYTES = OUT_STAGING_OFFSET + OUT_STAGING_BYTES + 1024;  // + alignment slack
constexpr int MN_BOX_BYTES = 32 * BK * 4;      // one MN-major TMA box: 32 (MN) x BK (K)
constexpr int H_TILE_BYTES = BM * BK * 2;      // 8 KiB: one bf16 operand tile of the hybrid split
constexpr int DEFAULT_K_CHUNK = 8;             // K blocks summed inside TMEM
constexpr int kMaxPeers = 15;                  // fused all-gather: peers besides this GPU
// Profile slots per CTA: cycles the producer waited for a free raw slot, the MMA thread for a
// free accumulator / for converted tiles, converter thread 0 for a free small slot / for TMA data /
// spent converting, the first epilogue warp for a full accumulator, and the CTA's lifetime.
enum { kProfProducerEmpty = 0, kProfMmaAccEmpty, kProfMmaConv, kProfConvSmallEmpty, kProfConvFull, kProfConvBusy,
       kProfEpiAccFull, kProfTotal, kProfSlots };

template <int CG>
struct Cfg {
    static constexpr int EPI_WGS = CG;                 // one epilogue warpgroup per 128 columns
    // Converting a stage is what bounds the kernel.  The one-CTA form gets half the tensor work
    // out of a converted stage, so it spends its spare warp slots on a second converter
    // warpgroup (two warps per scheduler hide each other's shared-memory latencies).
    static constexpr int NUM_CONV_WARPS = CG == 1 ? 8 : 4;
    static constexpr int NUM_WARPS = 4 + 4 * EPI_WGS + NUM_CONV_WARPS;  // 16 in both forms
    static constexpr int NUM_THREADS = NUM_WARPS * 32;
    static constexpr int FIRST_EPI_WARP = 4;
    static constexpr int FIRST_CONV_WARP = 4 + 4 * EPI_WGS;
    static constexpr int EPI_REGS = CG == 1 ? 216 : 184;  // setmaxnreg budget of the epilogue warps
    static constexpr int UMMA_M = BM * CG;
    static constexpr int UMMA_N = BNC * CG;
    static constexpr int ACC_COLS = UMMA_N;            // fp32 columns of one accumulator
    static constexpr int TMEM_COLS = 512;              // accumulators + the A operands of the correction MMAs
    // Tensor memory map (512 columns).  A operands of the hybrid split's correction products
    // (args.a_tmem): SMALL_STAGES slots of 32 columns -- 16 columns bf16(small A), 16 columns
    // bf16(A), two K elements per column -- behind the accumulators.  The pair form's
    // accumulator is 256 columns wide, so with the A slots there is room for ONE (the epilogue
    // drains it between chunks); without them, and in the one-CTA form, there are two.
    static constexpr int A_SLOT_COLS = 32;
    static constexpr int TILE_M = BM * CG;             // rows of C per CTA (pair)
    static constexpr int TILE_N = BNC * CG;
};

struct alignas(64) TcArgs {
    CUtensorMap tmap_a;
    CUtensorMap tmap_b;
    CUtensorMap tmap_c;  // C as {M, N, B} with 32 x 32 boxes, for the epilogue's bulk tensor stores
    CUtensorMap tmap_peer[kMaxPeers];  // the same view of every peer GPU's C (fused all-gather)
    int c_tma;           // tmap_c is valid (C rows contiguous and 16-byte aligned)
    int c_batch_mul;     // 0 pins the batch coordinate (B == 1)
    float *c;
    long long c_sb, c_si, c_sj;
    const float *d;  // fused epilogue: addend view (bias row / column, or C itself), nullptr = none
    long long d_sb, d_si, d_sj;
    int act;         // TTB_ACT_*
    int N, M, K, B;
    int a_mn_major, b_mn_major;
    int a_batch_mul, b_batch_mul;
    int tiles_m, tiles_n, total_tiles;
    int a_tmem;    // hybrid split: the correction MMAs read their A operands from tensor memory
    int extra_conv;  // pair form, hybrid split: warps 2-3 convert too (set by the host when they have no
                     // forwarding to do)
    int terms;     // 3 = split-TF32, 1 = single pass (test only)
    int k_chunk;   // K blocks per TMEM accumulation chunk
    int mask_big;  // converters also overwrite the raw tile with its masked big part
    int streamk;   // 1: K blocks are dealt out evenly over the units (see above), else whole tiles
    int sk_tile0;  // stream-K: tiles [0, sk_tile0) stay whole; the rest is cut by K blocks
    float *sk_partials;       // stream-K workspace: per unit, CTA and epilogue warp 32 x 128 partial sums
    unsigned int *sk_flags;   // stream-K flags, one per unit, CTA and epilogue warp: 1 while partial sums wait
    // Piece schedule (pieces > 1, instead of streamk): every tile's K range is cut into `pieces`
    // parts (a power of two) of piece_len K blocks, the parts are dealt out round-robin (part
    // g = unit + i * units belongs to tile g / pieces), so the parts of a tile run at the same time on neighbouring
    // units and `units / pieces` tiles complete every piece_len K blocks, all through the kernel,
    // instead of one tile per unit at the very end.  The fused all-gather wants that: the
    // exchange of a completed tile overlaps the parts that follow, and only the last few tiles'
    // exchange is exposed.  Every part writes its sums to a slot of the stream-K workspace (two
    // per unit, used in turn) and takes a ticket of its tile; the part that takes the last
    // ticket adds all parts in part order (its own included, read back, so that the result does
    // not depend on which part came last), lowers their flags and stores the tile.
    int pieces, pieces_log2, piece_len;
    // Paired stream-K (sk_pair, with streamk): odd units walk their K-block range backwards, so a
    // tile shared by an even unit and the odd one after it is finished by both at the END of
    // their runs (one completion for two units) and a tile shared by an odd unit and the even one
    // after it at the START.  Half as many tiles complete at the very end of the kernel, which is
    // what the fused all-gather cannot hide.  Neither side knows which comes second, so both
    // write their sums (the two slots of a unit: 0 for a tail, 1 for a head) and draw a ticket
    // of the tile; the second adds the first's sums to its own (a + b = b + a: deterministic)
    // and stores.  Needs every range to be at least one tile long (two contributors per tile).
    int sk_pair;
    unsigned int *sk_tickets;  // arrival counters, one per tile, CTA and epilogue warp; 0 between launches
    int n_peers;   // fused all-gather: number of peer GPUs that receive every tile
    float *mc_c;   // fused all-gather through an NVLink multicast address of C (same offset and strides
                   // as `c`): one multimem.st reaches every GPU, this one included; nullptr = off
    int peer_tma;  // 1: the epilogue sends every box to the peers itself with bulk tensor stores
                   // (tmap_peer); 0: the forwarding warps copy finished tiles with st.global
    float *peer_c[kMaxPeers];  // their C, laid out exactly like `c` (same offset and strides)
    DeviceStatus *status;
    int dbg;          // test / timing switches; results are wrong when set.  bit 0: converter moves no
                      // data; 1: no proxy fence; 2: converter loads but does not store; 3: hybrid split
                      // adds bf16(A).bf16(B) instead of the corrections (layout check); 4: the first
                      // stage is never loaded (the bounded waits must run out and the kernel unwind);
                      // 5: the epilogue issues no global stores; 6: every unit gets no work (set-up and
                      // tear-down only) -- both for timing experiments
    long long *prof;  // optional: per-CTA wait-cycle counters (kProfSlots each), see ttb_tc_profile
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait that also leaves early when another role of this CTA gave up.
// Time limit: 2 s of %globaltimer.  CLUSTER selects the cluster-scope acquire, needed
// when arrivals come from the peer CTA.
template <bool CLUSTER>
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                              long long *waited = nullptr) {
    unsigned long long t0 = 0;
    const long long c0 = waited ? clock64() : 0;
    for (uint32_t i = 0;; ++i) {
        (void)CLUSTER;  // arrivals from the peer CTA are waited for like local ones
        const bool ok = mbar_try_wait(bar, parity);
        if (ok) {
            if (waited) *waited += clock64() - c0;
            return true;
        }

        if ((i & 63u) == 63u) {
            if (*abort_flag) return false;
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > 2000000000ull) return false;
        }
    }
}

__device__ __forceinline__ void report(DeviceStatus *st, volatile int *abort_flag, unsigned code, unsigned detail) {
    if (atomicCAS(&st->error, 0u, code) == 0u) st->detail = detail;
    *abort_flag = 1;
    __threadfence_block();
}

// Hybrid split of one 16-byte chunk of a raw operand tile (4 fp32): low part d = x - trunc_tf32(x)
// (exact) and x itself, both rounded to bf16, 8 bytes each, at offset `dst` of the two bf16 tiles.
// Inf and NaN travel through the TF32 product alone: in the bf16 tiles a non-finite element is
// replaced by zero, otherwise its low part would be NaN and 0 x Inf would turn a correction term
// into NaN where the fp32 result is +-Inf.  d is NaN exactly for Inf / NaN (Inf - Inf, NaN - NaN),
// so one packed compare of the bf16 pair with itself gives the keep-mask of both tiles.
__device__ __forceinline__ void hybrid_chunk(const uint4 x, uint8_t *s16, uint8_t *x16, int dst) {
    const float f0 = __uint_as_float(x.x), f1 = __uint_as_float(x.y);
    const float f2 = __uint_as_float(x.z), f3 = __uint_as_float(x.w);
    const float d0 = f0 - __uint_as_float(x.x & 0xFFFFE000u);
    const float d1 = f1 - __uint_as_float(x.y & 0xFFFFE000u);
    const float d2 = f2 - __uint_as_float(x.z & 0xFFFFE000u);
    const float d3 = f3 - __uint_as_float(x.w & 0xFFFFE000u);
    const __nv_bfloat162 p0 = __floats2bfloat162_rn(d0, d1), p1 = __floats2bfloat162_rn(d2, d3);
    const __nv_bfloat162 q0 = __floats2bfloat162_rn(f0, f1), q1 = __floats2bfloat162_rn(f2, f3);
    const uint32_t m0 = __heq2_mask(p0, p0), m1 = __heq2_mask(p1, p1);
    *reinterpret_cast<uint2 *>(s16 + dst) = make_uint2(*reinterpret_cast<const uint32_t *>(&p0) & m0,
                                                       *reinterpret_cast<const uint32_t *>(&p1) & m1);
    *reinterpret_cast<uint2 *>(x16 + dst) = make_uint2(*reinterpret_cast<const uint32_t *>(&q0) & m0,
                                                       *reinterpret_cast<const uint32_t *>(&q1) & m1);
}

// The same split without the keep-mask, for the common case of finite operands: the caller passes
// two accumulators that stay finite as long as every element seen was finite (a product of two low
// parts is finite for finite inputs; the low part of Inf / NaN is NaN, and NaN survives every
// fused multiply-add after it).  A thread whose accumulators are not finite afterwards converts its
// chunks again with hybrid_chunk.  This takes the compare and four ANDs per chunk off the ALU pipe,
// which is the pipe the converter warps keep busiest; the accumulators run on the FMA pipe.
__device__ __forceinline__ void hybrid_chunk_unmasked(const uint4 x, uint8_t *s16, uint8_t *x16, int dst, float &za,
                                                      float &zb) {
    const float f0 = __uint_as_float(x.x), f1 = __uint_as_float(x.y);
    const float f2 = __uint_as_float(x.z), f3 = __uint_as_float(x.w);
    const float d0 = f0 - __uint_as_float(x.x & 0xFFFFE000u);
    const float d1 = f1 - __uint_as_float(x.y & 0xFFFFE000u);
    const float d2 = f2 - __uint_as_float(x.z & 0xFFFFE000u);
    const float d3 = f3 - __uint_as_float(x.w & 0xFFFFE000u);
    const __nv_bfloat162 p0 = __floats2bfloat162_rn(d0, d1), p1 = __floats2bfloat162_rn(d2, d3);
    const __nv_bfloat162 q0 = __floats2bfloat162_rn(f0, f1), q1 = __floats2bfloat162_rn(f2, f3);
    za = fmaf(d0, d1, za);
    zb = fmaf(d2, d3, zb);
    *reinterpret_cast<uint2 *>(s16 + dst) =
        make_uint2(*reinterpret_cast<const uint32_t *>(&p0), *reinterpret_cast<const uint32_t *>(&p1));
    *reinterpret_cast<uint2 *>(x16 + dst) =
        make_uint2(*reinterpret_cast<const uint32_t *>(&q0), *reinterpret_cast<const uint32_t *>(&q1));
}

// The small slot a converter is about to fill was last read by the MMAs of the K block
// SMALL_STAGES back.  Their completion arrives on that K block's raw-slot barrier (one
// tcgen05.commit per K block serves both rings): which barrier that is, and the parity of the
// phase it completes, from the raw ring's position (stage, phase) of the K block being converted.
// On the first SMALL_STAGES K blocks the parity names the phase before the barrier's first,
// which counts as complete.
__device__ __forceinline__ int small_release_bar(int stage) { return (stage + STAGES - SMALL_STAGES) % STAGES; }
__device__ __forceinline__ uint32_t small_release_parity(int stage, uint32_t phase) {
    return stage >= SMALL_STAGES ? phase : (phase ^ 1u);
}

__device__ __forceinline__ bool all_finite(float za, float zb) { return fabsf(za + zb) <= 3.0e38f; }

// Where the 16-byte chunk `ci` of a raw operand tile goes in the bf16 tiles, from undoing the raw
// tile's swizzle:
//  K-major  raw rows are 128 B with 16-B chunks XORed by (row & 7); the bf16 row is 64 B with
//           16-B chunks XORed by ((row >> 1) & 3) -- the XORs cancel up to the low bit, which
//           picks the half of the 16-byte chunk.
//  MN-major raw rows (one K index, 32 MN values) have 32-B chunks XORed by (k & 3); the bf16 row
//           is 64 B with 16-B chunks XORed by ((k >> 1) & 3).
// Chunks 8 rows (64 chunks) apart land 512 bytes apart in both layouts.
__device__ __forceinline__ int hybrid_dst(int ci, bool mn_major) {
    if (!mn_major) {
        const int r = ci >> 3, cp = ci & 7;
        return r * 64 + (cp >> 1) * 16 + (((cp ^ r) & 1) << 3);
    }
    const int box = ci >> 8, kr = (ci & 255) >> 3, c16 = ci & 7;
    const int lc = (c16 >> 1) ^ (kr & 3);
    return box * 2048 + kr * 64 + ((lc ^ ((kr >> 1) & 3)) << 4) + ((c16 & 1) << 3);
}

// Tile order: groups of 8 row tiles sweep all column tiles, so the CTAs running
// at one time share A rows and B columns in L2.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int &b, int &tm, int &tn) {
    const int per_batch = tiles_m * tiles_n;
    b = t / per_batch;
    const int r = t - b * per_batch;
    constexpr int G = 8;
    const int group_span = G * tiles_n;
    const int g = r / group_span;
    const int first_m = g * G;
    const int gsz = (tiles_m - first_m) < G ? (tiles_m - first_m) : G;
    const int in_g = r - g * group_span;
    tm = first_m + in_g % gsz;
    tn = in_g / gsz;
}

// Work distribution over the resident units (CTAs, or CTA pairs).
//  whole tiles: unit u takes tiles u, u + units, u + 2 units, ... with all of K.
//  stream-K   : the first sk_tile0 tiles (whole waves of tiles, a multiple of `units`) are dealt out
//               whole as above and processed first; the tile-major sequence of all K blocks of
//               the REMAINING tiles is cut into `units` equal contiguous ranges, so every unit
//               gets the same amount of work whatever the tile count, and only the last partial
//               wave pays for fix-ups (sk_tile0 == 0: every tile is cut that way).  A range falls into segments (tile, [kb0, kb1)), listed in shared memory
//               at kernel start (at most kMaxSegments; the host only picks stream-K when that
//               holds).  A segment with kb0 == 0 owns its tile: it stores C, after adding the
//               partial sums of the units whose ranges start inside the tile.  A segment with
//               kb0 > 0 (always the first of its range) writes its partial sums to a workspace
//               and raises a flag.  Owners wait only for units that do that work first, so no
//               wait is circular.
constexpr int kMaxSegments = 32;

// Fused all-gather: copies this CTA's 128 rows of tile `t` from this GPU's C (just written by
// the epilogue, still in L2) into the same place of every peer's C.  `tid` of `nthreads`
// threads share the work; consecutive threads take consecutive 16-byte pieces of a row, so a
// warp's store is one contiguous 512-byte piece of NVLink traffic.
template <int CG>
__device__ __forceinline__ void forward_tile(const TcArgs &args, int t, int cta_rank, int tid, int nthreads) {
    using C = Cfg<CG>;
    constexpr int ROW_VEC = C::TILE_N / 4;   // float4 per tile row
    constexpr int TOTAL_VEC = BM * ROW_VEC;  // this CTA's 128 rows
    constexpr int FWD_BATCH = 8;
    const bool vec_ok = args.c_sj == 1 && (args.c_si & 3) == 0 && (args.c_sb & 3) == 0 &&
                        (reinterpret_cast<uintptr_t>(args.c) & 15) == 0;
    int b, tm, tn;
    tile_coords(t, args.tiles_m, args.tiles_n, b, tm, tn);
    const int row0 = tm * C::TILE_M + cta_rank * BM;
    const int col0 = tn * C::TILE_N;
    const long long base = static_cast<long long>(b) * args.c_sb;
    if (vec_ok) {
        for (int first = tid; first < TOTAL_VEC; first += nthreads * FWD_BATCH) {
            float4 v[FWD_BATCH];
            unsigned valid = 0;
#pragma unroll
            for (int u = 0; u < FWD_BATCH; ++u) {
                const int idx = first + u * nthreads;
                const int r = row0 + idx / ROW_VEC;
                const int cc = col0 + (idx % ROW_VEC) * 4;
                // whole vectors only; a ragged right edge is handled below
                if (idx < TOTAL_VEC && r < args.N && cc + 4 <= args.M) {
                    valid |= 1u << u;
                    v[u] = __ldcg(reinterpret_cast<const float4 *>(args.c + base +
                                                                   static_cast<long long>(r) * args.c_si + cc));
                }
            }
#pragma unroll
            for (int u = 0; u < FWD_BATCH; ++u) {
                if (valid & (1u << u)) {
                    const int idx = first + u * nthreads;
                    const long long o = base + static_cast<long long>(row0 + idx / ROW_VEC) * args.c_si + col0 +
                                        (idx % ROW_VEC) * 4;
                    for (int pr = 0; pr < args.n_peers; ++pr) *reinterpret_cast<float4 *>(args.peer_c[pr] + o) = v[u];
                }
            }
        }
    }
    // Scalar path: everything when the destination is not vector-aligned, else only the
    // columns of a ragged right edge.
    if (!vec_ok || (args.M & 3) != 0) {
        const int edge_begin = vec_ok ? (args.M - (args.M & 3)) : 0;
        for (int idx = tid; idx < BM * C::TILE_N; idx += nthreads) {
            const int r = row0 + idx / C::TILE_N;
            const int cc = col0 + idx % C::TILE_N;
            if (r < args.N && cc < args.M && cc >= edge_begin) {
                const long long o = base + static_cast<long long>(r) * args.c_si + static_cast<long long>(cc) * args.c_sj;
                const float x = __ldcg(args.c + o);
                for (int pr = 0; pr < args.n_peers; ++pr) args.peer_c[pr][o] = x;
            }
        }
    }
}

// PROF: the roles count the cycles they wait and work (ttb_tc_profile); the clock reads cost each
// role a few dozen cycles per K block, so the counting build is a kernel of its own.
template <int CG, bool PROF>
__global__ void __launch_bounds__(Cfg<CG>::NUM_THREADS, 1) gemm_f32_3xtf32_kernel(const __grid_constant__ TcArgs args) {
    using C = Cfg<CG>;
    constexpr bool PAIR = CG == 2;

    extern __shared__ uint8_t smem_dyn[];
    __shared__ uint64_t full_bar[STAGES];   // TMA bytes landed (local)
    __shared__ uint64_t empty_bar[STAGES];  // the MMAs of the K block in this raw slot are done (local); the
                                            // converters wait on the same barriers, SMALL_STAGES K blocks back
    __shared__ uint64_t small_empty_bar[SMALL_STAGES];  // the MMAs that read the small slot are done (local)
    __shared__ uint64_t conv_bar[SMALL_STAGES];         // small tiles written (lives in the leader CTA)
    __shared__ uint64_t acc_full_bar[2];    // accumulator chunk complete (local)
    __shared__ uint64_t acc_empty_bar[2];   // accumulator read out (lives in the leader CTA)
    __shared__ uint64_t out_full_bar[2];    // tile stored into this GPU's C (epilogue -> forwarding warps)
    __shared__ uint64_t out_empty_bar[2];   // tile forwarded to every peer (forwarding warps -> epilogue)
    __shared__ uint64_t last_full_bar;      // the CTA's last tile stored into this GPU's C
    __shared__ uint64_t drain_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int seg_tile_s[kMaxSegments], seg_kb0_s[kMaxSegments], seg_kb1_s[kMaxSegments], seg_count_s;
    __shared__ int abort_flag_s;

    const long long kernel_t0 = args.prof ? clock64() : 0;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
    const bool leader = cta_rank == 0;
    volatile int *abort_flag = &abort_flag_s;

    // 1024-byte alignment of the tile area in the shared window (the swizzle patterns
    // repeat every 1024 bytes).
    const uint32_t dyn_base = smem_u32(smem_dyn);
    const uint32_t tiles_base = (dyn_base + 1023u) & ~1023u;
    uint8_t *tiles = smem_dyn + (tiles_base - dyn_base);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < SMALL_STAGES; ++s) {
            // converter warps of both CTAs, plus the two extra ones per CTA of the pair form (below)
            mbar_init(&small_empty_bar[s], 1);
            mbar_init(&conv_bar[s], (C::NUM_CONV_WARPS + ((PAIR && args.terms == 2 && args.extra_conv) ? 2 : 0)) * CG);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full_bar[a], 1);
            mbar_init(&acc_empty_bar[a], 4 * C::EPI_WGS * CG);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&out_full_bar[a], 4 * C::EPI_WGS);
            mbar_init(&out_empty_bar[a], 2);
        }
        mbar_init(&last_full_bar, 4 * C::EPI_WGS);
        mbar_init(&drain_bar, 1);
        if (args.pieces > 1) {
            // piece schedule (the host sets streamk with it): parts u, u + units, ... of all tiles' parts
            const int nkb = (args.K + BK - 1) / BK;
            const int u = PAIR ? (blockIdx.x >> 1) : blockIdx.x, us = PAIR ? (gridDim.x >> 1) : gridDim.x;
            const int total = args.total_tiles << args.pieces_log2;
            int n = 0;
            for (int g = u; g < total && n < kMaxSegments; g += us) {
                const int k0 = (g & (args.pieces - 1)) * args.piece_len;
                seg_tile_s[n] = g >> args.pieces_log2;
                seg_kb0_s[n] = k0;
                seg_kb1_s[n] = k0 + args.piece_len < nkb ? k0 + args.piece_len : nkb;
                ++n;
            }
            seg_count_s = n;
        } else if (args.streamk) {
            // cut this unit's K-block range into per-tile segments
            const int nkb = (args.K + BK - 1) / BK;
            const int u = PAIR ? (blockIdx.x >> 1) : blockIdx.x, us = PAIR ? (gridDim.x >> 1) : gridDim.x;
            int n = 0;
            for (int t = u; t < args.sk_tile0 && n < kMaxSegments; t += us) {  // whole tiles first
                seg_tile_s[n] = t;
                seg_kb0_s[n] = 0;
                seg_kb1_s[n] = nkb;
                ++n;
            }
            const long long all = static_cast<long long>(args.total_tiles - args.sk_tile0) * nkb;  // < 2^31 (host)
            int pos = static_cast<int>(all * u / us);
            const int end = static_cast<int>(all * (u + 1) / us);
            while (pos < end && n < kMaxSegments) {
                const int rel = pos / nkb, k0 = pos - rel * nkb;
                int stop = pos + (nkb - k0);
                if (stop > end) stop = end;
                seg_tile_s[n] = args.sk_tile0 + rel;
                seg_kb0_s[n] = k0;
                seg_kb1_s[n] = k0 + (stop - pos);
                ++n;
                pos = stop;
            }
            if (args.sk_pair && (u & 1)) {
                // odd unit: the cut range back to front
                int first = 0;
                while (first < n && seg_tile_s[first] < args.sk_tile0) ++first;
                for (int a = first, b = n - 1; a < b; ++a, --b) {
                    int x = seg_tile_s[a]; seg_tile_s[a] = seg_tile_s[b]; seg_tile_s[b] = x;
                    x = seg_kb0_s[a]; seg_kb0_s[a] = seg_kb0_s[b]; seg_kb0_s[b] = x;
                    x = seg_kb1_s[a]; seg_kb1_s[a] = seg_kb1_s[b]; seg_kb1_s[b] = x;
                }
            }
            seg_count_s = n;
        }
        abort_flag_s = 0;
        fence_mbar_init();
        tma_prefetch_desc(&args.tmap_a);
        tma_prefetch_desc(&args.tmap_b);
    }
    if (warp == 1) {
        tmem_alloc<CG>(&tmem_base_slot, C::TMEM_COLS);
        tmem_relinquish<CG>();
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) {
        // The peer's barriers must be initialised before anything arrives on them.
        cluster_arrive();
        cluster_wait();
    }
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    // A operands in tensor memory (hybrid split only): see the map at Cfg.
    const bool a_tmem = args.a_tmem != 0 && args.terms == 2 && !(args.dbg & 8);
    const int acc_bufs = (a_tmem && PAIR) ? 1 : 2;
    // The pair form has one converter warp per scheduler, and converting is what bounds the kernel;
    // its warps 2-3 have nothing to do unless they forward tiles to peers (the fallback form of the
    // fused all-gather), so they convert 5/8 of every B tile.
    const bool extra_conv = PAIR && args.terms == 2 && args.extra_conv != 0;
    const uint32_t a_slot_col0 = static_cast<uint32_t>(acc_bufs * C::ACC_COLS);

    const int num_kb = (args.K + BK - 1) / BK;
    const int k_chunk = args.k_chunk > 0 ? args.k_chunk : num_kb;
    // Peers served by the forwarding warps (none when the epilogue's tensor stores reach them).
    const int fwd_peers = (args.peer_tma || args.mc_c != nullptr) ? 0 : args.n_peers;
    const int unit = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
    const int units = PAIR ? (gridDim.x >> 1) : gridDim.x;
    // This unit's segments.  n_store of them store C (all of them with whole tiles); the fused
    // all-gather treats the last stored tile specially.
    int n_seg, n_store, last_store_tile;
    if (!args.streamk) {
        n_seg = (unit < args.total_tiles && !(args.dbg & 64)) ? (args.total_tiles - unit + units - 1) / units : 0;
        n_store = n_seg;
        last_store_tile = unit + (n_seg - 1) * units;
    } else {
        n_seg = seg_count_s;
        n_store = 0;
        last_store_tile = -1;
        for (int i = 0; i < n_seg; ++i) {
            if (seg_kb0_s[i] == 0) {
                ++n_store;
                last_store_tile = seg_tile_s[i];
            }
        }
    }
    // Segment i of this unit: (tile, [kb0, kb1)).
    auto segment = [&](int i, int &tile, int &kb0, int &kb1) {
        if (!args.streamk) {
            tile = unit + i * units;
            kb0 = 0;
            kb1 = num_kb;
        } else {
            tile = seg_tile_s[i];
            kb0 = seg_kb0_s[i];
            kb1 = seg_kb1_s[i];
        }
    };

    // Register budget per warpgroup (512 threads start with 128 registers each; the epilogue
    // holds 128 accumulators per thread and takes registers the other roles give up).  Each role's branch starts with its own setmaxnreg so that the
    // compiler allocates that branch against its own budget.
    if (warp < C::FIRST_EPI_WARP) {
      setmaxnreg_dec<64>();
      if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int issued = 0;
            long long w_a = 0;
            for (int seg = 0; seg < n_seg && ok; ++seg) {
                int t, kb0, kb1;
                segment(seg, t, kb0, kb1);
                int b, tm, tn;
                tile_coords(t, args.tiles_m, args.tiles_n, b, tm, tn);
                const int m0 = tm * C::TILE_M + static_cast<int>(cta_rank) * BM;
                const int n0 = tn * C::TILE_N + static_cast<int>(cta_rank) * BNC;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!wait_or_abort<PAIR>(&empty_bar[stage], phase ^ 1u, abort_flag, PROF ? &w_a : nullptr)) {
                        report(args.status, abort_flag, kErrProducerWait, static_cast<unsigned>(stage));
                        ok = false;
                        break;
                    }
                    uint8_t *a_dst = tiles + stage * STAGE_BYTES;
                    uint8_t *b_dst = a_dst + TILE_BYTES;
                    mbar_arrive_expect_tx(&full_bar[stage], RAW_BYTES);
                    const int k0 = kb * BK;
                    if ((args.dbg & 16) && issued == 0) {
                        // Test switch: the very first stage is armed but never loaded, so the
                        // waits downstream run out and the kernel must unwind by itself.
                        ++issued;
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        continue;
                    }
                    if (args.a_mn_major) {
                        for (int j = 0; j < BM / 32; ++j)
                            tma_load_3d(a_dst + j * MN_BOX_BYTES, &args.tmap_a, &full_bar[stage], m0 + 32 * j, k0,
                                        b * args.a_batch_mul);
                    } else {
                        tma_load_3d(a_dst, &args.tmap_a, &full_bar[stage], k0, m0, b * args.a_batch_mul);
                    }
                    if (args.b_mn_major) {
                        for (int j = 0; j < BNC / 32; ++j)
                            tma_load_3d(b_dst + j * MN_BOX_BYTES, &args.tmap_b, &full_bar[stage], n0 + 32 * j, k0,
                                        b * args.b_batch_mul);
                    } else {
                        tma_load_3d(b_dst, &args.tmap_b, &full_bar[stage], k0, n0, b * args.b_batch_mul);
                    }
                    ++issued;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok && issued > 0) {
                // Let the copies already in flight land before the CTA's shared
                // memory is given up: wait (bounded) for the last stage issued.
                const int last = (stage + STAGES - 1) % STAGES;
                const uint32_t last_phase = (stage == 0) ? (phase ^ 1u) : phase;
                for (int i = 0; i < 100000; ++i)
                    if (mbar_try_wait(&full_bar[last], last_phase)) break;
            }
            if (PROF && args.prof) args.prof[blockIdx.x * kProfSlots + kProfProducerEmpty] = w_a;
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            const uint32_t idesc = make_idesc_tf32(C::UMMA_M, C::UMMA_N, args.a_mn_major, args.b_mn_major);
            int stage = 0;
            uint32_t phase = 0;
            int sstage = 0;
            uint32_t sphase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            long long w_a = 0, w_b = 0;
            // Shared-memory descriptor fields per operand major.
            //  K-major : 128-byte swizzle (16 B chunks); rows of 128 B, 8-row groups 1024 B
            //            apart (SBO); a K step of 8 fp32 advances the start address by 32 B
            //            inside the swizzle row.
            //  MN-major: 128-byte swizzle with 32 B chunks (the only layout tcgen05.mma takes
            //            for MN-major tf32); a 32-element MN group is MN_BOX_BYTES from the next
            //            (LBO), 4-row K groups are 512 B apart (SBO); a K step of 8 rows
            //            advances by 1024 B.
            const uint32_t a_lbo = args.a_mn_major ? MN_BOX_BYTES : 16, a_sbo = args.a_mn_major ? 512 : 1024;
            const uint32_t a_kstep = args.a_mn_major ? 1024 : 32;
            const uint64_t a_swz = args.a_mn_major ? kSwizzle128Base32 : kSwizzle128;
            const uint32_t b_lbo = args.b_mn_major ? MN_BOX_BYTES : 16, b_sbo = args.b_mn_major ? 512 : 1024;
            const uint32_t b_kstep = args.b_mn_major ? 1024 : 32;
            const uint64_t b_swz = args.b_mn_major ? kSwizzle128Base32 : kSwizzle128;
            // bf16 tiles of the hybrid split (64-byte rows, 64-byte swizzle):
            //  K-major : 8-row groups 512 B apart (SBO); a K step of 16 bf16 advances by 32 B.
            //  MN-major: 32-element MN groups 2048 B apart (LBO), 8-row K groups 512 B apart
            //            (SBO); a K step of 16 rows advances by 1024 B.
            const uint32_t idesc16 = make_idesc_bf16(C::UMMA_M, C::UMMA_N, args.a_mn_major, args.b_mn_major);
            // A read from tensor memory is K-major whatever the raw tile's layout was
            const uint32_t idesc16_ts = make_idesc_bf16(C::UMMA_M, C::UMMA_N, 0, args.b_mn_major);
            const uint32_t a16_lbo = args.a_mn_major ? 2048 : 16, a16_kstep = args.a_mn_major ? 1024 : 32;
            const uint32_t b16_lbo = args.b_mn_major ? 2048 : 16, b16_kstep = args.b_mn_major ? 1024 : 32;
            
            for (int seg = 0; seg < n_seg && ok; ++seg) {
                int t, kb0, kb1;
                segment(seg, t, kb0, kb1);
                for (int kb_begin = kb0; kb_begin < kb1 && ok; kb_begin += k_chunk) {
                    if (!wait_or_abort<PAIR>(&acc_empty_bar[acc], acc_phase ^ 1u, abort_flag, PROF ? &w_a : nullptr)) {
                        report(args.status, abort_flag, kErrAccEmptyWait, static_cast<unsigned>(acc));
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * C::ACC_COLS);
                    const int kb_end = (kb_begin + k_chunk < kb1) ? kb_begin + k_chunk : kb1;
                    for (int kb = kb_begin; kb < kb_end; ++kb) {
                        if (!wait_or_abort<PAIR>(&conv_bar[sstage], sphase, abort_flag, PROF ? &w_b : nullptr)) {
                            report(args.status, abort_flag, kErrMmaWait, static_cast<unsigned>(stage));
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t a_raw = tiles_base + stage * STAGE_BYTES;
                        const uint32_t b_raw = a_raw + TILE_BYTES;
                        const uint32_t a_small = tiles_base + SMALL_RING_OFFSET + sstage * STAGE_BYTES;
                        const uint32_t b_small = a_small + TILE_BYTES;
                        if (args.terms == 2) {
                            // Hybrid split: big.big on the raw fp32 tiles as TF32, the two
                            // correction terms on bf16 tiles the converters wrote into the small
                            // slot ([A small | A | B small | B], 8 KiB each).  Half the tensor
                            // cycles of a TF32 correction term, half its shared-memory reads.
                            // The corrections go first and the small slot is released right behind
                            // them: the converters' round trip (slot free -> convert -> converted ->
                            // issue) then runs while the TF32 product of this K block, which reads
                            // the raw slot only, keeps the tensor pipe busy.
                            const uint32_t fresh0 = (kb != kb_begin) ? 1u : 0u;
                            const uint32_t a_s16 = a_small, a_x16 = a_small + H_TILE_BYTES;
                            const uint32_t b_s16 = a_small + 2 * H_TILE_BYTES, b_x16 = a_small + 3 * H_TILE_BYTES;
                            if (a_tmem) {
                                // A operands of the corrections from tensor memory (the converters put
                                // them there): no shared-memory read for them, and none was written.
                                const uint32_t t_s = tmem_base + a_slot_col0 + static_cast<uint32_t>(sstage * C::A_SLOT_COLS);
                                const uint32_t t_x = t_s + 16;
#pragma unroll
                                for (int k2 = 0; k2 < BK / 16; ++k2) {
                                    mma_f16_ts<CG>(d_tmem, t_s + k2 * 8,
                                                   make_smem_desc(b_x16 + k2 * b16_kstep, b16_lbo, 512, kSwizzle64), idesc16_ts,
                                                   k2 == 0 ? fresh0 : 1u);
                                    mma_f16_ts<CG>(d_tmem, t_x + k2 * 8,
                                                   make_smem_desc(b_s16 + k2 * b16_kstep, b16_lbo, 512, kSwizzle64), idesc16_ts, 1);
                                }
                            } else if (!(args.dbg & 8)) {
#pragma unroll
                                for (int k2 = 0; k2 < BK / 16; ++k2) {
                                    mma_f16<CG>(d_tmem, make_smem_desc(a_s16 + k2 * a16_kstep, a16_lbo, 512, kSwizzle64),
                                                make_smem_desc(b_x16 + k2 * b16_kstep, b16_lbo, 512, kSwizzle64), idesc16,
                                                k2 == 0 ? fresh0 : 1u);
                                    mma_f16<CG>(d_tmem, make_smem_desc(a_x16 + k2 * a16_kstep, a16_lbo, 512, kSwizzle64),
                                                make_smem_desc(b_s16 + k2 * b16_kstep, b16_lbo, 512, kSwizzle64), idesc16, 1);
                                }
                            } else {
                                // layout check only: bf16(A).bf16(B) under the TF32 product
#pragma unroll
                                for (int k2 = 0; k2 < BK / 16; ++k2)
                                    mma_f16<CG>(d_tmem, make_smem_desc(a_x16 + k2 * a16_kstep, a16_lbo, 512, kSwizzle64),
                                                make_smem_desc(b_x16 + k2 * b16_kstep, b16_lbo, 512, kSwizzle64), idesc16,
                                                k2 == 0 ? fresh0 : 1u);
                            }
                            if constexpr (PAIR)
                                mma_commit_both(smem_u32(&small_empty_bar[sstage]));
                            else
                                mma_commit<CG>(smem_u32(&small_empty_bar[sstage]));
#pragma unroll
                            for (int kk = 0; kk < BK / UMMA_K; ++kk)
                                mma_tf32<CG>(d_tmem, make_smem_desc(a_raw + kk * a_kstep, a_lbo, a_sbo, a_swz),
                                             make_smem_desc(b_raw + kk * b_kstep, b_lbo, b_sbo, b_swz), idesc, 1u);
                        } else
#pragma unroll
                        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                            const uint32_t fresh = (kb != kb_begin || kk != 0) ? 1u : 0u;
                            const uint64_t da_big = make_smem_desc(a_raw + kk * a_kstep, a_lbo, a_sbo, a_swz);
                            const uint64_t db_big = make_smem_desc(b_raw + kk * b_kstep, b_lbo, b_sbo, b_swz);
                            if (args.terms == 3) {
                                const uint64_t da_small = make_smem_desc(a_small + kk * a_kstep, a_lbo, a_sbo, a_swz);
                                const uint64_t db_small = make_smem_desc(b_small + kk * b_kstep, b_lbo, b_sbo, b_swz);
                                // Small terms first: they are ~2^-11 of the big term.
                                mma_tf32<CG>(d_tmem, da_small, db_big, idesc, fresh);
                                mma_tf32<CG>(d_tmem, da_big, db_small, idesc, 1);
                                mma_tf32<CG>(d_tmem, da_big, db_big, idesc, 1);
                            } else {
                                mma_tf32<CG>(d_tmem, da_big, db_big, idesc, fresh);
                            }
                        }
                        // One arrival per barrier reaches both CTAs of a pair.
                        if (args.terms != 2) {
                            if constexpr (PAIR)
                                mma_commit_both(smem_u32(&small_empty_bar[sstage]));
                            else
                                mma_commit<CG>(smem_u32(&small_empty_bar[sstage]));
                        }
                        if constexpr (PAIR)
                            mma_commit_both(smem_u32(&empty_bar[stage]));
                        else
                            mma_commit<CG>(smem_u32(&empty_bar[stage]));
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        if (++sstage == SMALL_STAGES) {
                            sstage = 0;
                            sphase ^= 1u;
                        }
                    }
                    if (!ok) break;
                    if constexpr (PAIR)
                        mma_commit_both(smem_u32(&acc_full_bar[acc]));
                    else
                        mma_commit<CG>(smem_u32(&acc_full_bar[acc]));
                    if (++acc == acc_bufs) {
                        acc = 0;
                        acc_phase ^= 1u;
                    }
                }
            }
            // Everything issued must have retired before TMEM is freed.
            mma_commit<CG>(smem_u32(&drain_bar));
            for (int i = 0; i < 1000000; ++i)
                if (mbar_try_wait(&drain_bar, 0)) break;
            if (PROF && args.prof) {
                args.prof[blockIdx.x * kProfSlots + kProfMmaAccEmpty] = w_a;
                args.prof[blockIdx.x * kProfSlots + kProfMmaConv] = w_b;
            }
        }
      } else if (fwd_peers > 0) {
        // ------------------------------------------------------------ forwarding (warps 2-3)
        // All-gather fused into the product: once the epilogue has stored a tile into this
        // GPU's C, these two warps read it back (it is still in L2) and store it into the same
        // place of every peer GPU's C through peer-mapped pointers (plain st.global over
        // NVLink).  They are the only threads that NVLink back-pressure can stall; the MMA,
        // converter and epilogue warps keep going, so the exchange overlaps the math tile by
        // tile.  The two-slot full/empty handshake keeps the epilogue at most two tiles ahead.
        // The CTA's LAST tile is not forwarded here: nothing is left to overlap it with, so all
        // warps of the CTA push it together after their own loops (see below).
        const int stid = threadIdx.x - 64;                    // 0..63
        int oslot = 0;
        uint32_t ophase = 0;
        bool ok = true;
        int stored = 0;
        for (int seg = 0; seg < n_seg && ok; ++seg) {
            int t, kb0, kb1;
            segment(seg, t, kb0, kb1);
            if (kb0 != 0) continue;             // a partial-sum segment stores nothing into C
            if (++stored == n_store) break;     // the last stored tile is forwarded by every warp
            if (!wait_or_abort<false>(&out_full_bar[oslot], ophase, abort_flag)) {
                if (lane == 0) report(args.status, abort_flag, kErrForwardWait, 16u + static_cast<unsigned>(oslot));
                ok = false;
                break;
            }
            forward_tile<CG>(args, t, static_cast<int>(cta_rank), stid, 64);
            __syncwarp();
            if (lane == 0) mbar_arrive(&out_empty_bar[oslot]);
            if (++oslot == 2) {
                oslot = 0;
                ophase ^= 1u;
            }
        }
        // Peer stores must have left this GPU before the kernel is reported complete.
        __threadfence_system();
      } else if (extra_conv) {
        // ------------------------------------------------------------ extra converters (warps 2-3, pair form)
        // Chunks [384, 1024) of every raw B tile: thread e takes 384 + e + 64 u, u = 0..9, which
        // land 512 bytes apart in the bf16 tiles (see hybrid_dst); the converter warpgroup keeps
        // the A tile and chunks [0, 384) of B, so its threads convert 11 chunks per K block and
        // these 10.  Same waits and the same converted barrier as the converter warpgroup.
        const int etid = threadIdx.x - 64;  // 0..63
        const int dst0 = hybrid_dst(384 + etid, args.b_mn_major != 0);
        const uint32_t conv_remote0 = PAIR ? mapa(smem_u32(&conv_bar[0]), 0) : 0u;
        int stage = 0, sstage = 0;
        uint32_t phase = 0, sphase = 0;
        bool ok = true;
        for (int seg = 0; seg < n_seg && ok; ++seg) {
            int t, kb0, kb1;
            segment(seg, t, kb0, kb1);
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!wait_or_abort<PAIR>(&small_empty_bar[sstage], sphase ^ 1u, abort_flag) ||
                    !wait_or_abort<false>(&full_bar[stage], phase, abort_flag)) {
                    if (lane == 0) report(args.status, abort_flag, kErrConverterWait, 64u + static_cast<unsigned>(stage));
                    ok = false;
                    break;
                }
                const uint4 *rt = reinterpret_cast<const uint4 *>(tiles + stage * STAGE_BYTES + TILE_BYTES) + 384 + etid;
                uint8_t *s16 = tiles + SMALL_RING_OFFSET + sstage * STAGE_BYTES + 2 * H_TILE_BYTES;
                uint8_t *x16 = s16 + H_TILE_BYTES;
#pragma unroll
                for (int b4 = 0; b4 < 10; b4 += 5) {
                    uint4 x[5];
#pragma unroll
                    for (int u = 0; u < 5; ++u) x[u] = rt[(b4 + u) * 64];
                    float za = 0.0f, zb = 0.0f;
#pragma unroll
                    for (int u = 0; u < 5; ++u) hybrid_chunk_unmasked(x[u], s16, x16, dst0 + (b4 + u) * 512, za, zb);
                    if (!all_finite(za, zb)) {
#pragma unroll
                        for (int u = 0; u < 5; ++u) hybrid_chunk(x[u], s16, x16, dst0 + (b4 + u) * 512);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(conv_remote0 + static_cast<uint32_t>(sstage * sizeof(uint64_t)));
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
                if (++sstage == SMALL_STAGES) {
                    sstage = 0;
                    sphase ^= 1u;
                }
            }
        }
      }
    } else if (warp < C::FIRST_CONV_WARP) {
        // ------------------------------------------------------------ epilogue
        setmaxnreg_inc<C::EPI_REGS>();
        const int quarter = warp & 3;                         // TMEM lanes [32*quarter, +32)
        const int col_half = (warp - C::FIRST_EPI_WARP) >> 2;  // which 128 accumulator columns
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        const bool vec_ok = args.c_sj == 1 && (args.c_si & 3) == 0 && (args.c_sb & 3) == 0 &&
                            (reinterpret_cast<uintptr_t>(args.c) & 15) == 0;
        const bool dvec_ok = args.d_sj == 1 && (args.d_si & 3) == 0 && (args.d_sb & 3) == 0 &&
                             (reinterpret_cast<uintptr_t>(args.d) & 15) == 0;
        uint32_t acc_empty_remote[2] = {0, 0};
        if constexpr (PAIR) {
            for (int a = 0; a < 2; ++a) acc_empty_remote[a] = mapa(smem_u32(&acc_empty_bar[a]), 0);
        }
        float sum[128];
        int oslot = 0;
        uint32_t ophase = 0;
        long long w_a = 0;
        // Stream-K workspace of this warp: [unit][CTA of the pair][epilogue warp][lane][128 floats].
        const int epi_warp = warp - C::FIRST_EPI_WARP;
        constexpr int EPI_WARPS = 4 * C::EPI_WGS;
        int stored = 0;
        for (int seg = 0; seg < n_seg && ok; ++seg) {
            int t, kb0, kb1;
            segment(seg, t, kb0, kb1);
            int b, tm, tn;
            tile_coords(t, args.tiles_m, args.tiles_n, b, tm, tn);
            for (int ch = kb0; ch < kb1; ch += k_chunk) {
                if (!wait_or_abort<PAIR>(&acc_full_bar[acc], acc_phase, abort_flag, PROF ? &w_a : nullptr)) {
                    if (lane == 0) report(args.status, abort_flag, kErrEpilogueWait, static_cast<unsigned>(acc));
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t t_row = tmem_base + static_cast<uint32_t>(acc * C::ACC_COLS + col_half * 128) +
                                       (static_cast<uint32_t>(quarter * 32) << 16);
                const bool first = ch == kb0;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    uint32_t v[16];
                    tmem_ld_32x16(t_row + static_cast<uint32_t>(q * 16), v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float x = __uint_as_float(v[j]);
                        sum[q * 16 + j] = first ? x : sum[q * 16 + j] + x;
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (PAIR)
                        mbar_arrive_cluster(acc_empty_remote[acc]);
                    else
                        mbar_arrive(&acc_empty_bar[acc]);
                }
                if (++acc == acc_bufs) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
            if (!ok) break;
            if (args.pieces > 1) {
                // Piece schedule: write this part's sums, draw a ticket; the last one in adds up.
                const int P = args.pieces, PL = args.pieces_log2;
                const long long my_slot =
                    ((static_cast<long long>(unit) * 2 + (seg & 1)) * CG + cta_rank) * EPI_WARPS + epi_warp;
                // The slot was last used two parts ago; whoever completed that tile has lowered
                // its flag long since, unless that unit fell far behind.
                unsigned long long t0 = 0;
                for (uint32_t spin = 0;; ++spin) {
                    if (*reinterpret_cast<volatile unsigned int *>(&args.sk_flags[my_slot]) == 0u) break;
                    if ((spin & 63u) == 63u) {
                        const unsigned long long now = global_ns();
                        if (t0 == 0) t0 = now;
                        if (*abort_flag || now - t0 > 2000000000ull) {
                            ok = false;
                            break;
                        }
                    }
                }
                if (!ok) {
                    if (lane == 0) report(args.status, abort_flag, kErrStreamKWait, 0x10000u + static_cast<unsigned>(unit));
                    break;
                }
                float4 *dst = reinterpret_cast<float4 *>(args.sk_partials + my_slot * 4096) + lane;
#pragma unroll
                for (int q = 0; q < 32; ++q)
                    dst[q * 32] = make_float4(sum[4 * q], sum[4 * q + 1], sum[4 * q + 2], sum[4 * q + 3]);
                __threadfence();
                __syncwarp();
                unsigned int ticket = 0;
                const long long tk = (static_cast<long long>(t) * CG + cta_rank) * EPI_WARPS + epi_warp;
                if (lane == 0) {
                    atomicExch(&args.sk_flags[my_slot], 1u);
                    __threadfence();
                    ticket = atomicAdd(&args.sk_tickets[tk], 1u);
                }
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                if (ticket != static_cast<unsigned int>(P - 1)) continue;
                __threadfence();
                // Part 0 replaces the registers, the others are added, in part order.
                {
                    const int gj = t << PL;
                    const int uj = gj % units, sj = gj / units;
                    const long long slot = ((static_cast<long long>(uj) * 2 + (sj & 1)) * CG + cta_rank) * EPI_WARPS + epi_warp;
                    const float4 *src = reinterpret_cast<const float4 *>(args.sk_partials + slot * 4096) + lane;
#pragma unroll
                    for (int v0 = 0; v0 < 32; v0 += 8) {
                        float4 pv[8];
#pragma unroll
                        for (int v = 0; v < 8; ++v) pv[v] = __ldcg(src + (v0 + v) * 32);
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            sum[4 * (v0 + v)] = pv[v].x;
                            sum[4 * (v0 + v) + 1] = pv[v].y;
                            sum[4 * (v0 + v) + 2] = pv[v].z;
                            sum[4 * (v0 + v) + 3] = pv[v].w;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) args.sk_flags[slot] = 0u;  // consumed
                }
                for (int j = 1; j < P; ++j) {
                    const int gj = (t << PL) + j;
                    const int uj = gj % units, sj = gj / units;
                    const long long slot = ((static_cast<long long>(uj) * 2 + (sj & 1)) * CG + cta_rank) * EPI_WARPS + epi_warp;
                    const float4 *src = reinterpret_cast<const float4 *>(args.sk_partials + slot * 4096) + lane;
#pragma unroll
                    for (int v0 = 0; v0 < 32; v0 += 8) {
                        float4 pv[8];
#pragma unroll
                        for (int v = 0; v < 8; ++v) pv[v] = __ldcg(src + (v0 + v) * 32);
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            sum[4 * (v0 + v)] += pv[v].x;
                            sum[4 * (v0 + v) + 1] += pv[v].y;
                            sum[4 * (v0 + v) + 2] += pv[v].z;
                            sum[4 * (v0 + v) + 3] += pv[v].w;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) args.sk_flags[slot] = 0u;  // consumed
                }
                if (lane == 0) args.sk_tickets[tk] = 0u;  // ready for the next launch
            } else if (args.sk_pair && (kb0 != 0 || kb1 != num_kb)) {
                // Paired stream-K: this unit holds one end of the tile, a neighbour the other.
                const int which = kb0 != 0 ? 0 : 1;   // tail : head
                const long long my_slot =
                    ((static_cast<long long>(unit) * 2 + which) * CG + cta_rank) * EPI_WARPS + epi_warp;
                float4 *dst = reinterpret_cast<float4 *>(args.sk_partials + my_slot * 4096) + lane;
#pragma unroll
                for (int q = 0; q < 32; ++q)
                    dst[q * 32] = make_float4(sum[4 * q], sum[4 * q + 1], sum[4 * q + 2], sum[4 * q + 3]);
                __threadfence();
                __syncwarp();
                unsigned int ticket = 0;
                const long long tk = (static_cast<long long>(t) * CG + cta_rank) * EPI_WARPS + epi_warp;
                if (lane == 0) ticket = atomicAdd(&args.sk_tickets[tk], 1u);
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                if (ticket == 0u) continue;           // first of the two: the other one stores
                __threadfence();
                const int other = which ? unit + 1 : unit - 1;
                const long long slot =
                    ((static_cast<long long>(other) * 2 + (which ^ 1)) * CG + cta_rank) * EPI_WARPS + epi_warp;
                const float4 *src = reinterpret_cast<const float4 *>(args.sk_partials + slot * 4096) + lane;
#pragma unroll
                for (int v0 = 0; v0 < 32; v0 += 8) {
                    float4 pv[8];
#pragma unroll
                    for (int v = 0; v < 8; ++v) pv[v] = __ldcg(src + (v0 + v) * 32);
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        sum[4 * (v0 + v)] += pv[v].x;
                        sum[4 * (v0 + v) + 1] += pv[v].y;
                        sum[4 * (v0 + v) + 2] += pv[v].z;
                        sum[4 * (v0 + v) + 3] += pv[v].w;
                    }
                }
                __syncwarp();
                if (lane == 0) args.sk_tickets[tk] = 0u;  // ready for the next launch
            } else if (kb0 != 0) {
                // Stream-K, a range that starts inside a tile: hand the partial sums to the unit
                // that owns the tile.  Warp w of the owner reads exactly what warp w wrote here
                // (same TMEM lanes, same columns), so one flag per warp is all the ordering needed.
                const long long slot = (static_cast<long long>(unit) * CG + cta_rank) * EPI_WARPS + epi_warp;
                // Slot layout [32 float4 steps][32 lanes]: a warp's store is one contiguous 512 bytes.
                float4 *dst = reinterpret_cast<float4 *>(args.sk_partials + slot * 4096) + lane;
#pragma unroll
                for (int q = 0; q < 32; ++q)
                    dst[q * 32] = make_float4(sum[4 * q], sum[4 * q + 1], sum[4 * q + 2], sum[4 * q + 3]);
                __threadfence();
                __syncwarp();
                // Flag protocol: the writer raises the flag, the one reader (the tile's owner)
                // lowers it again after reading, so every flag is back at 0 when the kernel ends.
                // Nothing depends on a host-side launch counter: a launch recorded into a CUDA
                // graph replays correctly.
                if (lane == 0) atomicExch(&args.sk_flags[slot], 1u);
                continue;
            } else if (kb1 != num_kb) {
                // Stream-K, the owner of a tile whose tail other units computed: add their sums.
                const long long all_kb = static_cast<long long>(args.total_tiles - args.sk_tile0) * num_kb;
                for (int q = unit + 1; q < units && ok; ++q) {
                    if (all_kb * q / units >= static_cast<long long>(t - args.sk_tile0 + 1) * num_kb) break;
                    const long long slot = (static_cast<long long>(q) * CG + cta_rank) * EPI_WARPS + epi_warp;
                    unsigned long long t0 = 0;
                    for (uint32_t spin = 0;; ++spin) {
                        if (*reinterpret_cast<volatile unsigned int *>(&args.sk_flags[slot]) != 0u) break;
                        if ((spin & 63u) == 63u) {
                            const unsigned long long now = global_ns();
                            if (t0 == 0) t0 = now;
                            if (*abort_flag || now - t0 > 2000000000ull) {
                                ok = false;
                                break;
                            }
                        }
                    }
                    if (!ok) {
                        if (lane == 0) report(args.status, abort_flag, kErrStreamKWait, static_cast<unsigned>(q));
                        break;
                    }
                    __threadfence();
                    const float4 *src = reinterpret_cast<const float4 *>(args.sk_partials + slot * 4096) + lane;
                    // eight loads in flight at a time: their L2 latencies overlap
#pragma unroll
                    for (int v0 = 0; v0 < 32; v0 += 8) {
                        float4 p[8];
#pragma unroll
                        for (int v = 0; v < 8; ++v) p[v] = __ldcg(src + (v0 + v) * 32);
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            sum[4 * (v0 + v)] += p[v].x;
                            sum[4 * (v0 + v) + 1] += p[v].y;
                            sum[4 * (v0 + v) + 2] += p[v].z;
                            sum[4 * (v0 + v) + 3] += p[v].w;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) args.sk_flags[slot] = 0u;  // consumed: ready for the next launch
                }
                if (!ok) break;
            }
            ++stored;
            const int row = tm * C::TILE_M + static_cast<int>(cta_rank) * BM + quarter * 32 + lane;
            const int col0 = tn * C::TILE_N + col_half * 128;
            if (fwd_peers > 0) {
                // The forwarding warps must be done with the tile that last used this slot.
                if (!wait_or_abort<false>(&out_empty_bar[oslot], ophase ^ 1u, abort_flag)) {
                    if (lane == 0) report(args.status, abort_flag, kErrForwardWait, static_cast<unsigned>(oslot));
                    ok = false;
                    break;
                }
            }
            if (col0 < args.M) {
                const bool mine = row < args.N;
                float *crow = args.c + static_cast<long long>(b) * args.c_sb + static_cast<long long>(row) * args.c_si;
                if (mine && args.d != nullptr) {
                    // Fused addend.  The thread that adds d[b,row,col] is the one that stores
                    // c[b,row,col], so d may be C itself (accumulation).
                    const float *drow =
                        args.d + static_cast<long long>(b) * args.d_sb + static_cast<long long>(row) * args.d_si;
                    if (args.d_sj == 0) {
                        const float v = __ldg(drow);
#pragma unroll
                        for (int j = 0; j < 128; ++j) sum[j] += v;
                    } else if (dvec_ok && col0 + 128 <= args.M) {
                        const float4 *src = reinterpret_cast<const float4 *>(drow + col0);
#pragma unroll
                        for (int q = 0; q < 32; ++q) {
                            const float4 v = src[q];
                            sum[4 * q] += v.x;
                            sum[4 * q + 1] += v.y;
                            sum[4 * q + 2] += v.z;
                            sum[4 * q + 3] += v.w;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 128; ++j)
                            if (col0 + j < args.M) sum[j] += drow[static_cast<long long>(col0 + j) * args.d_sj];
                    }
                }
                if (args.act == TTB_ACT_RELU) {
#pragma unroll
                    for (int j = 0; j < 128; ++j) sum[j] = sum[j] < 0.0f ? 0.0f : sum[j];
                }
                if (args.mc_c != nullptr && vec_ok) {
                    // Fused all-gather through the switch: the tile goes once to the multicast
                    // address of C and NVSwitch delivers it to every GPU (this one included), so
                    // a GPU sends each byte of its block once, not once per peer.  Same staging
                    // as below, 8 lanes per row: one instruction stores four 128-byte lines.
                    uint8_t *stg = tiles + OUT_STAGING_OFFSET + epi_warp * OUT_STAGING_WARP_BYTES;
                    const int row_base = row - lane;
                    float *mbase = args.mc_c + static_cast<long long>(b) * args.c_sb;
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<float4 *>(stg + lane * 128 + ((c ^ (lane & 7)) << 4)) =
                                make_float4(sum[ch * 32 + 4 * c], sum[ch * 32 + 4 * c + 1], sum[ch * 32 + 4 * c + 2],
                                            sum[ch * 32 + 4 * c + 3]);
                        __syncwarp();
                        const int cc = lane & 7;
                        const int gcol = col0 + ch * 32 + 4 * cc;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int r = 4 * i + (lane >> 3);
                            const float4 v = *reinterpret_cast<const float4 *>(stg + r * 128 + ((cc ^ (r & 7)) << 4));
                            const int grow = row_base + r;
                            // the host only takes this path when M is a multiple of 4
                            if (grow < args.N && gcol < args.M)
                                multimem_st_v4(mbase + static_cast<long long>(grow) * args.c_si + gcol, v);
                        }
                        __syncwarp();
                    }
                } else if (args.c_tma && fwd_peers == 0) {
                    // Row-contiguous, 16-byte-aligned C: each warp passes 32 columns at a time
                    // through its 4 KiB of shared memory, written in the 128-byte-swizzled layout
                    // (16-byte chunk XOR row) of a 32 x 32 TMA box, and one lane issues a bulk
                    // tensor store.  The copy engine writes whole lines and clips the box at the
                    // edges of C; the warp's LSU work is eight 16-byte shared stores per chunk.
                    uint8_t *stg = tiles + OUT_STAGING_OFFSET + epi_warp * OUT_STAGING_WARP_BYTES;
                    const int row_base = row - lane;
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        // the previous box must have been read out of the staging buffer
                        if (lane == 0) bulk_wait_read_all();
                        __syncwarp();
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<float4 *>(stg + lane * 128 + ((c ^ (lane & 7)) << 4)) =
                                make_float4(sum[ch * 32 + 4 * c], sum[ch * 32 + 4 * c + 1], sum[ch * 32 + 4 * c + 2],
                                            sum[ch * 32 + 4 * c + 3]);
                        fence_proxy_async_smem();
                        __syncwarp();
                        const int gcol = col0 + ch * 32;
                        if (lane == 0 && row_base < args.N && gcol < args.M && !(args.dbg & 32)) {
                            tma_store_3d(&args.tmap_c, stg, gcol, row_base, b * args.c_batch_mul);
                            // Fused all-gather: the same box goes to the same place of every
                            // peer GPU's C over NVLink, straight from the staging buffer.
                            for (int pr = 0; pr < args.n_peers; ++pr)
                                tma_store_3d(&args.tmap_peer[pr], stg, gcol, row_base, b * args.c_batch_mul);
                            bulk_commit_group();
                        }
                    }
                } else if (vec_ok) {
                    // Same staging, stored by the warp itself (fused all-gather: the forwarding
                    // warps read C back right after the flag below, which plain stores followed by
                    // a fence order): 8 lanes per row, so one store instruction writes four
                    // complete 128-byte lines instead of touching 32.
                    uint8_t *stg = tiles + OUT_STAGING_OFFSET + epi_warp * OUT_STAGING_WARP_BYTES;
                    const int row_base = row - lane;
                    float *cbase = args.c + static_cast<long long>(b) * args.c_sb;
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<float4 *>(stg + lane * 128 + ((c ^ (lane & 7)) << 4)) =
                                make_float4(sum[ch * 32 + 4 * c], sum[ch * 32 + 4 * c + 1], sum[ch * 32 + 4 * c + 2],
                                            sum[ch * 32 + 4 * c + 3]);
                        __syncwarp();
                        const int cc = lane & 7;
                        const int gcol = col0 + ch * 32 + 4 * cc;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int r = 4 * i + (lane >> 3);
                            const float4 v = *reinterpret_cast<const float4 *>(stg + r * 128 + ((cc ^ (r & 7)) << 4));
                            const int grow = row_base + r;
                            if (grow < args.N && !(args.dbg & 32)) {
                                float *dst = cbase + static_cast<long long>(grow) * args.c_si + gcol;
                                if (gcol + 4 <= args.M) {
                                    *reinterpret_cast<float4 *>(dst) = v;
                                } else {
                                    if (gcol < args.M) dst[0] = v.x;
                                    if (gcol + 1 < args.M) dst[1] = v.y;
                                    if (gcol + 2 < args.M) dst[2] = v.z;
                                }
                            }
                        }
                        __syncwarp();
                    }
                } else if (mine) {
#pragma unroll
                    for (int j = 0; j < 128; ++j)
                        if (col0 + j < args.M) crow[static_cast<long long>(col0 + j) * args.c_sj] = sum[j];
                }
            }
            if (fwd_peers > 0) {
                // Publish the tile (now in this GPU's C) to the forwarding warps.
                __threadfence();
                __syncwarp();
                // The CTA's last tile has its own single-phase barrier: the threads that forward
                // it have not followed the two-slot ring, and a parity wait is only meaningful to
                // a waiter that is at most one phase behind.
                const bool last_tile = stored == n_store;
                if (lane == 0) mbar_arrive(last_tile ? &last_full_bar : &out_full_bar[oslot]);
                if (++oslot == 2) {
                    oslot = 0;
                    ophase ^= 1u;
                }
            }
        }
        // Bulk tensor stores still in flight read this CTA's shared memory: they must be done
        // before the CTA gives it up.
        if (lane == 0) {
            bulk_wait_all();
            // stores to peer GPUs must have left this GPU before the kernel is reported complete
            if (args.n_peers > 0 || args.mc_c != nullptr) __threadfence_system();
        }
        if (args.prof && warp == C::FIRST_EPI_WARP && lane == 0) {
            if (PROF) args.prof[blockIdx.x * kProfSlots + kProfEpiAccFull] = w_a;
            args.prof[blockIdx.x * kProfSlots + kProfTotal] = clock64() - kernel_t0;
        }
    } else {
        // ------------------------------------------------------------ converters
        setmaxnreg_dec<72>();
        const int ctid = threadIdx.x - C::FIRST_CONV_WARP * 32;
        constexpr int NCT = C::NUM_CONV_WARPS * 32;
        int stage = 0;
        uint32_t phase = 0;
        int sstage = 0;
        uint32_t sphase = 0;
        bool ok = true;
        long long w_a = 0, w_b = 0, w_c = 0;
        const bool mask_big = args.mask_big != 0;
        uint32_t conv_remote[SMALL_STAGES] = {0, 0};
        if constexpr (PAIR) {
            for (int s = 0; s < SMALL_STAGES; ++s) conv_remote[s] = mapa(smem_u32(&conv_bar[s]), 0);
        }
        // Hybrid split: where this thread's first 16-byte chunk of a raw operand tile goes in the
        // bf16 tiles (see the layout note below).  Chunk ctid + u * NCT lands u * NCT * 8 bytes
        // further in both layouts (NCT chunks are 16 or 32 whole K-major rows, or half a / a whole
        // MN-major box, and neither changes the XOR terms), so the K loop needs no index math.
        const int hyb_dst0[2] = {hybrid_dst(ctid, args.a_mn_major != 0), hybrid_dst(ctid, args.b_mn_major != 0)};
        for (int seg = 0; seg < n_seg && ok; ++seg) {
            int t, kb0, kb1;
            segment(seg, t, kb0, kb1);
            for (int kb = kb0; kb < kb1; ++kb) {
                // The small slot must have been released by the MMAs that last read it, and the
                // raw slot must have landed.
                if (!wait_or_abort<PAIR>(&small_empty_bar[sstage], sphase ^ 1u, abort_flag, PROF ? &w_a : nullptr) ||
                    !wait_or_abort<false>(&full_bar[stage], phase, abort_flag, PROF ? &w_b : nullptr)) {
                    if (lane == 0) report(args.status, abort_flag, kErrConverterWait, static_cast<unsigned>(stage));
                    ok = false;
                    break;
                }
                if (a_tmem) tc_fence_after_sync();  // the MMAs that read this A slot are done (tcgen05.commit)
                const long long busy0 = PROF ? clock64() : 0;
                uint4 *raw = reinterpret_cast<uint4 *>(tiles + stage * STAGE_BYTES);
                uint4 *small = reinterpret_cast<uint4 *>(tiles + SMALL_RING_OFFSET + sstage * STAGE_BYTES);
                // All loads of a batch are issued before the first dependent instruction, so
                // their shared-memory latencies overlap instead of adding up (a store to
                // `small` could alias `raw` as far as the compiler knows, which would otherwise
                // keep every load behind the previous store).
                constexpr int PER_THREAD = RAW_BYTES / 16 / NCT;  // 16 x 16-byte words
                constexpr int BATCH = 8;
                static_assert(PER_THREAD % BATCH == 0, "converter batches must tile the stage");
                if (args.terms == 2) {
                    // Hybrid split: per raw operand tile write two bf16 tiles, small = x - trunc_tf32(x)
                    // and x itself, both rounded to nearest, in the 64-byte-swizzled layout the
                    // bf16 MMAs read.  A 16-byte chunk of the raw tile (4 fp32) becomes 8 bytes in
                    // each; where it goes follows from undoing the raw tile's swizzle:
                    //  K-major  raw rows are 128 B with 16-B chunks XORed by (row & 7); the bf16 row
                    //           is 64 B with 16-B chunks XORed by ((row >> 1) & 3) -- the XORs cancel
                    //           up to the low bit, which picks the half of the 16-byte chunk.
                    //  MN-major raw rows (one K index, 32 MN values) have 32-B chunks XORed by
                    //           (k & 3); the bf16 row is 64 B with 16-B chunks XORed by ((k >> 1) & 3).
                    const uint8_t *raw_b = tiles + stage * STAGE_BYTES;
                    uint8_t *out_b = tiles + SMALL_RING_OFFSET + sstage * STAGE_BYTES;
                    constexpr int PER_T = TILE_BYTES / 16 / NCT;  // chunks per thread per operand tile (8 or 4)
                    if (a_tmem) {
                        // A operand: this thread owns one row of the A tile -- the row whose tensor
                        // memory lane its warp can reach (lane quarter = warp % 4) -- and, in the
                        // one-CTA form with two converter warpgroups, one half of that row's K range.
                        // It reads the row from the raw tile (undoing the TMA swizzle), splits it, and
                        // stores bf16(small) and bf16(x), two K elements per 32-bit column, straight
                        // into the correction MMAs' A slot in tensor memory.
                        const int q = warp & 3;
                        const int row = q * 32 + lane;
                        constexpr int KPARTS = C::NUM_CONV_WARPS / 4;
                        constexpr int KLEN = BK / KPARTS;
                        const int kfirst = ((warp - C::FIRST_CONV_WARP) >> 2) * KLEN;
                        const uint32_t t_slot = tmem_base + a_slot_col0 + static_cast<uint32_t>(sstage * C::A_SLOT_COLS) +
                                                (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
                        for (int h = 0; h < KLEN / 16; ++h) {
                            const int k0 = kfirst + h * 16;
                            uint32_t w[16];
                            if (!args.a_mn_major) {
                                // K-major raw tile: row = 128 bytes, 16-byte chunk c stored at c ^ (row & 7)
                                const uint8_t *rowp = raw_b + row * 128;
#pragma unroll
                                for (int c = 0; c < 4; ++c) {
                                    const uint4 v = *reinterpret_cast<const uint4 *>(
                                        rowp + ((((k0 >> 2) + c) ^ (row & 7)) << 4));
                                    w[4 * c] = v.x;
                                    w[4 * c + 1] = v.y;
                                    w[4 * c + 2] = v.z;
                                    w[4 * c + 3] = v.w;
                                }
                            } else {
                                // MN-major raw tile: boxes of 32 rows (MN) x 32 K; one K index is a
                                // 128-byte line of 32 MN values whose 32-byte chunks are XORed by (k & 3)
                                const uint8_t *boxp = raw_b + (row >> 5) * MN_BOX_BYTES + (row & 7) * 4;
                                const int c32 = (row & 31) >> 3;
#pragma unroll
                                for (int i = 0; i < 16; ++i) {
                                    const int k = k0 + i;
                                    w[i] = *reinterpret_cast<const uint32_t *>(boxp + k * 128 + ((c32 ^ (k & 3)) << 5));
                                }
                            }
                            uint32_t s8[8], x8[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float f0 = __uint_as_float(w[2 * j]), f1 = __uint_as_float(w[2 * j + 1]);
                                const float d0 = f0 - __uint_as_float(w[2 * j] & 0xFFFFE000u);
                                const float d1 = f1 - __uint_as_float(w[2 * j + 1] & 0xFFFFE000u);
                                const __nv_bfloat162 pp = __floats2bfloat162_rn(d0, d1);
                                const __nv_bfloat162 qq = __floats2bfloat162_rn(f0, f1);
                                const uint32_t mm = __heq2_mask(pp, pp);   // zero where Inf / NaN (see below)
                                s8[j] = *reinterpret_cast<const uint32_t *>(&pp) & mm;
                                x8[j] = *reinterpret_cast<const uint32_t *>(&qq) & mm;
                            }
                            tmem_st_32x8(t_slot + static_cast<uint32_t>(k0 >> 1), s8);
                            tmem_st_32x8(t_slot + 16u + static_cast<uint32_t>(k0 >> 1), x8);
                        }
                        tmem_st_wait();
                        tc_fence_before_sync();
                    }
#pragma unroll
                    for (int half = a_tmem ? 1 : 0; half < 2; ++half) {
                        const uint4 *rt = reinterpret_cast<const uint4 *>(raw_b + half * TILE_BYTES);
                        uint8_t *s16 = out_b + half * 2 * H_TILE_BYTES;
                        uint8_t *x16 = s16 + H_TILE_BYTES;
                        // With the extra converter warps at work (pair form), they take chunks
                        // [384, 1024) of the B tile.
                        const int n_here = (half == 1 && extra_conv) ? 3 : PER_T;
                        uint4 x[PER_T];
#pragma unroll
                        for (int u = 0; u < PER_T; ++u)
                            if (u < n_here) x[u] = rt[ctid + u * NCT];
                        float za = 0.0f, zb = 0.0f;
#pragma unroll
                        for (int u = 0; u < PER_T; ++u)
                            if (u < n_here) hybrid_chunk_unmasked(x[u], s16, x16, hyb_dst0[half] + u * (NCT * 8), za, zb);
                        if (!all_finite(za, zb)) {
#pragma unroll
                            for (int u = 0; u < PER_T; ++u)
                                if (u < n_here) hybrid_chunk(x[u], s16, x16, hyb_dst0[half] + u * (NCT * 8));
                        }
                    }
                } else if (!(args.dbg & 1))
#pragma unroll
                for (int base = 0; base < PER_THREAD; base += BATCH) {
                    uint4 x[BATCH];
#pragma unroll
                    for (int u = 0; u < BATCH; ++u) x[u] = raw[ctid + (base + u) * NCT];
#pragma unroll
                    for (int u = 0; u < BATCH; ++u) {
                        uint4 big, sm;
                        big.x = x[u].x & 0xFFFFE000u;
                        big.y = x[u].y & 0xFFFFE000u;
                        big.z = x[u].z & 0xFFFFE000u;
                        big.w = x[u].w & 0xFFFFE000u;
                        // small = x - big is exact; + 0x1000 on its bits rounds it to the nearest
                        // TF32 value once the tensor core drops the low 13 bits.
                        sm.x = __float_as_uint(__uint_as_float(x[u].x) - __uint_as_float(big.x)) + 0x1000u;
                        sm.y = __float_as_uint(__uint_as_float(x[u].y) - __uint_as_float(big.y)) + 0x1000u;
                        sm.z = __float_as_uint(__uint_as_float(x[u].z) - __uint_as_float(big.z)) + 0x1000u;
                        sm.w = __float_as_uint(__uint_as_float(x[u].w) - __uint_as_float(big.w)) + 0x1000u;
                        if (!(args.dbg & 4)) small[ctid + (base + u) * NCT] = sm;
                        else if (sm.x == 0x12345678u) small[0] = sm;
                        if (mask_big) raw[ctid + (base + u) * NCT] = big;
                    }
                }
                if (!(args.dbg & 2)) fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (PAIR)
                        mbar_arrive_cluster(conv_remote[sstage]);
                    else
                        mbar_arrive(&conv_bar[sstage]);
                }
                if constexpr (PROF) w_c += clock64() - busy0;
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
                if (++sstage == SMALL_STAGES) {
                    sstage = 0;
                    sphase ^= 1u;
                }
            }
        }
        if (PROF && args.prof && ctid == 0) {
            args.prof[blockIdx.x * kProfSlots + kProfConvSmallEmpty] = w_a;
            args.prof[blockIdx.x * kProfSlots + kProfConvFull] = w_b;
            args.prof[blockIdx.x * kProfSlots + kProfConvBusy] = w_c;
        }
    }

    // ---------------------------------------------------------------- fused all-gather, last tile
    // Every warp is done with its role by the time it gets here; the CTA's last tile has no
    // further math to hide behind, so all of them forward it.
    if (fwd_peers > 0 && n_store > 0) {
        if (wait_or_abort<false>(&last_full_bar, 0u, abort_flag)) {
            forward_tile<CG>(args, last_store_tile, static_cast<int>(cta_rank), threadIdx.x, C::NUM_THREADS);
        } else if (threadIdx.x == 0) {
            report(args.status, abort_flag, kErrForwardWait, 32u);
        }
        // Peer stores must have left this GPU before the kernel is reported complete.
        __threadfence_system();
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) {
        // Neither CTA may leave while its peer can still signal its barriers or the
        // pair's MMAs can still write its TMEM.
        cluster_arrive();
        cluster_wait();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc<CG>(tmem_base, C::TMEM_COLS);
    }
}

struct TcPlan {
    OperandView a, b;
    OperandMajor a_major, b_major;
};

bool plan(const Problem &p, TcPlan *pl, char *why, int why_len) {
    if (p.N > 0x7FFFFFFFLL || p.M > 0x7FFFFFFFLL || p.K > 0x7FFFFFFFLL || p.B > 0x7FFFFFFFLL) {
        if (why) snprintf(why, why_len, "extent above 2^31-1");
        return false;
    }
    pl->a = OperandView{p.a, p.N, p.K, p.B, p.a_si, p.a_sk, p.a_sb};
    pl->b = OperandView{p.b, p.M, p.K, p.B, p.b_sj, p.b_sk, p.b_sb};
    char w[128] = "";
    pl->a_major = classify_operand(pl->a, 4, w, sizeof(w));
    if (pl->a_major == kMajorNone) {
        if (why) snprintf(why, why_len, "lhs: %s", w);
        return false;
    }
    pl->b_major = classify_operand(pl->b, 4, w, sizeof(w));
    if (pl->b_major == kMajorNone) {
        if (why) snprintf(why, why_len, "rhs: %s", w);
        return false;
    }
    const long long tiles = ((p.N + BM - 1) / BM) * ((p.M + BNC - 1) / BNC) * p.B;
    if (tiles > 0x7FFFFFFFLL) {
        if (why) snprintf(why, why_len, "too many tiles");
        return false;
    }
    return true;
}

template <int CG>
int launch_cg(const Problem &p, TcArgs &args, int sms, int streamk_opt, int pieces_opt, int pair_opt) {
    using C = Cfg<CG>;
    args.tiles_m = static_cast<int>((p.N + C::TILE_M - 1) / C::TILE_M);
    args.tiles_n = static_cast<int>((p.M + C::TILE_N - 1) / C::TILE_N);
    args.total_tiles = args.tiles_m * args.tiles_n * args.B;
    // Per-device launch set-up, done once; several host threads may arrive here together.
    static std::mutex setup_mu;
    static bool attr_set[2][64] = {{false}};
    static int max_clusters[64] = {0};
    const int prof = (args.prof != nullptr && profile_level() == 1) ? 1 : 0;
    auto kernel = prof ? gemm_f32_3xtf32_kernel<CG, true> : gemm_f32_3xtf32_kernel<CG, false>;
    {
        std::lock_guard<std::mutex> lk(setup_mu);
        if (!attr_set[prof][p.device & 63]) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
            if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(smem)");
            attr_set[prof][p.device & 63] = true;
        }
    }
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(C::NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = p.stream;
    cudaLaunchAttribute attr[1];
    int units = sms / CG;  // CTAs (CG = 1) or CTA pairs (CG = 2) resident at once
    if (CG == 2) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        std::lock_guard<std::mutex> lk(setup_mu);
        if (max_clusters[p.device & 63] == 0) {
            cfg.gridDim = dim3(static_cast<unsigned>(2 * units));
            int n = 0;
            cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
            if (e != cudaSuccess) return cuda_fail(e, "cudaOccupancyMaxActiveClusters");
            if (n < 1) {
                set_error("no CTA pair of the tcgen05 kernel fits on device %d", p.device);
                return TTB_ECUDA;
            }
            max_clusters[p.device & 63] = n;
        }
        if (units > max_clusters[p.device & 63]) units = max_clusters[p.device & 63];
    }
    // Whole tiles per unit leave SMs idle in the last wave (or all along, with fewer tiles
    // than units); stream-K deals the K blocks out evenly instead.  It pays when that loss is
    // noticeable and every unit still gets a few K blocks.
    const long long num_kb = (p.K + BK - 1) / BK;
    const long long total_kb = args.total_tiles * num_kb;
    // Few tiles (less than half the units would have one): cut every tile's K over several
    // units, four K blocks or more each, so that most of the GPU works on a small product.
    const bool sk_small = streamk_opt != 0 && args.total_tiles > 0 && args.total_tiles * 2 <= units && num_kb >= 8;
    if (sk_small) {
        long long u = total_kb / 4;
        if (u > units) u = units;
        if (u < args.total_tiles) u = args.total_tiles;
        units = static_cast<int>(u);
    }
    const long long waves = (args.total_tiles + units - 1) / units;
    const double busy = static_cast<double>(args.total_tiles) / static_cast<double>(waves * units);
    long long waves_full = args.total_tiles / units;
    const long long rem = args.total_tiles % units;
    // Whole waves of tiles stay whole; the K blocks of the last partial wave are dealt out over
    // all units (with no whole wave: of every tile).  That replaces a wave of num_kb K blocks
    // by one of cut_kb_per_unit plus a fix-up (worth a few K blocks), so it pays when the
    // difference is a dozen K blocks or more.
    // Fused all-gather: every tile is cut that way.  Whole waves finish all their tiles at the
    // same moment, so the exchange would come in bursts with the last one exposed; with every
    // unit's range crossing tile boundaries at its own time, tiles complete (and leave for the
    // peers) evenly over the whole kernel.
    const bool exchange = args.n_peers > 0 || args.mc_c != nullptr;
    if (exchange && waves_full < 3 && total_kb / units >= 16) waves_full = 0;  // (many waves: the bursts are small)
    const long long cut_tiles = waves_full > 0 ? rem : args.total_tiles;
    const long long cut_kb_per_unit = cut_tiles * num_kb / units;
    const bool sk_worth = waves_full > 0 ? num_kb - cut_kb_per_unit >= 12
                                         : ((num_kb >= 64 && cut_kb_per_unit >= 16) || (sk_small && units > args.total_tiles) ||
                                            (exchange && cut_kb_per_unit >= 16));
    const bool sk_possible = cut_tiles > 0 && cut_kb_per_unit >= 4 && cut_tiles * num_kb < 0x7FFFFFFFLL &&
                             waves_full + 3 <= kMaxSegments && args.total_tiles / units + 3 <= kMaxSegments;
    bool streamk = streamk_opt > 0 ? sk_possible
                                   : (streamk_opt < 0 && sk_possible && sk_worth && (busy < 0.93 || exchange));
    args.sk_tile0 = static_cast<int>(waves_full * units);
    if (streamk) {
        int rc = streamk_workspace(p.device, p.stream, &args.sk_partials, &args.sk_flags);
        if (rc != TTB_OK) {
            streamk = false;  // no workspace for this stream: whole tiles, and the call succeeds
            set_error("%s", "");
        }
    }
    args.streamk = streamk ? 1 : 0;
    if (!streamk && units > args.total_tiles) units = args.total_tiles;
    // Paired stream-K (see TcArgs): halves the number of tiles that complete at the very end.
    args.sk_pair = 0;
    {
        const bool sends = (args.n_peers > 0 && args.peer_tma) || args.mc_c != nullptr;
        const bool fwd = args.n_peers > 0 && !args.peer_tma && args.mc_c == nullptr;  // counts its stores ahead
        const bool want = pair_opt < 0 ? sends : pair_opt != 0;
        if (streamk && want && !fwd && cut_kb_per_unit >= num_kb + 1 &&
            static_cast<long long>(args.total_tiles) * CG * 8 <= kStreamKTickets) {
            args.sk_pair = 1;
            args.sk_tickets = args.sk_flags + static_cast<size_t>(sms) * 16;
        }
    }
    // Piece schedule instead (see TcArgs): wanted when tiles should complete all through the
    // kernel, i.e. with an all-gather fused into the product that the epilogue itself sends.
    args.pieces = 0;
    {
        const bool sends = (args.n_peers > 0 && args.peer_tma) || args.mc_c != nullptr;
        int want = pieces_opt < 0 ? 0 : pieces_opt;  // measured: the hand-overs cost more than the spread-out exchange gains
        (void)sends;
        if (args.n_peers > 0 && !args.peer_tma && args.mc_c == nullptr) want = 0;  // forwarding warps count stores ahead
        const int kc = args.k_chunk > 0 ? args.k_chunk : 1;
        if (want > 1 && num_kb >= 2 * kc && args.total_tiles > 0 &&
            static_cast<long long>(args.total_tiles) * CG * 8 <= kStreamKTickets) {
            // a power of two of equal non-empty parts, each a whole number of accumulation chunks
            int lg = 0;
            while ((2 << lg) <= want) ++lg;
            long long len = 0, parts = 0;
            int pu = sms / CG;
            if (CG == 2 && pu > max_clusters[p.device & 63]) pu = max_clusters[p.device & 63];
            for (; lg > 0; --lg) {
                len = (num_kb + (1 << lg) - 1) >> lg;
                len = (len + kc - 1) / kc * kc;
                parts = (num_kb + len - 1) / len;
                // equal parts, and a unit's list of parts must fit the kernel's segment table
                if (parts == (1 << lg) && (args.total_tiles * parts + pu - 1) / pu <= kMaxSegments) break;
            }
            if (lg > 0 && args.total_tiles * parts < 0x7FFFFFFFLL) {
                args.pieces_log2 = lg;
                int rc = TTB_OK;
                if (!streamk) rc = streamk_workspace(p.device, p.stream, &args.sk_partials, &args.sk_flags);
                if (rc == TTB_OK) {
                    args.pieces = static_cast<int>(parts);
                    args.piece_len = static_cast<int>(len);
                    args.sk_tickets = args.sk_flags + static_cast<size_t>(sms) * 16;
                    args.streamk = 1;   // the kernel reads its parts from the segment table, as for stream-K
                    units = sms / CG;
                    if (CG == 2 && units > max_clusters[p.device & 63]) units = max_clusters[p.device & 63];
                    if (units > args.total_tiles * parts) units = static_cast<int>(args.total_tiles * parts);
                } else {
                    set_error("%s", "");
                }
            }
        }
    }
    cfg.gridDim = dim3(static_cast<unsigned>(units * CG));
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args);
    if (e != cudaSuccess) return cuda_fail(e, "gemm_f32_3xtf32_kernel launch");
    note_launch(CG == 2 ? TTB_VARIANT_TCGEN05_2CTA : TTB_VARIANT_TCGEN05_3XTF32, 1);
    return TTB_OK;
}

}  // namespace

bool f32_tcgen05_eligible(const Problem &p, char *why, int why_len) {
    TcPlan pl;
    return plan(p, &pl, why, why_len);
}

int launch_f32_tcgen05(const Problem &p, const F32Options &opt, int n_peers, void *const *peer_c, void *mc_c) {
    TcPlan pl;
    char why[200] = "";
    if (!plan(p, &pl, why, sizeof(why))) {
        set_error("tcgen05 f32 kernel cannot take these views: %s", why);
        return TTB_EUNSUPPORTED;
    }
    TcArgs args;
    memset(&args, 0, sizeof(args));
    if (encode_operand_tmap(&args.tmap_a, pl.a, pl.a_major, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, 32, BM, BK,
                            &args.a_batch_mul, why, sizeof(why)) ||
        encode_operand_tmap(&args.tmap_b, pl.b, pl.b_major, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, 32, BNC, BK,
                            &args.b_batch_mul, why, sizeof(why))) {
        set_error("tensor map: %s", why);
        return TTB_EUNSUPPORTED;
    }
    {
        // C as a "K-major operand": inner dim = columns (unit stride), outer = rows.
        const OperandView cv{p.c, p.N, p.M, p.B, p.c_si, p.c_sj, p.c_sb};
        char cw[128] = "";
        args.c_tma = 0;
        if (p.c_sb != 0 && classify_operand(cv, 4, cw, sizeof(cw)) == kMajorK &&
            encode_operand_tmap(&args.tmap_c, cv, kMajorK, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, 32, 32, 32,
                                &args.c_batch_mul, cw, sizeof(cw)) == 0)
            args.c_tma = 1;
    }
    args.c = static_cast<float *>(p.c);
    args.c_sb = p.c_sb;
    args.c_si = p.c_si;
    args.c_sj = p.c_sj;
    args.d = static_cast<const float *>(p.d);
    args.d_sb = p.d_sb;
    args.d_si = p.d_si;
    args.d_sj = p.d_sj;
    args.act = p.act;
    args.N = static_cast<int>(p.N);
    args.M = static_cast<int>(p.M);
    args.K = static_cast<int>(p.K);
    args.B = static_cast<int>(p.B);
    args.a_mn_major = pl.a_major == kMajorMN;
    args.b_mn_major = pl.b_major == kMajorMN;
    args.terms = opt.terms;
    args.a_tmem = opt.a_tmem;
    args.extra_conv = opt.extra_conv;
    args.k_chunk = opt.k_chunk > 0 ? opt.k_chunk : DEFAULT_K_CHUNK;
    if (opt.k_chunk < 0) args.k_chunk = 0;  // whole K inside TMEM (test only)
    args.mask_big = opt.mask_big;
    if (n_peers < 0 || n_peers > kMaxPeers) {
        set_error("fused all-gather takes at most %d peers, got %d", kMaxPeers, n_peers);
        return TTB_ELIMIT;
    }
    args.n_peers = n_peers;
    for (int i = 0; i < n_peers; ++i) args.peer_c[i] = static_cast<float *>(peer_c[i]);
    args.mc_c = nullptr;
    if (mc_c != nullptr) {
        // multimem.st moves 16 bytes: rows of C must be 16-byte aligned and M a multiple of 4
        const bool ok = p.c_sj == 1 && (p.c_si & 3) == 0 && (p.c_sb & 3) == 0 && (p.M & 3) == 0 &&
                        (reinterpret_cast<uintptr_t>(p.c) & 15) == 0 && (reinterpret_cast<uintptr_t>(mc_c) & 15) == 0;
        if (!ok || n_peers != 0) {
            set_error("multicast all-gather needs row-contiguous, 16-byte-aligned C with M a multiple of 4 (and no peer list)");
            return TTB_EUNSUPPORTED;
        }
        args.mc_c = static_cast<float *>(mc_c);
    }
    // When C can be described to TMA here and on every peer, the epilogue sends each box to the
    // peers itself (bulk tensor stores from its staging buffer); otherwise the forwarding warps do.
    args.peer_tma = 0;
    if (n_peers > 0 && args.c_tma && opt.peer_tma) {
        args.peer_tma = 1;
        for (int i = 0; i < n_peers && args.peer_tma; ++i) {
            const OperandView pv{peer_c[i], p.N, p.M, p.B, p.c_si, p.c_sj, p.c_sb};
            char pw[128] = "";
            int mul = 0;
            if (classify_operand(pv, 4, pw, sizeof(pw)) != kMajorK ||
                encode_operand_tmap(&args.tmap_peer[i], pv, kMajorK, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, 32, 32, 32, &mul,
                                    pw, sizeof(pw)) != 0)
                args.peer_tma = 0;
        }
    }
    // Warps 2-3 either forward tiles to the peers (fallback form of the fused all-gather) or convert.
    if (args.n_peers > 0 && !args.peer_tma && args.mc_c == nullptr) args.extra_conv = 0;
    int rc = device_status_ptr(p.device, &args.status);
    if (rc != TTB_OK) return rc;
    args.prof = profile_ptr(p.device);
    args.dbg = opt.dbg;
    int sms = 148;
    sm_count(p.device, &sms);
    if (opt.two_cta) return launch_cg<2>(p, args, sms, opt.streamk, opt.pieces, opt.sk_pair);
    return launch_cg<1>(p, args, sms, opt.streamk, opt.pieces, opt.sk_pair);
}

}  // namespace ttb
