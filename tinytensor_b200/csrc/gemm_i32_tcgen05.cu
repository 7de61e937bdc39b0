// gemm_i32_tcgen05.cu -- i32 batched GEMM, exact mod 2^32, on the int8 tensor cores of sm_100a.
//
// C[b] = A[b] . B[b] with int32 operands and wrap-around sums, which is what the reference's
// matmul_kernel<int> computes on CUDA cores (tinytensor/tensor/backend/cuda/kernel/matmul.cuh:
// 27-151, accumulation in T).  Every operand word splits into four unsigned bytes,
//   x = x0 + x1 2^8 + x2 2^16 + x3 2^24   (two's complement bits),
// so  a.b = sum over i, j of a_i b_j 2^(8(i+j))  and, mod 2^32, only the ten pairs with
// i + j <= 3 survive.  Per byte weight s = i + j the tensor cores accumulate
//   P_s = sum over k and over i + j = s of a_i[k] b_j[k]
// with tcgen05.mma kind::i8 (u8 x u8 -> s32, no saturation, so P_s itself wraps mod 2^32,
// which is all the result needs), and the epilogue combines
//   C = P_0 + (P_1 << 8) + (P_2 << 16) + (P_3 << 24)   mod 2^32.
// Bit-exact for every input, any K.  Ten int8 MMAs (at twice the bf16 rate) replace the
// 32-bit multiply-adds of the CUDA-core kernel.
//
// Two forms.  CG = 1: one CTA per SM, persistent over 128 x 128 tiles.  CG = 2: CTA pairs
// (cta_group::2) over 256 x 128 tiles: each CTA loads and splits 128 rows of A and 64 columns
// of B and owns 128 rows of the four accumulators; the pair's MMAs read both halves of B, so a
// CTA moves a quarter less through shared memory per product (the binding resource).  Roles by
// warp (in each CTA; only the leader CTA of a pair issues MMAs):
//   warp 0       TMA producer: raw int32 tiles of A and B (32 K-elements = 128 bytes per row),
//                through the same stride-derived tensor maps as the f32 kernel, so permuted
//                views need no copy;
//   warp 1       MMA issuer: per K block ten tcgen05.mma into four TMEM accumulators
//                (4 x 128 columns = all of tensor memory);
//   warps 4-11   epilogue (two warps per TMEM lane quarter, 64 columns each): tcgen05.ld the
//                four accumulators 16 columns at a time, shift, add, add the fused addend if
//                any, store C;
//   warps 12-15  converters: split the raw tiles into four byte planes per operand, each a
//                K-major 128 x 32-byte tile in the unswizzled core-matrix layout
//                ([K half][row][16 bytes]), fence.proxy.async, signal.
// The MMAs never read the raw tiles, so a raw slot is released by the converters and a plane
// slot by tcgen05.commit.  All waits are bounded; a wait that gives up writes an error word and
// the CTA unwinds (TMEM freed) instead of hanging.
#include <cuda.h>

#include <cstdio>
#include <cstring>

#include "common.cuh"
#include "ptx.cuh"
#include "tma_desc.cuh"

namespace ttb {
namespace {

using namespace ptx;

constexpr int BM = 128;               // rows of A / columns of B per tile
constexpr int BK = 32;                // int32 per K block = 128 bytes = one swizzle row
constexpr int RAW_STAGES = 4;         // raw ring (TMA -> converters)
constexpr int PLANE_STAGES = 2;       // byte-plane ring (converters -> MMAs)
constexpr int TILE_BYTES = BM * BK * 4;      // 16 KiB: one raw operand tile
constexpr int STAGE_BYTES = 2 * TILE_BYTES;  // raw A + raw B; a plane slot has the same size
constexpr int PLANE_BYTES = BM * BK;         // 4 KiB: one byte plane of one operand
constexpr int PLANE_RING_OFFSET = RAW_STAGES * STAGE_BYTES;
constexpr int OUT_STAGING_OFFSET = (RAW_STAGES + PLANE_STAGES) * STAGE_BYTES;  // epilogue store staging
constexpr int OUT_STAGING_WARP_BYTES = 32 * 128;                               // 32 rows x 32 words per warp
constexpr int SMEM_BYTES = OUT_STAGING_OFFSET + 8 * OUT_STAGING_WARP_BYTES + 1024;
constexpr int MN_BOX_BYTES = 32 * BK * 4;    // one MN-major TMA box: 32 (MN) x BK (K)
constexpr int EPI_WARPS = 8;           // two per TMEM lane quarter: each takes 64 of a tile's 128 columns
constexpr int FIRST_EPI_WARP = 4, FIRST_CONV_WARP = FIRST_EPI_WARP + EPI_WARPS, NUM_CONV_WARPS = 4;
constexpr int NUM_THREADS = (FIRST_CONV_WARP + NUM_CONV_WARPS) * 32;
constexpr int TMEM_COLS = 512;        // P_0 .. P_3, 128 columns each
constexpr int BN = 128;               // columns of B per tile (split over the CTAs of a pair)

struct alignas(64) I8Args {
    CUtensorMap tmap_a;
    CUtensorMap tmap_b;
    CUtensorMap tmap_c;  // C as {M, N, B} with 32 x 32 boxes, for the epilogue's bulk tensor stores
    int c_tma;           // tmap_c is valid (C rows contiguous and 16-byte aligned)
    int c_batch_mul;     // 0 pins the batch coordinate (B == 1)
    int32_t *c;
    long long c_sb, c_si, c_sj;
    const int32_t *d;  // fused addend view (bias row / column, or C itself), nullptr = none
    long long d_sb, d_si, d_sj;
    int N, M, K, B;
    int a_mn_major, b_mn_major;
    int a_batch_mul, b_batch_mul;
    int tiles_m, tiles_n, total_tiles;
    DeviceStatus *status;
    int dbg;  // test switch, bit 4: the first stage is armed but never loaded, so the bounded waits
              // downstream must run out and the kernel unwind by itself (results are absent then)
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait (2 s of %globaltimer) that also leaves early when another role of this CTA gave up.
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
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

// Tile order: groups of 8 row tiles sweep all column tiles, so the CTAs running at one time
// share A rows and B columns in L2.
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

// D[tmem] (+)= A * B with 8-bit integer inputs over a CTA pair (cta_group::2).
__device__ __forceinline__ void mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "setp.ne.b32 P, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, P;\n\t"
        "}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// Four words (k, k+1, k+2, k+3 of one row) -> one word per byte plane, byte i = plane of word i.
__device__ __forceinline__ void planes_of(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t &p0,
                                          uint32_t &p1, uint32_t &p2, uint32_t &p3) {
    const uint32_t lo01 = prmt(w0, w1, 0x5140), lo23 = prmt(w2, w3, 0x5140);  // bytes 0 and 1 of each word
    const uint32_t hi01 = prmt(w0, w1, 0x7362), hi23 = prmt(w2, w3, 0x7362);  // bytes 2 and 3
    p0 = prmt(lo01, lo23, 0x5410);
    p1 = prmt(lo01, lo23, 0x7632);
    p2 = prmt(hi01, hi23, 0x5410);
    p3 = prmt(hi01, hi23, 0x7632);
}

template <int CG>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_i32_limb_kernel(const __grid_constant__ I8Args args) {
    constexpr bool PAIR = CG == 2;
    constexpr int TILE_M = BM * CG;       // rows of C per CTA (pair)
    constexpr int B_COLS = BN / CG;       // columns of B this CTA loads and splits
    constexpr int B_RAW_BYTES = B_COLS * BK * 4;
    constexpr int B_PLANE_BYTES = B_COLS * BK;
    extern __shared__ uint8_t smem_dyn[];
    __shared__ uint64_t full_bar[RAW_STAGES];     // TMA bytes landed
    __shared__ uint64_t empty_bar[RAW_STAGES];    // converters are done with the raw slot
    __shared__ uint64_t plane_full_bar[PLANE_STAGES];   // byte planes written (lives in the leader CTA)
    __shared__ uint64_t plane_empty_bar[PLANE_STAGES];  // MMAs that read the plane slot are done (local)
    __shared__ uint64_t acc_full_bar;             // all K blocks of the tile accumulated (local)
    __shared__ uint64_t acc_empty_bar;            // accumulators read out (lives in the leader CTA)
    __shared__ uint64_t drain_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag_s;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
    const bool leader = cta_rank == 0;
    volatile int *abort_flag = &abort_flag_s;
    const uint32_t dyn_base = smem_u32(smem_dyn);
    const uint32_t tiles_base = (dyn_base + 1023u) & ~1023u;
    uint8_t *tiles = smem_dyn + (tiles_base - dyn_base);

    if (threadIdx.x == 0) {
        for (int s = 0; s < RAW_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], NUM_CONV_WARPS);
        }
        for (int s = 0; s < PLANE_STAGES; ++s) {
            mbar_init(&plane_full_bar[s], NUM_CONV_WARPS * CG);
            mbar_init(&plane_empty_bar[s], 1);
        }
        mbar_init(&acc_full_bar, 1);
        mbar_init(&acc_empty_bar, EPI_WARPS * CG);
        mbar_init(&drain_bar, 1);
        abort_flag_s = 0;
        fence_mbar_init();
        tma_prefetch_desc(&args.tmap_a);
        tma_prefetch_desc(&args.tmap_b);
    }
    if (warp == 1) {
        tmem_alloc<CG>(&tmem_base_slot, TMEM_COLS);
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

    const int num_kb = (args.K + BK - 1) / BK;
    const int unit = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int units = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    const int n_tiles = unit < args.total_tiles ? (args.total_tiles - unit + units - 1) / units : 0;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int issued = 0;
            for (int i = 0; i < n_tiles && ok; ++i) {
                int b, tm, tn;
                tile_coords(unit + i * units, args.tiles_m, args.tiles_n, b, tm, tn);
                const int m0 = tm * TILE_M + static_cast<int>(cta_rank) * BM;
                const int n0 = tn * BN + static_cast<int>(cta_rank) * B_COLS;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!wait_or_abort(&empty_bar[stage], phase ^ 1u, abort_flag)) {
                        report(args.status, abort_flag, kErrProducerWait, static_cast<unsigned>(stage));
                        ok = false;
                        break;
                    }
                    uint8_t *a_dst = tiles + stage * STAGE_BYTES;
                    uint8_t *b_dst = a_dst + TILE_BYTES;
                    mbar_arrive_expect_tx(&full_bar[stage], TILE_BYTES + B_RAW_BYTES);
                    const int k0 = kb * BK;
                    if ((args.dbg & 16) && issued == 0) {
                        ++issued;
                        if (++stage == RAW_STAGES) {
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
                        for (int j = 0; j < B_COLS / 32; ++j)
                            tma_load_3d(b_dst + j * MN_BOX_BYTES, &args.tmap_b, &full_bar[stage], n0 + 32 * j, k0,
                                        b * args.b_batch_mul);
                    } else {
                        tma_load_3d(b_dst, &args.tmap_b, &full_bar[stage], k0, n0, b * args.b_batch_mul);
                    }
                    ++issued;
                    if (++stage == RAW_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok && issued > 0) {
                // Let the copies already in flight land before the CTA's shared memory is given
                // up: wait (bounded) for the last stage issued.
                const int last = (stage + RAW_STAGES - 1) % RAW_STAGES;
                const uint32_t last_phase = (stage == 0) ? (phase ^ 1u) : phase;
                for (int i = 0; i < 100000; ++i)
                    if (mbar_try_wait(&full_bar[last], last_phase)) break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && leader) {
            const uint32_t idesc = make_idesc_u8(BM * CG, BN);
            int ps = 0;
            uint32_t pphase = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int i = 0; i < n_tiles && ok; ++i) {
                if (!wait_or_abort(&acc_empty_bar, acc_phase ^ 1u, abort_flag)) {
                    report(args.status, abort_flag, kErrAccEmptyWait, 0u);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!wait_or_abort(&plane_full_bar[ps], pphase, abort_flag)) {
                        report(args.status, abort_flag, kErrMmaWait, static_cast<unsigned>(ps));
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    // Plane tile: [K half][row][16 bytes]: core matrices (8 rows x 16 B) 128 B apart
                    // along the rows (SBO), the two K halves one half-tile apart (LBO): 2048 B for
                    // the 128 rows of A, 16 B x this CTA's columns of B.
                    const uint32_t a_planes = tiles_base + PLANE_RING_OFFSET + ps * STAGE_BYTES;
                    const uint32_t b_planes = a_planes + 4 * PLANE_BYTES;
                    const uint32_t fresh = kb != 0 ? 1u : 0u;
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
#pragma unroll
                        for (int ia = 0; ia <= s; ++ia) {
                            const int ib = s - ia;
                            const uint64_t da = make_smem_desc(a_planes + ia * PLANE_BYTES, 2048, 128, kSwizzleNone);
                            const uint64_t db =
                                make_smem_desc(b_planes + ib * B_PLANE_BYTES, B_COLS * 16, 128, kSwizzleNone);
                            if constexpr (PAIR)
                                mma_i8_pair(tmem_base + static_cast<uint32_t>(s * BN), da, db, idesc, ia == 0 ? fresh : 1u);
                            else
                                mma_i8(tmem_base + static_cast<uint32_t>(s * BN), da, db, idesc, ia == 0 ? fresh : 1u);
                        }
                    }
                    // (one arrival per barrier reaches both CTAs of a pair)
                    if constexpr (PAIR)
                        mma_commit_both(smem_u32(&plane_empty_bar[ps]));
                    else
                        mma_commit<CG>(smem_u32(&plane_empty_bar[ps]));
                    if (++ps == PLANE_STAGES) {
                        ps = 0;
                        pphase ^= 1u;
                    }
                }
                if (!ok) break;
                if constexpr (PAIR)
                    mma_commit_both(smem_u32(&acc_full_bar));
                else
                    mma_commit<CG>(smem_u32(&acc_full_bar));
                acc_phase ^= 1u;
            }
            // Everything issued must have retired before TMEM is freed.
            mma_commit<CG>(smem_u32(&drain_bar));
            for (int i = 0; i < 1000000; ++i)
                if (mbar_try_wait(&drain_bar, 0)) break;
        }
    } else if (warp >= FIRST_EPI_WARP && warp < FIRST_CONV_WARP) {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;  // TMEM lanes [32 * quarter, +32)
        const int col_half = (warp - FIRST_EPI_WARP) >> 2;  // columns [64 * col_half, +64) of the tile
        uint32_t acc_phase = 0;
        bool ok = true;
        const uint32_t acc_empty_remote = PAIR ? mapa(smem_u32(&acc_empty_bar), 0) : 0u;
        const bool vec_ok = args.c_sj == 1 && (args.c_si & 3) == 0 && (args.c_sb & 3) == 0 &&
                            (reinterpret_cast<uintptr_t>(args.c) & 15) == 0;
        for (int i = 0; i < n_tiles && ok; ++i) {
            int b, tm, tn;
            tile_coords(unit + i * units, args.tiles_m, args.tiles_n, b, tm, tn);
            if (!wait_or_abort(&acc_full_bar, acc_phase, abort_flag)) {
                if (lane == 0) report(args.status, abort_flag, kErrEpilogueWait, 0u);
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const int row = tm * TILE_M + static_cast<int>(cta_rank) * BM + quarter * 32 + lane;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
            int32_t *crow = args.c + static_cast<long long>(b) * args.c_sb + static_cast<long long>(row) * args.c_si;
            const int32_t *drow = args.d ? args.d + static_cast<long long>(b) * args.d_sb +
                                               static_cast<long long>(row) * args.d_si
                                         : nullptr;
            // Read this warp's 32 rows x 64 columns of all four accumulators, combining as they
            // arrive, then hand tensor memory back to the MMA thread BEFORE storing: the stores of
            // this tile overlap the next tile's products.
            uint32_t out[64];
            const uint32_t t_col = t_row + static_cast<uint32_t>(col_half * 64);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                uint32_t p0[8], p1[8], p2[8], p3[8];
                tmem_ld_32x8(t_col + static_cast<uint32_t>(0 * BN + q * 8), p0);
                tmem_ld_32x8(t_col + static_cast<uint32_t>(1 * BN + q * 8), p1);
                tmem_ld_32x8(t_col + static_cast<uint32_t>(2 * BN + q * 8), p2);
                tmem_ld_32x8(t_col + static_cast<uint32_t>(3 * BN + q * 8), p3);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j) out[q * 8 + j] = p0[j] + (p1[j] << 8) + (p2[j] << 16) + (p3[j] << 24);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR)
                    mbar_arrive_cluster(acc_empty_remote);
                else
                    mbar_arrive(&acc_empty_bar);
            }
            const int col0 = tn * BN + col_half * 64;
            if (col0 < args.M) {
                if (drow && row < args.N) {
#pragma unroll
                    for (int j = 0; j < 64; ++j)
                        if (col0 + j < args.M)
                            out[j] += static_cast<uint32_t>(drow[static_cast<long long>(col0 + j) * args.d_sj]);
                }
                if (args.c_tma) {
                    // Row-contiguous, 16-byte-aligned C: 32 columns at a time go through this
                    // warp's 4 KiB of shared memory in the 128-byte-swizzled layout of a 32 x 32 TMA
                    // box and leave as one bulk tensor store, which writes whole lines and clips
                    // at the edges of C.  A thread storing its own row from registers would make
                    // every store instruction touch 32 different lines and crowd the load/store
                    // unit the converters need.
                    uint8_t *stg = tiles + OUT_STAGING_OFFSET + (warp - FIRST_EPI_WARP) * OUT_STAGING_WARP_BYTES;
                    const int row_base = row - lane;
#pragma unroll
                    for (int ch = 0; ch < 2; ++ch) {
                        if (lane == 0) bulk_wait_read_all();  // the previous box has left the buffer
                        __syncwarp();
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<uint4 *>(stg + lane * 128 + ((c ^ (lane & 7)) << 4)) =
                                make_uint4(out[ch * 32 + 4 * c], out[ch * 32 + 4 * c + 1], out[ch * 32 + 4 * c + 2],
                                           out[ch * 32 + 4 * c + 3]);
                        fence_proxy_async_smem();
                        __syncwarp();
                        const int gcol = col0 + ch * 32;
                        if (lane == 0 && row_base < args.N && gcol < args.M) {
                            tma_store_3d(&args.tmap_c, stg, gcol, row_base, b * args.c_batch_mul);
                            bulk_commit_group();
                        }
                    }
                } else if (row < args.N) {
                    if (vec_ok && col0 + 64 <= args.M) {
                        uint4 *dst = reinterpret_cast<uint4 *>(crow + col0);
#pragma unroll
                        for (int v = 0; v < 16; ++v)
                            dst[v] = make_uint4(out[4 * v], out[4 * v + 1], out[4 * v + 2], out[4 * v + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 64; ++j)
                            if (col0 + j < args.M)
                                crow[static_cast<long long>(col0 + j) * args.c_sj] = static_cast<int32_t>(out[j]);
                    }
                }
            }
            acc_phase ^= 1u;
        }
        // Bulk tensor stores in flight read this CTA's shared memory: done before it is given up.
        if (lane == 0) bulk_wait_all();
    } else if (warp >= FIRST_CONV_WARP) {
        // ------------------------------------------------------------ converters
        const int r = threadIdx.x - FIRST_CONV_WARP * 32;  // 0..127: the row of A this thread splits
        uint32_t plane_full_remote[PLANE_STAGES] = {0, 0};
        if constexpr (PAIR) {
            for (int s = 0; s < PLANE_STAGES; ++s) plane_full_remote[s] = mapa(smem_u32(&plane_full_bar[s]), 0);
        }
        int stage = 0;
        uint32_t phase = 0;
        int ps = 0;
        uint32_t pphase = 0;
        bool ok = true;
        const long long total_kb = static_cast<long long>(n_tiles) * num_kb;
        for (long long it = 0; it < total_kb; ++it) {
            if (!wait_or_abort(&plane_empty_bar[ps], pphase ^ 1u, abort_flag) ||
                !wait_or_abort(&full_bar[stage], phase, abort_flag)) {
                if (lane == 0) report(args.status, abort_flag, kErrConverterWait, static_cast<unsigned>(stage));
                ok = false;
                break;
            }
            const uint8_t *raw = tiles + stage * STAGE_BYTES;
            uint8_t *planes = tiles + PLANE_RING_OFFSET + ps * STAGE_BYTES;
            // One work item = 16 consecutive K elements of one row (A) or column (B): four byte
            // planes x 16 bytes.  A has 128 rows x 2 K halves; B has B_COLS columns x 2 K halves.
            // Thread r takes both halves of A's row r and, for B, column (item % B_COLS) and half
            // (item / B_COLS) of items r (and r + 128 when a CTA holds all 128 columns).
            auto split = [&](const uint8_t *rt, uint8_t *pl, bool mn, int rr, int half, int lbo) {
                uint32_t w[16];
                if (!mn) {
                    // K-major raw tile: 128-byte rows, 16-byte chunks XORed with (row & 7)
                    const uint8_t *row = rt + rr * 128;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint4 v = *reinterpret_cast<const uint4 *>(row + (((half * 4 + c) ^ (rr & 7)) << 4));
                        w[4 * c] = v.x;
                        w[4 * c + 1] = v.y;
                        w[4 * c + 2] = v.z;
                        w[4 * c + 3] = v.w;
                    }
                } else {
                    // MN-major raw tile: boxes of 32 (MN) x 32 (K); a K row is 128 bytes with
                    // 32-byte chunks XORed with (k & 3)
                    const uint8_t *box = rt + (rr >> 5) * MN_BOX_BYTES + ((rr & 7) << 2);
                    const int chunk = (rr & 31) >> 3;
#pragma unroll
                    for (int kk = 0; kk < 16; ++kk) {
                        const int k = half * 16 + kk;
                        w[kk] = *reinterpret_cast<const uint32_t *>(box + k * 128 + ((chunk ^ (k & 3)) << 5));
                    }
                }
                uint4 q0, q1, q2, q3;
                planes_of(w[0], w[1], w[2], w[3], q0.x, q1.x, q2.x, q3.x);
                planes_of(w[4], w[5], w[6], w[7], q0.y, q1.y, q2.y, q3.y);
                planes_of(w[8], w[9], w[10], w[11], q0.z, q1.z, q2.z, q3.z);
                planes_of(w[12], w[13], w[14], w[15], q0.w, q1.w, q2.w, q3.w);
                const int plane_bytes = lbo * 2;
                uint8_t *dst = pl + half * lbo + rr * 16;
                *reinterpret_cast<uint4 *>(dst) = q0;
                *reinterpret_cast<uint4 *>(dst + plane_bytes) = q1;
                *reinterpret_cast<uint4 *>(dst + 2 * plane_bytes) = q2;
                *reinterpret_cast<uint4 *>(dst + 3 * plane_bytes) = q3;
            };
            const bool a_mn = args.a_mn_major != 0, b_mn = args.b_mn_major != 0;
            split(raw, planes, a_mn, r, 0, 2048);
            split(raw, planes, a_mn, r, 1, 2048);
#pragma unroll
            for (int item = r; item < 2 * B_COLS; item += 128)
                split(raw + TILE_BYTES, planes + 4 * PLANE_BYTES, b_mn, item % B_COLS, item / B_COLS, B_COLS * 16);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR)
                    mbar_arrive_cluster(plane_full_remote[ps]);
                else
                    mbar_arrive(&plane_full_bar[ps]);
                mbar_arrive(&empty_bar[stage]);
            }
            if (++stage == RAW_STAGES) {
                stage = 0;
                phase ^= 1u;
            }
            if (++ps == PLANE_STAGES) {
                ps = 0;
                pphase ^= 1u;
            }
        }
        (void)ok;
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) {
        // Neither CTA may leave while its peer can still signal its barriers or the pair's MMAs
        // can still write its TMEM.
        cluster_arrive();
        cluster_wait();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc<CG>(tmem_base, TMEM_COLS);
    }
}

struct I8Plan {
    OperandView a, b;
    OperandMajor a_major, b_major;
};

bool plan(const Problem &p, I8Plan *pl, char *why, int why_len) {
    if (p.dtype != TTB_I32) {
        if (why) snprintf(why, why_len, "dtype is not i32");
        return false;
    }
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
    const long long tiles = ((p.N + BM - 1) / BM) * ((p.M + BM - 1) / BM) * p.B;
    if (tiles > 0x7FFFFFFFLL) {
        if (why) snprintf(why, why_len, "too many tiles");
        return false;
    }
    return true;
}

}  // namespace

bool i32_tcgen05_eligible(const Problem &p, char *why, int why_len) {
    I8Plan pl;
    return plan(p, &pl, why, why_len);
}

namespace {

template <int CG>
int launch_i32_cg(const Problem &p, const I8Plan &pl, int dbg) {
    char why[200] = "";
    I8Args args;
    memset(&args, 0, sizeof(args));
    // The raw tiles are moved as 32-bit words; the same maps as the f32 kernel's.  A K-major
    // rhs is boxed by the columns one CTA loads (all 128, or 64 in a CTA pair).
    if (encode_operand_tmap(&args.tmap_a, pl.a, pl.a_major, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, 32, BM, BK,
                            &args.a_batch_mul, why, sizeof(why)) ||
        encode_operand_tmap(&args.tmap_b, pl.b, pl.b_major, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, 32, BN / CG, BK,
                            &args.b_batch_mul, why, sizeof(why))) {
        set_error("tensor map: %s", why);
        return TTB_EUNSUPPORTED;
    }
    {
        // C as a "K-major operand": inner dim = columns (unit stride), outer = rows.
        const OperandView cv{p.c, p.N, p.M, p.B, p.c_si, p.c_sj, p.c_sb};
        char cw[128] = "";
        if (p.c_sb != 0 && classify_operand(cv, 4, cw, sizeof(cw)) == kMajorK &&
            encode_operand_tmap(&args.tmap_c, cv, kMajorK, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, 32, 32, 32,
                                &args.c_batch_mul, cw, sizeof(cw)) == 0)
            args.c_tma = 1;
    }
    args.c = static_cast<int32_t *>(p.c);
    args.c_sb = p.c_sb;
    args.c_si = p.c_si;
    args.c_sj = p.c_sj;
    args.d = static_cast<const int32_t *>(p.d);
    args.d_sb = p.d_sb;
    args.d_si = p.d_si;
    args.d_sj = p.d_sj;
    args.N = static_cast<int>(p.N);
    args.M = static_cast<int>(p.M);
    args.K = static_cast<int>(p.K);
    args.B = static_cast<int>(p.B);
    args.a_mn_major = pl.a_major == kMajorMN;
    args.b_mn_major = pl.b_major == kMajorMN;
    args.tiles_m = static_cast<int>((p.N + BM * CG - 1) / (BM * CG));
    args.tiles_n = static_cast<int>((p.M + BN - 1) / BN);
    args.total_tiles = args.tiles_m * args.tiles_n * args.B;
    args.dbg = dbg;
    int rc = device_status_ptr(p.device, &args.status);
    if (rc != TTB_OK) return rc;
    auto kernel = gemm_i32_limb_kernel<CG>;
    static bool attr_set[64] = {false};
    if (!attr_set[p.device & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(smem)");
        attr_set[p.device & 63] = true;
    }
    int sms = 148;
    sm_count(p.device, &sms);
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = p.stream;
    cudaLaunchAttribute attr[1];
    int units = sms / CG;  // CTAs, or CTA pairs, resident at once
    if (CG == 2) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        static int max_clusters[64] = {0};
        if (max_clusters[p.device & 63] == 0) {
            cfg.gridDim = dim3(static_cast<unsigned>(2 * units));
            int n = 0;
            cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
            if (e != cudaSuccess) return cuda_fail(e, "cudaOccupancyMaxActiveClusters");
            if (n < 1) {
                set_error("no CTA pair of the i32 tcgen05 kernel fits on device %d", p.device);
                return TTB_ECUDA;
            }
            max_clusters[p.device & 63] = n;
        }
        if (units > max_clusters[p.device & 63]) units = max_clusters[p.device & 63];
    }
    if (units > args.total_tiles) units = args.total_tiles;
    cfg.gridDim = dim3(static_cast<unsigned>(units * CG));
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args);
    if (e != cudaSuccess) return cuda_fail(e, "gemm_i32_limb_kernel launch");
    note_launch(TTB_VARIANT_TCGEN05_I8LIMB, 1);
    return TTB_OK;
}

}  // namespace

int launch_i32_tcgen05(const Problem &p, int two_cta, int dbg) {
    I8Plan pl;
    char why[200] = "";
    if (!plan(p, &pl, why, sizeof(why))) {
        set_error("tcgen05 i32 kernel cannot take these views: %s", why);
        return TTB_EUNSUPPORTED;
    }
    // CTA pairs (256 x 128 tiles) move a quarter less through shared memory per product; they
    // need more than one 128-row tile of rows and enough pair tiles to occupy the GPU.
    int sms = 148;
    sm_count(p.device, &sms);
    const long long pair_tiles = ((p.N + 255) / 256) * ((p.M + BN - 1) / BN) * p.B;
    const bool pair = two_cta < 0 ? (p.N > 128 && pair_tiles >= sms / 4) : two_cta != 0;
    return pair ? launch_i32_cg<2>(p, pl, dbg) : launch_i32_cg<1>(p, pl, dbg);
}

}  // namespace ttb
