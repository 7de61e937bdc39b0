// gemm_f64_dmma.cu -- f64 batched GEMM on the FP64 tensor-core path (DMMA).
//
// There is no f64 kind of tcgen05.mma; double precision runs on warp-level
// mma.sync (m16n8k4, f64 in / f64 accumulate).  The accumulation is IEEE fp64 FMA
// in the tensor core, so results sit within a few ulp of the reference's fp64 sums
// (tinytensor/tensor/backend/cuda/kernel/matmul.cuh:74,131 accumulate in T).
// Replaces matmul_kernel<double> of the reference.
//
// One CTA: 128 x 64 output tile, 4 warps as 2 (rows) x 2 (columns), each warp a
// 64 x 32 tile = 4 x 4 MMA tiles of 16 x 8, accumulators in registers; two CTAs per SM, so that
// one keeps the DMMA pipe busy while the other sits at its per-K-block barrier.  K runs in
// blocks of 8, staged in shared memory as [k][row] for both operands (lhs is stored
// transposed) with a row pitch of tile+4 doubles, which makes every fragment read
// conflict-free.  Global loads go through registers (prefetch of the next block while
// the current one is multiplied), so any element strides are accepted: f64 views never
// need a copy and never need to satisfy TMA alignment.
#include "common.cuh"

namespace ttb {
namespace {

constexpr int BM = 128, BN = 64, BK = 8;
constexpr int PITCH_A = BM + 4, PITCH_B = BN + 4;
constexpr int THREADS = 128;
constexpr int WM = 64, WN = 32;  // warp tile
constexpr int WARPS_N = BN / WN; // warps side by side along the columns
constexpr int MT = WM / 16, NT = WN / 8;

struct DmmaArgs {
    const double *a;
    const double *b;
    double *c;
    long long N, K, M;
    long long a_sb, a_si, a_sk;
    long long b_sb, b_sk, b_sj;
    long long c_sb, c_si, c_sj;
    Epilogue ep;
};

__device__ __forceinline__ void dmma_m16n8k4(double (&c)[4], double a0, double a1, double b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k4.row.col.f64.f64.f64.f64 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%0, %1, %2, %3};"
        : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
        : "d"(a0), "d"(a1), "d"(b0));
}

__global__ void __launch_bounds__(THREADS, 2) gemm_f64_dmma_kernel(DmmaArgs p) {
    __shared__ __align__(16) double As[2][BK][PITCH_A];
    __shared__ __align__(16) double Bs[2][BK][PITCH_B];

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;  // MMA fragment coordinates
    const int wm = (warp / WARPS_N) * WM;   // warp's row offset in the CTA tile
    const int wn = (warp % WARPS_N) * WN;
    const long long m0 = static_cast<long long>(blockIdx.y) * BM;
    const long long n0 = static_cast<long long>(blockIdx.x) * BN;
    const long long batch = blockIdx.z;
    const double *__restrict__ a = p.a + batch * p.a_sb;
    const double *__restrict__ b = p.b + batch * p.b_sb;
    double *__restrict__ c = p.c + batch * p.c_sb;

    // Loading threads walk the dim with the smaller stride fastest.
    const bool a_k_fast = p.a_sk <= p.a_si;
    const bool b_j_fast = p.b_sj <= p.b_sk;
    constexpr int ELEMS_A = BM * BK / THREADS, ELEMS_B = BN * BK / THREADS;  // 8 and 4 per thread
    double ra[ELEMS_A], rb[ELEMS_B];

    auto load_global = [&](long long k0) {
#pragma unroll
        for (int l = 0; l < ELEMS_A; ++l) {
            const int idx = tid + l * THREADS;
            const int kk = a_k_fast ? idx % BK : idx / BM;
            const int r = a_k_fast ? idx / BK : idx % BM;
            const long long gi = m0 + r, gk = k0 + kk;
            ra[l] = (gi < p.N && gk < p.K) ? a[gi * p.a_si + gk * p.a_sk] : 0.0;
        }
#pragma unroll
        for (int l = 0; l < ELEMS_B; ++l) {
            const int idx = tid + l * THREADS;
            const int kk = b_j_fast ? idx / BN : idx % BK;
            const int j = b_j_fast ? idx % BN : idx / BK;
            const long long gj = n0 + j, gk = k0 + kk;
            rb[l] = (gj < p.M && gk < p.K) ? b[gk * p.b_sk + gj * p.b_sj] : 0.0;
        }
    };
    auto store_shared = [&](int buf) {
#pragma unroll
        for (int l = 0; l < ELEMS_A; ++l) {
            const int idx = tid + l * THREADS;
            const int kk = a_k_fast ? idx % BK : idx / BM;
            const int r = a_k_fast ? idx / BK : idx % BM;
            As[buf][kk][r] = ra[l];
        }
#pragma unroll
        for (int l = 0; l < ELEMS_B; ++l) {
            const int idx = tid + l * THREADS;
            const int kk = b_j_fast ? idx / BN : idx % BK;
            const int j = b_j_fast ? idx % BN : idx / BK;
            Bs[buf][kk][j] = rb[l];
        }
    };

    double acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.0;

    int buf = 0;
    load_global(0);
    store_shared(0);
    __syncthreads();

    for (long long k0 = 0; k0 < p.K; k0 += BK) {
        const bool has_next = k0 + BK < p.K;
        if (has_next) load_global(k0 + BK);
#pragma unroll
        for (int ks = 0; ks < BK; ks += 4) {
            // Fragments of m16n8k4: A(row g / g+8, col t), B(row t, col g).
            double af[MT][2], bf[NT];
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                af[i][0] = As[buf][ks + t][wm + i * 16 + g];
                af[i][1] = As[buf][ks + t][wm + i * 16 + g + 8];
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) bf[j] = Bs[buf][ks + t][wn + j * 8 + g];
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) dmma_m16n8k4(acc[i][j], af[i][0], af[i][1], bf[j]);
        }
        if (has_next) store_shared(buf ^ 1);
        __syncthreads();
        buf ^= 1;
    }

    // C fragment: c0,c1 -> row g, cols 2t,2t+1; c2,c3 -> row g+8.
    const bool vec_ok = p.c_sj == 1 && (p.c_si & 1) == 0 && (p.c_sb & 1) == 0 &&
                        (reinterpret_cast<uintptr_t>(p.c) & 15) == 0;
#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const long long gi = m0 + wm + i * 16 + g + h * 8;
            if (gi >= p.N) continue;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const long long gj = n0 + wn + j * 8 + 2 * t;
                if (gj >= p.M) continue;
                double *dst = c + gi * p.c_si + gj * p.c_sj;
                double v0 = acc[i][j][2 * h], v1 = acc[i][j][2 * h + 1];
                if (p.ep.d) {
                    // addend (bias row / column, or C itself): same thread reads, then writes
                    const double *d = static_cast<const double *>(p.ep.d) + batch * p.ep.d_sb + gi * p.ep.d_si +
                                      gj * p.ep.d_sj;
                    v0 += d[0];
                    if (gj + 1 < p.M) v1 += d[p.ep.d_sj];
                }
                if (p.ep.act == TTB_ACT_RELU) {
                    v0 = v0 < 0.0 ? 0.0 : v0;
                    v1 = v1 < 0.0 ? 0.0 : v1;
                }
                if (vec_ok && gj + 1 < p.M) {
                    *reinterpret_cast<double2 *>(dst) = make_double2(v0, v1);
                } else {
                    dst[0] = v0;
                    if (gj + 1 < p.M) dst[p.c_sj] = v1;
                }
            }
        }
    }
}

// The FP64 tensor-core rate itself: every warp keeps the GEMM kernel's 16 independent 16 x 8
// accumulator tiles in registers and issues m16n8k4 MMAs on register operands, with no memory
// traffic.  What this loop reaches is the ceiling the GEMM kernel's roofline is quoted against.
constexpr int PEAK_THREADS = 256;
__global__ void __launch_bounds__(PEAK_THREADS) dmma_peak_kernel(double *sink, int iters, double a_seed, double b_seed) {
    double acc[MT * NT][4];
#pragma unroll
    for (int j = 0; j < MT * NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.0;
    double a0 = a_seed + threadIdx.x * 1e-9, a1 = a_seed - threadIdx.x * 1e-9, b0 = b_seed;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int j = 0; j < MT * NT; ++j) dmma_m16n8k4(acc[j], a0, a1, b0);
        b0 = -b0;  // keeps the sums bounded and the loop from being folded
    }
    double s = 0.0;
#pragma unroll
    for (int j = 0; j < MT * NT; ++j) s += acc[j][0] + acc[j][1] + acc[j][2] + acc[j][3];
    if (s == 123456.789) sink[0] = s;  // never true: the result only has to look used
}

}  // namespace

// Runs dmma_peak_kernel on `device` (two CTAs of 8 warps per SM) and returns the best of three
// launches in TFLOP/s (2 flops per multiply-add of an m16n8k4 MMA).
int measure_fp64_tensor_peak(int device, double *tflops) {
    int sms = 0;
    int rc = sm_count(device, &sms);
    if (rc != TTB_OK) return rc;
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    double *sink = nullptr;
    e = cudaMalloc(&sink, sizeof(double));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc");
    cudaEvent_t t0, t1;
    cudaEventCreate(&t0);
    cudaEventCreate(&t1);
    const int iters = 1 << 14;
    const int ctas = 2 * sms;
    const double flop = 2.0 * 16 * 8 * 4 * (MT * NT) * static_cast<double>(iters) * (PEAK_THREADS / 32) * ctas;
    double best = 0.0;
    for (int rep = 0; rep < 4 && e == cudaSuccess; ++rep) {  // the first launch is the warm-up
        cudaEventRecord(t0, nullptr);
        dmma_peak_kernel<<<ctas, PEAK_THREADS>>>(sink, iters, 1.0000001, 0.9999999);
        cudaEventRecord(t1, nullptr);
        e = cudaEventSynchronize(t1);
        float ms = 0.f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, t0, t1);
        if (e == cudaSuccess && rep > 0 && ms > 0.f && flop / (ms * 1e9) > best) best = flop / (ms * 1e9);
    }
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    cudaFree(sink);
    if (e != cudaSuccess) return cuda_fail(e, "dmma_peak_kernel");
    note_launch(-1, 4);
    *tflops = best;
    return TTB_OK;
}

bool f64_dmma_eligible(const Problem &p) {
    const long long gy = (p.N + BM - 1) / BM, gz = p.B;
    return p.dtype == TTB_F64 && gy <= 65535 && gz <= 65535;
}

int launch_f64_dmma(const Problem &p) {
    if (!f64_dmma_eligible(p)) {
        set_error("f64 DMMA kernel: grid exceeds launch limits");
        return TTB_ELIMIT;
    }
    DmmaArgs a{};
    a.a = static_cast<const double *>(p.a);
    a.b = static_cast<const double *>(p.b);
    a.c = static_cast<double *>(p.c);
    a.N = p.N;
    a.K = p.K;
    a.M = p.M;
    a.a_sb = p.a_sb;
    a.a_si = p.a_si;
    a.a_sk = p.a_sk;
    a.b_sb = p.b_sb;
    a.b_sk = p.b_sk;
    a.b_sj = p.b_sj;
    a.c_sb = p.c_sb;
    a.c_si = p.c_si;
    a.c_sj = p.c_sj;
    a.ep = epilogue_of(p);
    dim3 grid(static_cast<unsigned>((p.M + BN - 1) / BN), static_cast<unsigned>((p.N + BM - 1) / BM),
              static_cast<unsigned>(p.B));
    gemm_f64_dmma_kernel<<<grid, THREADS, 0, p.stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "gemm_f64_dmma_kernel launch");
    note_launch(TTB_VARIANT_DMMA_F64, 1);
    return TTB_OK;
}

}  // namespace ttb
