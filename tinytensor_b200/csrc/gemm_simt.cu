// gemm_simt.cu -- CUDA-core batched GEMM with warp-level register tiling.
//
// Takes every dtype tinytensor's matmul accepts (u8, i16, i32, i64, f32, f64) and
// every view (arbitrary element strides, including 0 and permuted dims), so it is
// both the integer path and the universal path for operands the TMA-fed
// tensor-core kernels cannot take.  Replaces the reference's 64x64x8 kernel
// (tinytensor/tensor/backend/cuda/kernel/matmul.cuh:27-151), which needs
// contiguous operands.
//
// Integer semantics: the reference accumulates in T and therefore wraps mod 2^w
// (kernel/matmul.cuh:74,131; CPU simd.h:99-128).  Here narrow integers are
// widened to an unsigned 32-bit accumulator and truncated once at the store;
// that is bit-identical because truncation is a ring homomorphism.
//
// Layout of one CTA: a BM x BN output tile, BK-deep slices of lhs and rhs
// staged in shared memory (lhs transposed so both operands are read as
// vectors), double-buffered with register prefetch; each thread owns a
// TM x TN register tile split in two halves per dim so that shared-memory reads
// are conflict-free and global stores coalesce.
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace ttb {
namespace {

template <typename T>
struct AccOf {
    using type = T;
};
template <>
struct AccOf<uint8_t> {
    using type = uint32_t;
};
template <>
struct AccOf<int16_t> {
    using type = uint32_t;
};
template <>
struct AccOf<int32_t> {
    using type = uint32_t;
};
template <>
struct AccOf<int64_t> {
    using type = unsigned long long;
};

template <typename T>
__device__ __forceinline__ typename AccOf<T>::type widen(T v) {
    using A = typename AccOf<T>::type;
    if constexpr (std::is_same_v<T, int16_t>) {
        return static_cast<A>(static_cast<int32_t>(v));  // sign-extend, then reinterpret
    } else {
        return static_cast<A>(v);
    }
}
template <typename T>
__device__ __forceinline__ T narrow(typename AccOf<T>::type v) {
    return static_cast<T>(v);  // modular for integers, identity for floats
}

template <typename A>
__device__ __forceinline__ A mad(A a, A b, A c) {
    if constexpr (std::is_same_v<A, float>) {
        return fmaf(a, b, c);
    } else if constexpr (std::is_same_v<A, double>) {
        return fma(a, b, c);
    } else {
        return a * b + c;  // unsigned: wraps, no UB
    }
}

template <typename A, int W>
struct alignas(sizeof(A) * W <= 16 ? sizeof(A) * W : 16) Pack {
    A v[W];
};

struct SimtArgs {
    const void *a;
    const void *b;
    void *c;
    long long N, K, M;
    long long a_sb, a_si, a_sk;
    long long b_sb, b_sk, b_sj;
    long long c_sb, c_si, c_sj;
    int splits;          // K is cut into `splits` ranges of k_per_split (grid.z = B * splits)
    long long k_per_split;
    long long c_ss;      // stride between split partials in c (split-K only)
    Epilogue ep;         // applied by whoever writes the final value (not to split partials)
};

// acc (+ addend) -> T, then the activation.  Integer sums wrap: widening the addend and
// narrowing once equals adding in T.  ReLU is std::max(x, 0): NaN and -0.0 pass through.
template <typename T, typename A>
__device__ __forceinline__ T finish(A acc, const Epilogue &ep, long long b, long long i, long long j) {
    if (ep.d) acc = acc + widen<T>(static_cast<const T *>(ep.d)[b * ep.d_sb + i * ep.d_si + j * ep.d_sj]);
    T r = narrow<T>(acc);
    if constexpr (std::is_floating_point_v<T>) {
        if (ep.act == TTB_ACT_RELU) r = r < T(0) ? T(0) : r;
    }
    return r;
}

template <typename T, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN)) simt_gemm_kernel(SimtArgs p) {
    using A = typename AccOf<T>::type;
    constexpr int NT = (BM / TM) * (BN / TN);
    constexpr int TX = BN / TN;
    constexpr int HM = TM / 2 > 0 ? TM / 2 : 1;  // half-tile extents
    constexpr int HN = TN / 2 > 0 ? TN / 2 : 1;
    constexpr int PM = TM >= 2 ? 2 : 1;          // number of halves per dim
    constexpr int PN = TN >= 2 ? 2 : 1;
    constexpr int PAD = 16 / sizeof(A);
    constexpr int A_ELEMS = (BM * BK + NT - 1) / NT;
    constexpr int B_ELEMS = (BK * BN + NT - 1) / NT;

    __shared__ __align__(16) A As[2][BK][BM + PAD];
    __shared__ __align__(16) A Bs[2][BK][BN];

    const int tid = threadIdx.x;
    const int tx = tid % TX;
    const int ty = tid / TX;
    const long long m0 = static_cast<long long>(blockIdx.y) * BM;
    const long long n0 = static_cast<long long>(blockIdx.x) * BN;
    const long long batch = blockIdx.z / p.splits;
    const int split = blockIdx.z % p.splits;
    const long long k_begin = static_cast<long long>(split) * p.k_per_split;
    const long long k_end = (k_begin + p.k_per_split < p.K) ? k_begin + p.k_per_split : p.K;

    const T *__restrict__ a = static_cast<const T *>(p.a) + batch * p.a_sb;
    const T *__restrict__ b = static_cast<const T *>(p.b) + batch * p.b_sb;
    T *__restrict__ c = static_cast<T *>(p.c) + batch * p.c_sb + static_cast<long long>(split) * p.c_ss;

    // Which dim the loading threads walk fastest: the one with the smaller
    // stride, so that neighbouring threads touch neighbouring addresses.
    const bool a_k_fast = p.a_sk <= p.a_si;
    const bool b_j_fast = p.b_sj <= p.b_sk;

    A ra[A_ELEMS];
    A rb[B_ELEMS];

    auto load_global = [&](long long k0) {
#pragma unroll
        for (int l = 0; l < A_ELEMS; ++l) {
            const int idx = tid + l * NT;
            int r, kk;
            if (a_k_fast) {
                kk = idx % BK;
                r = idx / BK;
            } else {
                r = idx % BM;
                kk = idx / BM;
            }
            const long long gi = m0 + r;
            const long long gk = k0 + kk;
            A v = A(0);
            if (idx < BM * BK && gi < p.N && gk < k_end) v = widen<T>(a[gi * p.a_si + gk * p.a_sk]);
            ra[l] = v;
        }
#pragma unroll
        for (int l = 0; l < B_ELEMS; ++l) {
            const int idx = tid + l * NT;
            int j, kk;
            if (b_j_fast) {
                j = idx % BN;
                kk = idx / BN;
            } else {
                kk = idx % BK;
                j = idx / BK;
            }
            const long long gj = n0 + j;
            const long long gk = k0 + kk;
            A v = A(0);
            if (idx < BK * BN && gj < p.M && gk < k_end) v = widen<T>(b[gk * p.b_sk + gj * p.b_sj]);
            rb[l] = v;
        }
    };
    auto store_shared = [&](int buf) {
#pragma unroll
        for (int l = 0; l < A_ELEMS; ++l) {
            const int idx = tid + l * NT;
            int r, kk;
            if (a_k_fast) {
                kk = idx % BK;
                r = idx / BK;
            } else {
                r = idx % BM;
                kk = idx / BM;
            }
            if (idx < BM * BK) As[buf][kk][r] = ra[l];
        }
#pragma unroll
        for (int l = 0; l < B_ELEMS; ++l) {
            const int idx = tid + l * NT;
            int j, kk;
            if (b_j_fast) {
                j = idx % BN;
                kk = idx / BN;
            } else {
                kk = idx % BK;
                j = idx / BK;
            }
            if (idx < BK * BN) Bs[buf][kk][j] = rb[l];
        }
    };

    A acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = A(0);

    int buf = 0;
    if (k_begin < k_end) {
        load_global(k_begin);
        store_shared(0);
    }
    __syncthreads();

    for (long long k0 = k_begin; k0 < k_end; k0 += BK) {
        const bool has_next = k0 + BK < k_end;
        if (has_next) load_global(k0 + BK);

#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            A av[TM];
            A bv[TN];
#pragma unroll
            for (int h = 0; h < PM; ++h) {
                const Pack<A, HM> pa =
                    *reinterpret_cast<const Pack<A, HM> *>(&As[buf][kk][h * (BM / 2) + ty * HM]);
#pragma unroll
                for (int i = 0; i < HM; ++i) av[h * HM + i] = pa.v[i];
            }
#pragma unroll
            for (int h = 0; h < PN; ++h) {
                const Pack<A, HN> pb =
                    *reinterpret_cast<const Pack<A, HN> *>(&Bs[buf][kk][h * (BN / 2) + tx * HN]);
#pragma unroll
                for (int j = 0; j < HN; ++j) bv[h * HN + j] = pb.v[j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = mad<A>(av[i], bv[j], acc[i][j]);
        }

        if (has_next) store_shared(buf ^ 1);
        __syncthreads();
        buf ^= 1;
    }

    // Store.  Row/column of register (i, j): half h = i / HM, etc.
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const long long gi = m0 + (i / HM) * (BM / 2) + ty * HM + (i % HM);
        if (gi >= p.N) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const long long gj = n0 + (j / HN) * (BN / 2) + tx * HN + (j % HN);
            if (gj < p.M) c[gi * p.c_si + gj * p.c_sj] = finish<T>(acc[i][j], p.ep, batch, gi, gj);
        }
    }
}

// Sums `splits` partials (each [B,N,M] contiguous, split-major) into the strided output.
template <typename T>
__global__ void splitk_reduce_kernel(const T *__restrict__ part, T *__restrict__ c, long long B, long long N,
                                     long long M, int splits, long long c_sb, long long c_si, long long c_sj,
                                     Epilogue ep) {
    using A = typename AccOf<T>::type;
    const long long total = B * N * M;
    for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        A s = A(0);
        for (int sp = 0; sp < splits; ++sp) s = s + widen<T>(part[sp * total + idx]);
        const long long bb = idx / (N * M);
        const long long r = (idx / M) % N;
        const long long col = idx % M;
        c[bb * c_sb + r * c_si + col * c_sj] = finish<T>(s, ep, bb, r, col);
    }
}

template <typename T, int BM, int BN, int BK, int TM, int TN>
int launch_tile(const Problem &p, int splits, void *scratch) {
    SimtArgs a{};
    a.a = p.a;
    a.b = p.b;
    a.N = p.N;
    a.K = p.K;
    a.M = p.M;
    a.a_sb = p.a_sb;
    a.a_si = p.a_si;
    a.a_sk = p.a_sk;
    a.b_sb = p.b_sb;
    a.b_sk = p.b_sk;
    a.b_sj = p.b_sj;
    a.splits = splits;
    if (splits > 1) {
        const long long kb = (p.K + BK - 1) / BK;
        a.k_per_split = ((kb + splits - 1) / splits) * BK;
        a.c = scratch;
        a.c_sb = p.N * p.M;
        a.c_si = p.M;
        a.c_sj = 1;
        a.c_ss = p.B * p.N * p.M;
        a.ep = Epilogue{nullptr, 0, 0, 0, 0};
    } else {
        a.k_per_split = p.K;
        a.c = p.c;
        a.c_sb = p.c_sb;
        a.c_si = p.c_si;
        a.c_sj = p.c_sj;
        a.c_ss = 0;
        a.ep = epilogue_of(p);
    }
    const long long gx = (p.M + BN - 1) / BN, gy = (p.N + BM - 1) / BM, gz = p.B * splits;
    if (gy > 65535 || gz > 65535) {
        set_error("simt kernel: grid (%lld,%lld,%lld) exceeds launch limits", gx, gy, gz);
        return TTB_ELIMIT;
    }
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(gz));
    simt_gemm_kernel<T, BM, BN, BK, TM, TN><<<grid, (BM / TM) * (BN / TN), 0, p.stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "simt_gemm_kernel launch");
    if (splits > 1) {
        const long long total = p.B * p.N * p.M;
        const int blocks = static_cast<int>((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
        splitk_reduce_kernel<T><<<blocks, 256, 0, p.stream>>>(static_cast<const T *>(scratch),
                                                              static_cast<T *>(p.c), p.B, p.N, p.M, splits,
                                                              p.c_sb, p.c_si, p.c_sj, epilogue_of(p));
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "splitk_reduce_kernel launch");
    }
    return TTB_OK;
}

#include "gemm_skinny.cuh"

}  // namespace

int workspace_get(int device, cudaStream_t stream, size_t bytes, void **out);

namespace {

// out^T = rhs^T . lhs^T: the same product with the roles of the two operands (and of the
// output's dims) exchanged, so that a tiny N is handled by the kernels written for a tiny M.
Problem transposed(const Problem &p) {
    Problem t = p;
    t.a = p.b;
    t.a_sb = p.b_sb;
    t.a_si = p.b_sj;
    t.a_sk = p.b_sk;
    t.b = p.a;
    t.b_sb = p.a_sb;
    t.b_sk = p.a_sk;
    t.b_sj = p.a_si;
    t.N = p.M;
    t.M = p.N;
    t.c_si = p.c_sj;
    t.c_sj = p.c_si;
    t.d_si = p.d_sj;
    t.d_sj = p.d_si;
    return t;
}

template <typename U>
bool vec4_ok(const void *base, long long s_inner, long long s_a, long long s_b) {
    return s_inner == 1 && (s_a & 3) == 0 && (s_b & 3) == 0 &&
           reinterpret_cast<uintptr_t>(base) % alignof(skinny::Vec4T<U>) == 0;
}

// Streams a product with one tiny dim (see gemm_skinny.cuh).  Returns TTB_OK when it launched,
// 1 when the shape or the strides are not for these kernels, or a negative status.
template <typename T>
int launch_skinny_typed(const Problem &p0, int sms) {
    using A = typename AccOf<T>::type;
    Problem p = p0;
    if (p.N <= skinny::kMaxSmall && p.M > skinny::kMaxSmall && p.K > skinny::kMaxSmall) p = transposed(p0);
    if (p.B > 65535) return 1;
    SimtArgs a{};
    a.a = p.a;
    a.b = p.b;
    a.c = p.c;
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
    a.splits = 1;
    a.k_per_split = p.K;
    a.c_ss = 0;
    a.ep = epilogue_of(p);
    cudaError_t e;
    if (p.K <= skinny::kMaxSmall && p.M >= 32) {
        const long long gblocks = ((p.M + 3) / 4 + 255) / 256;
        if (p.N > 0x7FFFFFFFLL || gblocks > 65535) return 1;
        dim3 grid(static_cast<unsigned>(p.N), static_cast<unsigned>(gblocks), static_cast<unsigned>(p.B));
        skinny::outer_kernel<T><<<grid, 256, 0, p.stream>>>(a, static_cast<int>(p.K),
                                                            vec4_ok<T>(p.b, p.b_sj, p.b_sk, p.b_sb) ? 1 : 0,
                                                            vec4_ok<T>(p.c, p.c_sj, p.c_si, p.c_sb) ? 1 : 0);
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "outer_kernel launch");
        note_launch(TTB_VARIANT_SIMT_SKINNY, 1);
        return TTB_OK;
    }
    if (p.M > skinny::kMaxSmall || p.K < 64) return 1;
    const size_t bs_bytes = static_cast<size_t>(p.M) * p.K * sizeof(A);
    const int mc = static_cast<int>((p.M + 3) / 4 * 4);
    if (p.a_sk == 1 && p.N >= 32 && bs_bytes <= 96 * 1024) {
        auto kernel = mc == 4 ? skinny::row_dot_kernel<T, 4>
                      : mc == 8 ? skinny::row_dot_kernel<T, 8>
                      : mc == 12 ? skinny::row_dot_kernel<T, 12>
                                 : skinny::row_dot_kernel<T, 16>;
        if (bs_bytes > 48 * 1024) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
            if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(row_dot smem)");
        }
        long long groups = (p.N + 31) / 32;
        const long long cap = (2LL * sms + p.B - 1) / p.B;  // about two CTAs of 32 warps per SM
        if (groups > cap) groups = cap;
        dim3 grid(static_cast<unsigned>(groups), static_cast<unsigned>(p.B));
        kernel<<<grid, 1024, bs_bytes, p.stream>>>(a, static_cast<int>(p.M));
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "row_dot_kernel launch");
        note_launch(TTB_VARIANT_SIMT_SKINNY, 1);
        return TTB_OK;
    }
    if (p.a_si == 1 && p.N >= 128) {
        const long long row_blocks = (p.N + 127) / 128;
        long long splits = (2LL * sms + row_blocks * p.B - 1) / (row_blocks * p.B);
        if (splits > p.K / 64) splits = p.K / 64;
        if (splits > 65535) splits = 65535;
        if (splits < 1) splits = 1;
        void *scratch = nullptr;
        if (splits > 1) {
            int rc = workspace_get(p.device, p.stream, static_cast<size_t>(splits) * p.B * p.N * p.M * sizeof(T), &scratch);
            if (rc != TTB_OK) return rc;
            a.splits = static_cast<int>(splits);
            a.k_per_split = (p.K + splits - 1) / splits;
            a.c = scratch;
            a.c_sb = p.N * p.M;
            a.c_si = p.M;
            a.c_sj = 1;
            a.c_ss = p.B * p.N * p.M;
            a.ep = Epilogue{nullptr, 0, 0, 0, 0};
        }
        if (row_blocks > 0x7FFFFFFFLL) return 1;
        dim3 grid(static_cast<unsigned>(row_blocks), static_cast<unsigned>(splits), static_cast<unsigned>(p.B));
        auto kernel = mc == 4 ? skinny::col_stream_kernel<T, 4>
                      : mc == 8 ? skinny::col_stream_kernel<T, 8>
                      : mc == 12 ? skinny::col_stream_kernel<T, 12>
                                 : skinny::col_stream_kernel<T, 16>;
        kernel<<<grid, 128, 0, p.stream>>>(a, static_cast<int>(p.M));
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "col_stream_kernel launch");
        if (splits > 1) {
            const long long total = p.B * p.N * p.M;
            const int blocks = static_cast<int>((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
            splitk_reduce_kernel<T><<<blocks, 256, 0, p.stream>>>(static_cast<const T *>(scratch), static_cast<T *>(p.c),
                                                                  p.B, p.N, p.M, static_cast<int>(splits), p.c_sb,
                                                                  p.c_si, p.c_sj, epilogue_of(p));
            e = cudaGetLastError();
            if (e != cudaSuccess) return cuda_fail(e, "splitk_reduce_kernel launch");
        }
        note_launch(TTB_VARIANT_SIMT_SKINNY, splits > 1 ? 2 : 1);
        return TTB_OK;
    }
    return 1;
}

}  // namespace

// Chooses a tile from the output shape, and a K split when the output alone
// cannot fill the GPU.
template <typename T>
int launch_simt_typed(const Problem &p, bool allow_splitk, bool allow_skinny) {
    int sms = 148;
    sm_count(p.device, &sms);
    if (allow_skinny) {
        const int rc = launch_skinny_typed<T>(p, sms);
        if (rc <= 0) return rc;  // launched, or failed; 1 = not a shape for the streaming kernels
    }
    constexpr int BKs = sizeof(T) >= 8 ? 8 : 16;
    auto tiles = [&](long long bm, long long bn) {
        return ((p.N + bm - 1) / bm) * ((p.M + bn - 1) / bn) * p.B;
    };
    enum { L, MID, SKN, SKM, S } shape;
    if (p.M <= 16 && p.N > 16)
        shape = SKN;
    else if (p.N <= 16 && p.M > 16)
        shape = SKM;
    else if (tiles(128, 128) >= sms)
        shape = L;
    else if (tiles(64, 64) >= sms || (p.N > 32 && p.M > 32))
        shape = MID;
    else
        shape = S;

    long long ntiles;
    int bk = BKs;
    switch (shape) {
        case L: ntiles = tiles(128, 128); break;
        case MID: ntiles = tiles(64, 64); break;
        case SKN: ntiles = tiles(128, 16); break;
        case SKM: ntiles = tiles(16, 128); break;
        default: ntiles = tiles(32, 32); break;
    }
    int splits = 1;
    void *scratch = nullptr;
    if (allow_splitk && ntiles < sms && p.K >= 512) {
        long long want = (2LL * sms + ntiles - 1) / ntiles;
        long long max_by_k = p.K / (8LL * bk);
        if (want > max_by_k) want = max_by_k;
        if (want > 64) want = 64;
        if (want >= 2) {
            splits = static_cast<int>(want);
            size_t bytes = static_cast<size_t>(splits) * p.B * p.N * p.M * sizeof(T);
            int rc = workspace_get(p.device, p.stream, bytes, &scratch);
            if (rc != TTB_OK) return rc;
        }
    }
    int rc;
    switch (shape) {
        case L: rc = launch_tile<T, 128, 128, BKs, 8, 8>(p, splits, scratch); break;
        case MID: rc = launch_tile<T, 64, 64, BKs, 4, 4>(p, splits, scratch); break;
        case SKN: rc = launch_tile<T, 128, 16, BKs, 4, 2>(p, splits, scratch); break;
        case SKM: rc = launch_tile<T, 16, 128, BKs, 2, 4>(p, splits, scratch); break;
        default: rc = launch_tile<T, 32, 32, BKs, 2, 2>(p, splits, scratch); break;
    }
    if (rc == TTB_OK) note_launch(splits > 1 ? TTB_VARIANT_SIMT_SPLITK : TTB_VARIANT_SIMT, splits > 1 ? 2 : 1);
    return rc;
}

int launch_simt(const Problem &p, bool allow_splitk, bool allow_skinny) {
    switch (p.dtype) {
        case TTB_U8: return launch_simt_typed<uint8_t>(p, allow_splitk, allow_skinny);
        case TTB_I16: return launch_simt_typed<int16_t>(p, allow_splitk, allow_skinny);
        case TTB_I32: return launch_simt_typed<int32_t>(p, allow_splitk, allow_skinny);
        case TTB_I64: return launch_simt_typed<int64_t>(p, allow_splitk, allow_skinny);
        case TTB_F32: return launch_simt_typed<float>(p, allow_splitk, allow_skinny);
        case TTB_F64: return launch_simt_typed<double>(p, allow_splitk, allow_skinny);
        default: set_error("unsupported dtype %d", p.dtype); return TTB_EDTYPE;
    }
}

}  // namespace ttb

// ---------------------------------------------------------------------------
// Split-K product with its scratch in a fixed device array (no allocation).
//
// Who needs this: a host program that has handed all device memory to an allocator of
// its own (or runs under a hard memory budget), so that a cudaMalloc from inside this
// library would fail or break the budget; and a latency-sensitive loop that cannot accept
// the device-wide synchronisation cudaMalloc / cudaFree imply.  The ordinary entry points
// grow a cached workspace with cudaMalloc when the K split needs one; this one never
// allocates: the partial sums of the K split live in the array below, which is part of the
// library's device image: a GPU holds it from the moment that image is loaded there (with the
// driver's default lazy loading: this entry point's first call on that GPU) until exit.
namespace ttb {
namespace {

constexpr size_t kStaticScratchBytes = size_t(16) << 20;  // 16 MiB, the documented limit
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address:
// the address has to be asked for, per device, with that device current.
constexpr int kStaticMaxDevices = 64;
void *g_static_scratch_ptr[kStaticMaxDevices] = {nullptr};
int g_static_sms[kStaticMaxDevices] = {0};
std::mutex g_static_mu;

int static_scratch_setup(int device, void **ptr, int *sms) {
    if (device < 0 || device >= kStaticMaxDevices) {
        set_error("device id %d out of range", device);
        return TTB_EDEVICE;
    }
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (g_static_scratch_ptr[device] == nullptr) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        int n = 0;
        e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
        g_static_scratch_ptr[device] = p;
        g_static_sms[device] = n;
    }
    *ptr = g_static_scratch_ptr[device];
    *sms = g_static_sms[device];
    return TTB_OK;
}

template <typename T>
int launch_static_scratch_typed(const Problem &p, void *scratch, int sms) {
    constexpr int BKs = sizeof(T) >= 8 ? 8 : 16;
    const size_t per_split = static_cast<size_t>(p.B) * p.N * p.M * sizeof(T);
    if (per_split == 0 || per_split * 2 > kStaticScratchBytes) {
        set_error("result of %lld x %lld x %lld elements needs %zu bytes of scratch per K split; two splits do "
                  "not fit the fixed %zu-byte scratch array of the no-allocation entry point",
                  static_cast<long long>(p.B), static_cast<long long>(p.N), static_cast<long long>(p.M), per_split,
                  kStaticScratchBytes);
        return TTB_ELIMIT;
    }
    // Tile by output shape, as the ordinary SIMT dispatch does.
    enum { MID, SKN, SKM, S } shape;
    long long bm, bn;
    if (p.M <= 16 && p.N > 16) {
        shape = SKN; bm = 128; bn = 16;
    } else if (p.N <= 16 && p.M > 16) {
        shape = SKM; bm = 16; bn = 128;
    } else if (p.N > 64 && p.M > 64) {
        shape = MID; bm = 64; bn = 64;
    } else {
        shape = S; bm = 32; bn = 32;
    }
    const long long ntiles = ((p.N + bm - 1) / bm) * ((p.M + bn - 1) / bn) * p.B;
    // As many K splits as fill the GPU twice over, at least two (this variant always goes
    // through the scratch), each at least 8 K-blocks deep when K allows, and no more than
    // the scratch array holds.
    long long splits = (2LL * sms + ntiles - 1) / ntiles;
    const long long by_k = p.K / (8LL * BKs);
    if (splits > by_k) splits = by_k;
    if (splits > 64) splits = 64;
    const long long by_mem = static_cast<long long>(kStaticScratchBytes / per_split);
    if (splits > by_mem) splits = by_mem;
    if (splits < 2) splits = 2;
    int rc;
    switch (shape) {
        case SKN: rc = launch_tile<T, 128, 16, BKs, 4, 2>(p, static_cast<int>(splits), scratch); break;
        case SKM: rc = launch_tile<T, 16, 128, BKs, 2, 4>(p, static_cast<int>(splits), scratch); break;
        case MID: rc = launch_tile<T, 64, 64, BKs, 4, 4>(p, static_cast<int>(splits), scratch); break;
        default: rc = launch_tile<T, 32, 32, BKs, 2, 2>(p, static_cast<int>(splits), scratch); break;
    }
    if (rc == TTB_OK) note_launch(TTB_VARIANT_SIMT_SPLITK, 2);
    return rc;
}

}  // namespace

int resolve_problem(const ttb_view *lhs, const ttb_view *rhs, void *out, int dtype, int device, void *stream,
                    Problem *p);

}  // namespace ttb

extern "C" TTB_API int ttb_batched_matmul_static_scratch(const ttb_view *lhs, const ttb_view *rhs, void *out,
                                                         int dtype, int device_id, void *stream) {
    using namespace ttb;
    Problem p{};
    int rc = resolve_problem(lhs, rhs, out, dtype, device_id, stream, &p);
    if (rc != TTB_OK) return rc;
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceCount");
    if (device_id < 0 || device_id >= ndev) {
        set_error("device id %d out of range (have %d)", device_id, ndev);
        return TTB_EDEVICE;
    }
    // This entry point leaves the calling thread's current device as it found it.
    struct RestoreDevice {
        int prev = -1;
        RestoreDevice() {
            if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        }
        ~RestoreDevice() {
            if (prev >= 0) (void)cudaSetDevice(prev);
        }
    } restore;
    e = cudaSetDevice(device_id);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    void *scratch = nullptr;
    int sms = 0;
    rc = static_scratch_setup(device_id, &scratch, &sms);
    if (rc != TTB_OK) return rc;
    switch (p.dtype) {
        case TTB_U8: return launch_static_scratch_typed<uint8_t>(p, scratch, sms);
        case TTB_I16: return launch_static_scratch_typed<int16_t>(p, scratch, sms);
        case TTB_I32: return launch_static_scratch_typed<int32_t>(p, scratch, sms);
        case TTB_I64: return launch_static_scratch_typed<int64_t>(p, scratch, sms);
        case TTB_F32: return launch_static_scratch_typed<float>(p, scratch, sms);
        case TTB_F64: return launch_static_scratch_typed<double>(p, scratch, sms);
        default: set_error("unsupported dtype %d", p.dtype); return TTB_EDTYPE;
    }
}
