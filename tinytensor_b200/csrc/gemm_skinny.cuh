// gemm_skinny.cuh -- bandwidth-bound products with one tiny dim (included by gemm_simt.cu).
//
// A classifier head or its gradient (tinytensor's MNIST example: H[4096,1024] . W2^T[1024,10],
// dC[4096,10] . W2[10,1024], H^T[1024,4096] . dC[4096,10]) has 5-20 flops per byte: what counts
// is reading the large operand once, coalesced, with the tiny one kept on chip.  The register-
// tiled kernel spends its time on tile bookkeeping there (16-22 us for 17 MB); these three
// kernels stream:
//   row_dot      M <= 16, lhs rows contiguous along K: a warp per output row, lanes walk K,
//                rhs transposed in shared memory, M warp-reduced sums per row;
//   col_stream   M <= 16, lhs contiguous along its rows (a transposed view): a thread per
//                output row, the K range of the CTA's split streamed with the rhs slice
//                broadcast from shared memory; partial sums per split, fixed-order reduce;
//   outer        K <= 16: a thread per four output columns, lhs row and rhs rows from L1.
// All dtypes; integer sums wrap as everywhere else (unsigned accumulators); the fused addend /
// relu is applied by whoever writes the final value.
#pragma once

namespace skinny {

constexpr int kMaxSmall = 16;  // largest M (row_dot, col_stream) or K (outer)

// Four elements moved as one when the view allows (16 bytes at most per access).
template <typename T>
struct alignas(sizeof(T) * 4 > 16 ? 16 : sizeof(T) * 4) Vec4T {
    T v[4];
};

// ---- row_dot: out[b,n,j] = sum_k A[b,n,k] B[b,k,j], a_sk == 1.  MC = m_cols rounded up to 4.
// grid (CTAs striding over rows, B); block 1024 = 32 warps, a warp per row at a time; dynamic
// shared memory m_cols x K accumulator words (the rhs transposed, staged once per CTA).
template <typename T, int MC>
__global__ void __launch_bounds__(1024) row_dot_kernel(SimtArgs p, int m_cols) {
    using A = typename AccOf<T>::type;
    extern __shared__ __align__(16) unsigned char skinny_smem[];
    A *bs = reinterpret_cast<A *>(skinny_smem);  // [j][k]
    const long long batch = blockIdx.y;
    const T *__restrict__ a = static_cast<const T *>(p.a) + batch * p.a_sb;
    const T *__restrict__ b = static_cast<const T *>(p.b) + batch * p.b_sb;
    T *__restrict__ c = static_cast<T *>(p.c) + batch * p.c_sb;
    const int K = static_cast<int>(p.K);  // m_cols * K words fit shared memory, so K fits an int
    const bool k_fast = p.b_sk <= p.b_sj;  // walk the rhs along its smaller stride
    for (int idx = threadIdx.x; idx < K * m_cols; idx += 1024) {
        const int k = k_fast ? idx % K : idx / m_cols;
        const int j = k_fast ? idx / K : idx % m_cols;
        bs[j * K + k] = widen<T>(b[k * p.b_sk + j * p.b_sj]);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (long long n = static_cast<long long>(blockIdx.x) * 32 + warp; n < p.N; n += static_cast<long long>(gridDim.x) * 32) {
        const T *__restrict__ row = a + n * p.a_si;
        A acc[MC];
#pragma unroll
        for (int j = 0; j < MC; ++j) acc[j] = A(0);
        for (int k0 = 0; k0 < K; k0 += 128) {
            A av[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int k = k0 + u * 32 + lane;
                av[u] = k < K ? widen<T>(row[k]) : A(0);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int k = k0 + u * 32 + lane;
                if (k < K) {
#pragma unroll
                    for (int j = 0; j < MC; ++j)
                        if (j < m_cols) acc[j] = mad<A>(av[u], bs[j * K + k], acc[j]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < MC; ++j) {
            if (j < m_cols) {
                A v = acc[j];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v = v + __shfl_xor_sync(0xFFFFFFFFu, v, off);
                if (lane == j) c[n * p.c_si + j * p.c_sj] = finish<T>(v, p.ep, batch, n, j);
            }
        }
    }
}

// ---- col_stream: out[b,i,j] (+)= sum over this split's k of A[b,i,k] B[b,k,j], a_si == 1.
// grid (row blocks of 128, splits, B); block 128.  With splits > 1 the destination is the split's
// slab of the scratch ([split][B][N][M], contiguous) and the epilogue is left to the reduce.
template <typename T, int MC>
__global__ void __launch_bounds__(128) col_stream_kernel(SimtArgs p, int m_cols) {
    using A = typename AccOf<T>::type;
    constexpr int KC = 128;  // rhs rows staged at a time
    __shared__ __align__(16) A bs[KC][MC];
    const long long batch = blockIdx.z;
    const int split = blockIdx.y;
    const long long k_begin = static_cast<long long>(split) * p.k_per_split;
    const long long k_end = (k_begin + p.k_per_split < p.K) ? k_begin + p.k_per_split : p.K;
    const T *__restrict__ a = static_cast<const T *>(p.a) + batch * p.a_sb;
    const T *__restrict__ b = static_cast<const T *>(p.b) + batch * p.b_sb;
    T *__restrict__ c = static_cast<T *>(p.c) + batch * p.c_sb + static_cast<long long>(split) * p.c_ss;
    const long long i = static_cast<long long>(blockIdx.x) * 128 + threadIdx.x;
    A acc[MC];
#pragma unroll
    for (int j = 0; j < MC; ++j) acc[j] = A(0);
    for (long long k0 = k_begin; k0 < k_end; k0 += KC) {
        const int kc = static_cast<int>(k_end - k0 < KC ? k_end - k0 : KC);
        __syncthreads();
        for (int idx = threadIdx.x; idx < kc * MC; idx += 128) {
            const int kk = idx / MC, j = idx % MC;  // columns past m_cols are zero: no predicate below
            bs[kk][j] = j < m_cols ? widen<T>(b[(k0 + kk) * p.b_sk + j * p.b_sj]) : A(0);
        }
        __syncthreads();
        if (i < p.N) {
            const T *__restrict__ col = a + i + k0 * p.a_sk;
#pragma unroll 4
            for (int kk = 0; kk < kc; ++kk) {
                const A av = widen<T>(col[kk * p.a_sk]);
#pragma unroll
                for (int j4 = 0; j4 < MC; j4 += 4) {
                    const Vec4T<A> bv = *reinterpret_cast<const Vec4T<A> *>(&bs[kk][j4]);  // broadcast read
#pragma unroll
                    for (int u = 0; u < 4; ++u) acc[j4 + u] = mad<A>(av, bv.v[u], acc[j4 + u]);
                }
            }
        }
    }
    if (i < p.N) {
#pragma unroll
        for (int j = 0; j < MC; ++j)
            if (j < m_cols) c[i * p.c_si + j * p.c_sj] = finish<T>(acc[j], p.ep, batch, i, j);
    }
}

// ---- outer: out[b,n,j..j+3] = sum_{k < K <= 16} A[b,n,k] B[b,k,j..j+3].  One thread per four
// columns; grid (rows, column-group blocks, B) so that no index needs a division.
template <typename T>
__global__ void __launch_bounds__(256) outer_kernel(SimtArgs p, int k_dim, int b_vec, int c_vec) {
    using A = typename AccOf<T>::type;
    const long long n = blockIdx.x, batch = blockIdx.z;
    const long long g = static_cast<long long>(blockIdx.y) * 256 + threadIdx.x;
    if (g * 4 >= p.M) return;
    {
        const T *__restrict__ a = static_cast<const T *>(p.a) + batch * p.a_sb + n * p.a_si;
        const T *__restrict__ b = static_cast<const T *>(p.b) + batch * p.b_sb;
        T *__restrict__ c = static_cast<T *>(p.c) + batch * p.c_sb + n * p.c_si;
        const bool full = g * 4 + 4 <= p.M;
        A acc[4] = {A(0), A(0), A(0), A(0)};
#pragma unroll
        for (int k = 0; k < kMaxSmall; ++k) {
            if (k < k_dim) {
                const A av = widen<T>(a[k * p.a_sk]);
                if (b_vec && full) {
                    const Vec4T<T> bv = *reinterpret_cast<const Vec4T<T> *>(b + k * p.b_sk + g * 4);
#pragma unroll
                    for (int u = 0; u < 4; ++u) acc[u] = mad<A>(av, widen<T>(bv.v[u]), acc[u]);
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const long long j = g * 4 + u;
                        if (j < p.M) acc[u] = mad<A>(av, widen<T>(b[k * p.b_sk + j * p.b_sj]), acc[u]);
                    }
                }
            }
        }
        if (c_vec && full) {
            Vec4T<T> out;
#pragma unroll
            for (int u = 0; u < 4; ++u) out.v[u] = finish<T>(acc[u], p.ep, batch, n, g * 4 + u);
            *reinterpret_cast<Vec4T<T> *>(c + g * 4) = out;
        } else {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long j = g * 4 + u;
                if (j < p.M) c[j * p.c_sj] = finish<T>(acc[u], p.ep, batch, n, j);
            }
        }
    }
}

}  // namespace skinny
