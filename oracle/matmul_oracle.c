/* matmul_oracle.c -- CPU restatement of tinytensor's CPU-backend matmul.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product path (the tinytensor_b200
 * package, libttb.so) may link, import or call this file; only tests/, the smoke
 * check and the benchmark's CPU-baseline leg use it, as the checker.
 *
 * Parity is pinned: tests/test_oracle.py checks this file against
 *  (1) the known-answer cases of the reference's own tests/test_matmul.cpp:50-237
 *      (naive wrapping triple loop on (i+j)%100 data, six dtypes, ragged sizes), and
 *  (2) oracle/_ref/libttref.so, the reference's own kernel compiled from its
 *      sources, when that library has been built.
 *
 * What is restated (paths relative to the reference tree):
 *  - tinytensor/tensor/backend/cpu/matmul.cpp:25-74   batched_matmul_runner:
 *      operands made contiguous, then a serial loop over the batch.
 *  - tinytensor/tensor/backend/cpu/kernel/matmul.hpp:153-225  matmul_kernel:
 *      column tiles of 64, row tiles of 64, K chunks of 64; within a chunk each
 *      C element is a k-sequential sum started from zero (tile_kernel, :113-150),
 *      and the chunk sum is then added to C (:141-149).
 *  - tinytensor/tensor/backend/cpu/kernel/simd.h:96-128: multiply and add are
 *      separate operations (no fused multiply-add is asked for); integer lanes
 *      wrap modulo 2^w, including the hand-built u8 and s64 multiplies.
 * The padding to multiples of 8 rows / 4 vectors and the aligned scratch copies
 * (matmul.hpp:157-196) only add zero terms and are not reproduced.
 *
 * Build with -ffp-contract=off so that mul and add stay separate.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>

#define ORACLE_CHUNK 64 /* TILE_STRIDE, matmul.hpp:27 */

#define DEFINE_MATMUL(NAME, T, ACC)                                                          \
    void oracle_matmul_##NAME(const T *A, const T *B, T *C, int64_t batch, int64_t N,        \
                              int64_t K, int64_t M) {                                        \
        for (int64_t b = 0; b < batch; ++b) {                                                \
            const T *a = A + b * N * K;                                                      \
            const T *bm = B + b * K * M;                                                     \
            T *c = C + b * N * M;                                                            \
            memset(c, 0, sizeof(T) * (size_t)(N * M));                                       \
            for (int64_t l = 0; l < K; l += ORACLE_CHUNK) {                                  \
                const int64_t r = (l + ORACLE_CHUNK < K) ? l + ORACLE_CHUNK : K;             \
                for (int64_t i = 0; i < N; ++i) {                                            \
                    for (int64_t j = 0; j < M; ++j) {                                        \
                        ACC t = 0;                                                           \
                        for (int64_t k = l; k < r; ++k) {                                    \
                            const ACC prod = (ACC)((ACC)a[i * K + k] * (ACC)bm[k * M + j]);  \
                            t = (ACC)(t + prod);                                             \
                        }                                                                    \
                        c[i * M + j] = (T)((ACC)c[i * M + j] + t);                           \
                    }                                                                        \
                }                                                                            \
            }                                                                                \
        }                                                                                    \
    }

/* Integer accumulators are unsigned of the same width: wrap-around without
 * undefined behaviour, identical bits to two's-complement signed wrap. */
DEFINE_MATMUL(u8, uint8_t, uint8_t)
DEFINE_MATMUL(i16, int16_t, uint16_t)
DEFINE_MATMUL(i32, int32_t, uint32_t)
DEFINE_MATMUL(i64, int64_t, uint64_t)
DEFINE_MATMUL(f32, float, float)
DEFINE_MATMUL(f64, double, double)

/* Cache-friendlier variant used for timing and for larger parity cases: same
 * arithmetic per C element (chunked, k-sequential, mul then add), loops reordered
 * so the inner loop streams over j.  Bit-identical to the functions above because
 * every C element sees the same sequence of operations. */
#define DEFINE_MATMUL_FAST(NAME, T, ACC)                                                     \
    void oracle_matmul_fast_##NAME(const T *A, const T *B, T *C, int64_t batch, int64_t N,   \
                                   int64_t K, int64_t M, ACC *row_scratch) {                 \
        for (int64_t b = 0; b < batch; ++b) {                                                \
            const T *a = A + b * N * K;                                                      \
            const T *bm = B + b * K * M;                                                     \
            T *c = C + b * N * M;                                                            \
            memset(c, 0, sizeof(T) * (size_t)(N * M));                                       \
            for (int64_t l = 0; l < K; l += ORACLE_CHUNK) {                                  \
                const int64_t r = (l + ORACLE_CHUNK < K) ? l + ORACLE_CHUNK : K;             \
                for (int64_t i = 0; i < N; ++i) {                                            \
                    for (int64_t j = 0; j < M; ++j) row_scratch[j] = 0;                      \
                    for (int64_t k = l; k < r; ++k) {                                        \
                        const ACC av = (ACC)a[i * K + k];                                    \
                        const T *brow = bm + k * M;                                          \
                        for (int64_t j = 0; j < M; ++j) {                                    \
                            const ACC prod = (ACC)(av * (ACC)brow[j]);                       \
                            row_scratch[j] = (ACC)(row_scratch[j] + prod);                   \
                        }                                                                    \
                    }                                                                        \
                    for (int64_t j = 0; j < M; ++j)                                          \
                        c[i * M + j] = (T)((ACC)c[i * M + j] + row_scratch[j]);              \
                }                                                                            \
            }                                                                                \
        }                                                                                    \
    }

DEFINE_MATMUL_FAST(u8, uint8_t, uint8_t)
DEFINE_MATMUL_FAST(i16, int16_t, uint16_t)
DEFINE_MATMUL_FAST(i32, int32_t, uint32_t)
DEFINE_MATMUL_FAST(i64, int64_t, uint64_t)
DEFINE_MATMUL_FAST(f32, float, float)
DEFINE_MATMUL_FAST(f64, double, double)
