/* conv_oracle.c -- CPU restatement of the reference's conv2d forward / backward.
 *
 * TEST INFRASTRUCTURE ONLY: nothing in the product links or calls this file.
 * It follows the reference's CPU runner step by step, so that results can be compared bit
 * for bit with the reference's own code compiled into oracle/_ref/libttref*.so:
 *   forward  (tinytensor/tensor/backend/cpu/conv.cpp:36-133): per batch item unroll
 *            (backend/cpu/kernel/conv.hpp:12-47), W[C_out, C_in*K*K] . unrolled
 *            (the matmul restated in matmul_oracle.c), then + bias in T.
 *   backward (conv.cpp:135-289): per batch item unroll-transposed (conv.hpp:49-82),
 *            grad_w += g_out[b] . unrolled^T, unrolled = W^T . g_out[b], col2im
 *            (conv.hpp:84-119); grad_bias = sums of g_out over w, then h, then batch
 *            (conv.cpp:283).
 * Pinned by tests/test_oracle_conv.py against the reference's own test data
 * (tests/test_conv.cpp:99-145, the direct 7-loop definition) and against libttref.so.
 * Integer sums wrap (unsigned arithmetic); floats keep mul and add separate
 * (-ffp-contract=off in the Makefile).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define DECLARE_MATMUL(NAME, T) \
    void oracle_matmul_##NAME(const T *A, const T *B, T *C, int64_t batch, int64_t N, int64_t K, int64_t M);
DECLARE_MATMUL(u8, uint8_t)
DECLARE_MATMUL(i16, int16_t)
DECLARE_MATMUL(i32, int32_t)
DECLARE_MATMUL(i64, int64_t)
DECLARE_MATMUL(f32, float)
DECLARE_MATMUL(f64, double)

#define DEFINE_CONV(NAME, T, ACC)                                                                      \
    /* transposed == 0: U[(c*K*K + p*K + q)][h*W_out + w]; else U[h*W_out + w][c*K*K + p*K + q] */      \
    static void unroll_##NAME(const T *X, T *U, int b, int C_in, int H_in, int W_in, int K, int S,     \
                              int P, int transposed) {                                                 \
        const int H_out = (H_in + 2 * P - K) / S + 1, W_out = (W_in + 2 * P - K) / S + 1;              \
        const int64_t width = (int64_t)H_out * W_out, rows = (int64_t)C_in * K * K;                     \
        for (int c = 0; c < C_in; ++c)                                                                 \
            for (int p = 0; p < K; ++p)                                                                \
                for (int q = 0; q < K; ++q)                                                            \
                    for (int h = 0; h < H_out; ++h)                                                    \
                        for (int w = 0; w < W_out; ++w) {                                              \
                            const int h_in = S * h + p - P, w_in = S * w + q - P;                      \
                            const int64_t r = (int64_t)c * K * K + p * K + q, col = (int64_t)h * W_out + w; \
                            const int inside = !(h_in < 0 || w_in < 0 || h_in >= H_in || w_in >= W_in);  \
                            const T v = inside ? X[(((int64_t)b * C_in + c) * H_in + h_in) * W_in + w_in] : (T)0; \
                            U[transposed ? col * rows + r : r * width + col] = v;                      \
                        }                                                                              \
    }                                                                                                  \
    static void col2im_##NAME(T *X, const T *U, int C_in, int H_in, int W_in, int K, int S, int P) {   \
        const int H_out = (H_in + 2 * P - K) / S + 1, W_out = (W_in + 2 * P - K) / S + 1;              \
        const int64_t width = (int64_t)H_out * W_out;                                                  \
        for (int c = 0; c < C_in; ++c)                                                                 \
            for (int p = 0; p < K; ++p)                                                                \
                for (int q = 0; q < K; ++q)                                                            \
                    for (int h = 0; h < H_out; ++h)                                                    \
                        for (int w = 0; w < W_out; ++w) {                                              \
                            const int h_in = S * h + p - P, w_in = S * w + q - P;                      \
                            if (h_in < 0 || w_in < 0 || h_in >= H_in || w_in >= W_in) continue;        \
                            T *dst = &X[((int64_t)c * H_in + h_in) * W_in + w_in];                     \
                            *dst = (T)((ACC)*dst + (ACC)U[((int64_t)c * K * K + p * K + q) * width + (int64_t)h * W_out + w]); \
                        }                                                                              \
    }                                                                                                  \
    void oracle_conv2d_forward_##NAME(const T *X, const T *W, const T *bias, T *Y, int B, int C_in,    \
                                      int H_in, int W_in, int C_out, int K, int S, int P) {            \
        const int H_out = (H_in + 2 * P - K) / S + 1, W_out = (W_in + 2 * P - K) / S + 1;              \
        const int64_t width = (int64_t)H_out * W_out, rows = (int64_t)C_in * K * K;                     \
        T *U = (T *)malloc((size_t)(rows * width) * sizeof(T));                                        \
        for (int b = 0; b < B; ++b) {                                                                  \
            T *res = Y + (int64_t)b * C_out * width;                                                   \
            unroll_##NAME(X, U, b, C_in, H_in, W_in, K, S, P, 0);                                      \
            oracle_matmul_##NAME(W, U, res, 1, C_out, rows, width);                                    \
            if (bias)                                                                                  \
                for (int m = 0; m < C_out; ++m)                                                        \
                    for (int64_t i = 0; i < width; ++i)                                                \
                        res[m * width + i] = (T)((ACC)res[m * width + i] + (ACC)bias[m]);              \
        }                                                                                              \
        free(U);                                                                                       \
    }                                                                                                  \
    void oracle_conv2d_backward_##NAME(const T *G, const T *X, const T *W, T *GX, T *GW, T *GB, int B, \
                                       int C_in, int H_in, int W_in, int C_out, int K, int S, int P) { \
        const int H_out = (H_in + 2 * P - K) / S + 1, W_out = (W_in + 2 * P - K) / S + 1;              \
        const int64_t width = (int64_t)H_out * W_out, rows = (int64_t)C_in * K * K;                     \
        const int64_t wn = (int64_t)C_out * rows, xn = (int64_t)C_in * H_in * W_in;                    \
        T *U = (T *)malloc((size_t)(rows * width) * sizeof(T));                                        \
        T *Wt = (T *)malloc((size_t)wn * sizeof(T));                                                   \
        T *local = (T *)malloc((size_t)wn * sizeof(T));                                                \
        for (int64_t r = 0; r < rows; ++r)                                                             \
            for (int m = 0; m < C_out; ++m) Wt[r * C_out + m] = W[m * rows + r];                       \
        memset(GX, 0, (size_t)(B * xn) * sizeof(T));                                                   \
        memset(GW, 0, (size_t)wn * sizeof(T));                                                         \
        for (int b = 0; b < B; ++b) {                                                                  \
            const T *g = G + (int64_t)b * C_out * width;                                               \
            unroll_##NAME(X, U, b, C_in, H_in, W_in, K, S, P, 1);                                      \
            oracle_matmul_##NAME(g, U, local, 1, C_out, width, rows);                                  \
            for (int64_t i = 0; i < wn; ++i) GW[i] = (T)((ACC)GW[i] + (ACC)local[i]);                  \
            oracle_matmul_##NAME(Wt, g, U, 1, rows, C_out, width);                                     \
            col2im_##NAME(GX + b * xn, U, C_in, H_in, W_in, K, S, P);                                  \
        }                                                                                              \
        if (GB) {                                                                                      \
            /* sum(3), sum(2), sum(0): rows of w first, then h, then the batch */                     \
            T *hsum = (T *)malloc((size_t)((int64_t)B * C_out) * sizeof(T));                           \
            for (int64_t bm = 0; bm < (int64_t)B * C_out; ++bm) {                                      \
                ACC over_h = (ACC)0;                                                                   \
                for (int h = 0; h < H_out; ++h) {                                                      \
                    ACC over_w = (ACC)0;                                                               \
                    for (int w = 0; w < W_out; ++w) over_w = (ACC)(over_w + (ACC)G[bm * width + (int64_t)h * W_out + w]); \
                    over_h = (ACC)(over_h + (ACC)(T)over_w);                                           \
                }                                                                                      \
                hsum[bm] = (T)over_h;                                                                  \
            }                                                                                          \
            for (int m = 0; m < C_out; ++m) {                                                          \
                ACC s = (ACC)0;                                                                        \
                for (int b = 0; b < B; ++b) s = (ACC)(s + (ACC)hsum[(int64_t)b * C_out + m]);          \
                GB[m] = (T)s;                                                                          \
            }                                                                                          \
            free(hsum);                                                                                \
        }                                                                                              \
        free(U);                                                                                       \
        free(Wt);                                                                                      \
        free(local);                                                                                   \
    }

DEFINE_CONV(u8, uint8_t, uint8_t)
DEFINE_CONV(i16, int16_t, uint16_t)
DEFINE_CONV(i32, int32_t, uint32_t)
DEFINE_CONV(i64, int64_t, uint64_t)
DEFINE_CONV(f32, float, float)
DEFINE_CONV(f64, double, double)
