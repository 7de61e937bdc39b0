// ref_driver.cpp -- thin C entry points around the REFERENCE's own CPU matmul kernel.
//
// TEST INFRASTRUCTURE ONLY.  This file contains no arithmetic of its own: it
// includes tinytensor/tensor/backend/cpu/kernel/matmul.hpp from the reference tree
// where it lies (the include path is given on the command line by the Makefile),
// instantiates kernel::matmul::matmul_kernel<T> (matmul.hpp:153) and loops over
// the batch exactly as cpu::batched_matmul_runner does
// (tinytensor/tensor/backend/cpu/matmul.cpp:56-68).  The result, libttref.so,
// goes to oracle/_ref/ and is used to validate oracle/matmul_oracle.c and as the
// timed CPU baseline.  No reference source is copied into this repository.
#include <cstddef>
#include <cstdint>

#include "tensor/backend/common/span.h"
#include "tensor/backend/cpu/kernel/matmul.hpp"

namespace {
template <typename T>
void run(const T *A, const T *B, T *C, int64_t batch, int N, int K, int M) {
    using namespace tinytensor;
    using namespace tinytensor::cpu::kernel::matmul;
    for (int64_t b = 0; b < batch; ++b) {
        const HostSpan<const T> lhs{A + b * N * K, static_cast<std::size_t>(N) * K};
        const HostSpan<const T> rhs{B + b * K * M, static_cast<std::size_t>(K) * M};
        HostSpan<T> res{C + b * N * M, static_cast<std::size_t>(N) * M};
        matmul_kernel<T>(lhs, rhs, res, N, K, M);
    }
}
}  // namespace

#define EXPORT extern "C" __attribute__((visibility("default")))
EXPORT void ref_matmul_u8(const uint8_t *A, const uint8_t *B, uint8_t *C, int64_t b, int N, int K, int M) { run(A, B, C, b, N, K, M); }
EXPORT void ref_matmul_i16(const int16_t *A, const int16_t *B, int16_t *C, int64_t b, int N, int K, int M) { run(A, B, C, b, N, K, M); }
EXPORT void ref_matmul_i32(const int32_t *A, const int32_t *B, int32_t *C, int64_t b, int N, int K, int M) { run(A, B, C, b, N, K, M); }
EXPORT void ref_matmul_i64(const int64_t *A, const int64_t *B, int64_t *C, int64_t b, int N, int K, int M) { run(A, B, C, b, N, K, M); }
EXPORT void ref_matmul_f32(const float *A, const float *B, float *C, int64_t b, int N, int K, int M) { run(A, B, C, b, N, K, M); }
EXPORT void ref_matmul_f64(const double *A, const double *B, double *C, int64_t b, int N, int K, int M) { run(A, B, C, b, N, K, M); }

// ---- conv2d: the reference's CPU kernels (backend/cpu/kernel/conv.hpp) driven in the order
// cpu::batched_conv2d_forward_runner / batched_conv2d_backward_runner drive them
// (tinytensor/tensor/backend/cpu/conv.cpp:108-127 and :216-262).  The only arithmetic written
// here is the element-wise `+` of the bias and of the weight-gradient accumulation, which the
// reference performs with its binary add kernel in the same type T.
#include <vector>

#include "tensor/backend/cpu/kernel/conv.hpp"

namespace {
template <typename T>
void conv_fwd(const T *X, const T *W, const T *bias, T *Y, int B, int C_in, int H_in, int W_in, int C_out, int K,
              int S, int P) {
    using namespace tinytensor;
    using namespace tinytensor::cpu::kernel::conv;
    using namespace tinytensor::cpu::kernel::matmul;
    const int H_out = (H_in + 2 * P - K) / S + 1, W_out = (W_in + 2 * P - K) / S + 1;
    const int rows = C_in * K * K, width = H_out * W_out;
    std::vector<T> unrolled(static_cast<std::size_t>(rows) * width);
    const HostSpan<const T> x_span{X, static_cast<std::size_t>(B) * C_in * H_in * W_in};
    const HostSpan<const T> w_span{W, static_cast<std::size_t>(C_out) * rows};
    HostSpan<T> u_span{unrolled};
    for (int b = 0; b < B; ++b) {
        unroll_kernel(x_span, u_span, b, C_in, H_in, W_in, K, S, P);
        T *res = Y + static_cast<std::size_t>(b) * C_out * width;
        const HostSpan<T> res_span{res, static_cast<std::size_t>(C_out) * width};
        matmul_kernel(w_span, HostSpan<const T>{u_span}, res_span, C_out, rows, width);
        if (bias)
            for (int m = 0; m < C_out; ++m)
                for (int i = 0; i < width; ++i) res[m * width + i] = static_cast<T>(res[m * width + i] + bias[m]);
    }
}

template <typename T>
void conv_bwd(const T *G, const T *X, const T *W, T *GX, T *GW, int B, int C_in, int H_in, int W_in, int C_out,
              int K, int S, int P) {
    using namespace tinytensor;
    using namespace tinytensor::cpu::kernel::conv;
    using namespace tinytensor::cpu::kernel::matmul;
    const int H_out = (H_in + 2 * P - K) / S + 1, W_out = (W_in + 2 * P - K) / S + 1;
    const int rows = C_in * K * K, width = H_out * W_out;
    const std::size_t wn = static_cast<std::size_t>(C_out) * rows, xn = static_cast<std::size_t>(C_in) * H_in * W_in;
    std::vector<T> unrolled(static_cast<std::size_t>(rows) * width, 0), local(wn, 0), wt(wn);
    for (int r = 0; r < rows; ++r)  // weight.reshape({C_out, rows}).permute({1, 0}).contiguous()
        for (int m = 0; m < C_out; ++m) wt[static_cast<std::size_t>(r) * C_out + m] = W[static_cast<std::size_t>(m) * rows + r];
    for (std::size_t i = 0; i < wn; ++i) GW[i] = 0;
    for (std::size_t i = 0; i < xn * B; ++i) GX[i] = 0;
    const HostSpan<const T> x_span{X, xn * B};
    const HostSpan<const T> wt_span{wt.data(), wn};
    HostSpan<T> u_span{unrolled};
    HostSpan<T> local_span{local};
    for (int b = 0; b < B; ++b) {
        unroll_transpose_kernel(x_span, u_span, b, C_in, H_in, W_in, K, S, P);
        const HostSpan<const T> g_span{G + static_cast<std::size_t>(b) * C_out * width,
                                       static_cast<std::size_t>(C_out) * width};
        matmul_kernel(g_span, HostSpan<const T>{u_span}, local_span, C_out, width, rows);
        for (std::size_t i = 0; i < wn; ++i) GW[i] = static_cast<T>(GW[i] + local[i]);
        matmul_kernel(wt_span, g_span, u_span, rows, C_out, width);
        HostSpan<T> gx_span{GX + b * xn, xn};
        col2im_kernel(gx_span, HostSpan<const T>{u_span}, 0, C_in, H_in, W_in, K, S, P);
    }
}
}  // namespace

#define CONV_EXPORTS(NAME, T)                                                                                     \
    EXPORT void ref_conv2d_forward_##NAME(const T *X, const T *W, const T *bias, T *Y, int B, int C_in, int H_in, \
                                          int W_in, int C_out, int K, int S, int P) {                             \
        conv_fwd(X, W, bias, Y, B, C_in, H_in, W_in, C_out, K, S, P);                                             \
    }                                                                                                             \
    EXPORT void ref_conv2d_backward_##NAME(const T *G, const T *X, const T *W, T *GX, T *GW, int B, int C_in,     \
                                           int H_in, int W_in, int C_out, int K, int S, int P) {                  \
        conv_bwd(G, X, W, GX, GW, B, C_in, H_in, W_in, C_out, K, S, P);                                           \
    }
CONV_EXPORTS(u8, uint8_t)
CONV_EXPORTS(i16, int16_t)
CONV_EXPORTS(i32, int32_t)
CONV_EXPORTS(i64, int64_t)
CONV_EXPORTS(f32, float)
CONV_EXPORTS(f64, double)
