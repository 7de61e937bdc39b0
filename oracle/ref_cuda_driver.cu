// ref_cuda_driver.cu -- thin C entry points around the REFERENCE's own CUDA matmul kernel.
//
// TEST / BENCHMARK INFRASTRUCTURE ONLY.  No arithmetic of its own: it includes
// tinytensor/tensor/backend/cuda/kernel/matmul.cuh from the reference tree where it lies
// (include path given by the Makefile), instantiates kernel::matmul::matmul_kernel<T>
// (matmul.cuh:27) and launches it with the grid the reference's runner uses
// (tinytensor/tensor/backend/cuda/matmul.cu:62-72: 64 threads, grid = (ceil(M/64),
// ceil(N/64), B), default stream unless one is passed).  Operands must be contiguous, as the
// reference's runner makes them.  The result, libttref_cuda.so, goes to oracle/_ref/ and is
// the "existing GPU kernel" comparator: parity (bit-exact for integers) and timing.
#include <cstddef>
#include <cstdint>

#include "tensor/backend/cuda/kernel/matmul.cuh"

namespace {
template <typename T>
int run(const T *A, const T *B, T *C, int batch, int N, int K, int M, void *stream) {
    using namespace tinytensor::cuda;
    using namespace tinytensor::cuda::kernel::matmul;
    const DeviceSpan<const T> a{A, static_cast<std::size_t>(batch) * N * K};
    const DeviceSpan<const T> b{B, static_cast<std::size_t>(batch) * K * M};
    DeviceSpan<T> c{C, static_cast<std::size_t>(batch) * N * M};
    const dim3 block{(properties::TILE_WIDTH * properties::TILE_HEIGHT) / (properties::TN * properties::TM)};
    const dim3 grid{static_cast<unsigned>((M + properties::TILE_WIDTH - 1) / properties::TILE_WIDTH),
                    static_cast<unsigned>((N + properties::TILE_HEIGHT - 1) / properties::TILE_HEIGHT),
                    static_cast<unsigned>(batch)};
    matmul_kernel<T><<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(a, b, c, N, K, M);
    return static_cast<int>(cudaGetLastError());
}
}  // namespace

#define EXPORT extern "C" __attribute__((visibility("default")))
EXPORT int ref_cuda_matmul_u8(const uint8_t *A, const uint8_t *B, uint8_t *C, int b, int N, int K, int M, void *s) { return run(A, B, C, b, N, K, M, s); }
EXPORT int ref_cuda_matmul_i16(const int16_t *A, const int16_t *B, int16_t *C, int b, int N, int K, int M, void *s) { return run(A, B, C, b, N, K, M, s); }
EXPORT int ref_cuda_matmul_i32(const int32_t *A, const int32_t *B, int32_t *C, int b, int N, int K, int M, void *s) { return run(A, B, C, b, N, K, M, s); }
EXPORT int ref_cuda_matmul_i64(const int64_t *A, const int64_t *B, int64_t *C, int b, int N, int K, int M, void *s) { return run(A, B, C, b, N, K, M, s); }
EXPORT int ref_cuda_matmul_f32(const float *A, const float *B, float *C, int b, int N, int K, int M, void *s) { return run(A, B, C, b, N, K, M, s); }
EXPORT int ref_cuda_matmul_f64(const double *A, const double *B, double *C, int b, int N, int K, int M, void *s) { return run(A, B, C, b, N, K, M, s); }

// ---- conv2d forward without bias, as the reference's runner launches it per batch item
// (tinytensor/tensor/backend/cuda/conv.cu:110-160): unroll_kernel on a 1-D grid of
// THREADS_PER_BLOCK-thread blocks over the unrolled matrix, then matmul_kernel<T> of
// W[C_out, C_in*K*K] with it.  `unrolled` is a caller-provided buffer of C_in*K*K*H_out*W_out
// elements (the runner allocates it once per call, conv.cu:100-101).
#include "tensor/backend/cuda/kernel/conv.cuh"

namespace {
template <typename T>
int run_conv_fwd(const T *X, const T *W, T *Y, T *unrolled, int B, int C_in, int H_in, int W_in, int C_out, int K,
                 int S, int P, void *stream) {
    using namespace tinytensor::cuda;
    using namespace tinytensor::cuda::kernel::conv;
    using namespace tinytensor::cuda::kernel::matmul;
    const int H_out = (H_in + 2 * P - K) / S + 1, W_out = (W_in + 2 * P - K) / S + 1;
    const int rows = C_in * K * K, width = H_out * W_out;
    const DeviceSpan<const T> x{X, static_cast<std::size_t>(B) * C_in * H_in * W_in};
    const DeviceSpan<const T> w{W, static_cast<std::size_t>(C_out) * rows};
    DeviceSpan<T> u{unrolled, static_cast<std::size_t>(rows) * width};
    const dim3 block_unroll{static_cast<unsigned>(THREADS_PER_BLOCK)};
    const dim3 grid_unroll{static_cast<unsigned>((rows * width + THREADS_PER_BLOCK - 1) / THREADS_PER_BLOCK)};
    const dim3 block_mm{(properties::TILE_WIDTH * properties::TILE_HEIGHT) / (properties::TN * properties::TM)};
    const dim3 grid_mm{static_cast<unsigned>((width + properties::TILE_WIDTH - 1) / properties::TILE_WIDTH),
                       static_cast<unsigned>((C_out + properties::TILE_HEIGHT - 1) / properties::TILE_HEIGHT), 1};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int b = 0; b < B; ++b) {
        unroll_kernel<T><<<grid_unroll, block_unroll, 0, st>>>(x, u, b, C_in, H_in, W_in, K, S, P);
        DeviceSpan<T> res{Y + static_cast<std::size_t>(b) * C_out * width, static_cast<std::size_t>(C_out) * width};
        matmul_kernel<T><<<grid_mm, block_mm, 0, st>>>(w, DeviceSpan<const T>{u}, res, C_out, rows, width);
    }
    return static_cast<int>(cudaGetLastError());
}
}  // namespace

EXPORT int ref_cuda_conv2d_forward_f32(const float *X, const float *W, float *Y, float *unrolled, int B, int C_in,
                                       int H_in, int W_in, int C_out, int K, int S, int P, void *s) {
    return run_conv_fwd(X, W, Y, unrolled, B, C_in, H_in, W_in, C_out, K, S, P, s);
}
EXPORT int ref_cuda_conv2d_forward_i32(const int32_t *X, const int32_t *W, int32_t *Y, int32_t *unrolled, int B,
                                       int C_in, int H_in, int W_in, int C_out, int K, int S, int P, void *s) {
    return run_conv_fwd(X, W, Y, unrolled, B, C_in, H_in, W_in, C_out, K, S, P, s);
}
EXPORT int ref_cuda_conv2d_forward_f64(const double *X, const double *W, double *Y, double *unrolled, int B,
                                       int C_in, int H_in, int W_in, int C_out, int K, int S, int P, void *s) {
    return run_conv_fwd(X, W, Y, unrolled, B, C_in, H_in, W_in, C_out, K, S, P, s);
}
