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
