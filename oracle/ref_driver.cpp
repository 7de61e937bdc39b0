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
