// tma_desc.cuh -- builds TMA tensor maps straight from a tinytensor view's
// strides and offset, so strided / transposed operands are consumed without the
// contiguous copy the reference makes (tinytensor/tensor/backend/cuda/matmul.cu:40-41).
//
// An operand is seen as a matrix with one "MN" dim (rows of lhs / columns of rhs)
// and the K dim, plus the batch dim:
//   K-major  : K has element stride 1  -> map dims {K, MN, B}, box {32, rows, 1}
//   MN-major : MN has element stride 1 -> map dims {MN, K, B}, box {32, 32, 1}
// Both use a 128-byte swizzle span (32 fp32 = one swizzle row): K-major tiles with
// 16-byte chunks, MN-major fp32 tiles with 32-byte chunks (the layout tcgen05.mma
// requires for MN-major tf32 operands).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ttb {

enum OperandMajor { kMajorK = 0, kMajorMN = 1, kMajorNone = -1 };

struct OperandView {
    const void *ptr;      // first element
    int64_t mn, k, batch; // extents
    int64_t s_mn, s_k, s_b; // element strides
};

// Classifies a view for TMA.  Returns kMajorNone (and a reason) when it cannot be fed
// through a tensor map: misaligned base, no unit-stride matrix dim, a byte stride that
// is not a multiple of 16, or a zero stride on a matrix dim.
OperandMajor classify_operand(const OperandView &v, size_t elem_size, char *why, int why_len);

// Encodes the tensor map.  `box_mn_rows` is the MN extent of the K-major box
// (<= 256).  `batch_mul` receives 0 when the batch dim is broadcast (stride 0) and
// the kernel must pin the batch coordinate to 0, else 1.
// Returns 0 on success, non-zero (with `why`) when the driver rejects the map.
int encode_operand_tmap(CUtensorMap *map, const OperandView &v, OperandMajor major, CUtensorMapDataType dt,
                        size_t elem_size, int box_inner, int box_mn_rows, int box_k_rows, int *batch_mul,
                        char *why, int why_len);

// Hits and misses of the calling thread's tensor-map cache (encode_operand_tmap keeps the maps
// it has built, keyed by pointer, extents, strides, element type and box).
void tensor_map_cache_stats(uint64_t *hits, uint64_t *misses);

}  // namespace ttb
