// tt_reduce_all_shim.cu -- test-build adapter: defines tinytensor::cuda::reduce_all_runner<Op>
// (declared in tinytensor/tensor/backend/cuda/reduce.h:13-14) in terms of the reference's own
// reduce_dim_runner<Op> on the flattened tensor.
//
// Why: the reference's reduce_all_kernel (backend/cuda/kernel/reduce.cuh:46-114) lets every
// thread of its 512-thread block read partial_reduction_val[tid + 32] and
// partial_reduction_idx[tid + 32] before the `threadIdx.x < WARP_SIZE` test (:86-87), so threads
// 480-511 read up to 32 elements past the end of both shared arrays.  sm_100a reports that as an
// illegal memory access, which takes the context down.  The kernel sits outside the matmul path
// but under `allclose`, which every test of the reference uses to compare results -- so a
// tinytensor build for this GPU needs a reduce-all that does not fault before any of the
// reference's CUDA tests can say something about matmul.  reduce_dim_kernel (:19-38) is a plain
// loop per output element with no shared memory; over a flattened tensor with dim 0 it computes
// the same value, the same flat argmin / argmax index (ties to the smaller index) and the same
// result dtype and shape {1}.
//
// Build: compile backend/cuda/reduce.cu with -Dreduce_all_runner=<unused name> and add this file.
// Not part of libttb.so; it needs tinytensor's headers.
#include <tt/tensor.h>

#include "tensor/backend/common/reduce.h"
#include "tensor/backend/cuda/reduce.h"

namespace tinytensor::cuda {

using common::reduce::ReduceOpT;

template <ReduceOpT Op>
auto reduce_all_runner(const Tensor &tensor) -> Tensor {
    return reduce_dim_runner<Op>(tensor.flatten(), 0);
}

template Tensor reduce_all_runner<ReduceOpT::min>(const Tensor &tensor);
template Tensor reduce_all_runner<ReduceOpT::argmin>(const Tensor &tensor);
template Tensor reduce_all_runner<ReduceOpT::max>(const Tensor &tensor);
template Tensor reduce_all_runner<ReduceOpT::argmax>(const Tensor &tensor);
template Tensor reduce_all_runner<ReduceOpT::sum>(const Tensor &tensor);
template Tensor reduce_all_runner<ReduceOpT::all>(const Tensor &tensor);
template Tensor reduce_all_runner<ReduceOpT::any>(const Tensor &tensor);

}    // namespace tinytensor::cuda
