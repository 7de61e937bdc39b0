// tt_runner_shim.cu -- the tinytensor-side adapter: a drop-in replacement for
// tinytensor/tensor/backend/cuda/matmul.cu.
//
// It defines tinytensor::cuda::batched_matmul_runner with the signature declared in
// tinytensor/tensor/backend/cuda/matmul.h:11, so BackendCUDA::batched_matmul
// (backend/cuda/backend_cuda.cpp:385-387) needs no change: compile this file into the
// tinytensor CUDA backend in place of matmul.cu and link libttb.so.
//
// Unlike the file it replaces it makes no contiguous copies: the operands' shape, stride
// and element offset go straight into ttb_view.  The output is allocated through
// DeviceMemory<T>::AllocateElements like the reference does (matmul.cu:50), which keeps
// tinytensor's per-device byte counters (storage_cuda.h:66-67) truthful, and the kernels
// run on the legacy default stream like every other tinytensor kernel
// (kernel_launch.cuh:24).
//
// This file is not part of libttb.so; it needs tinytensor's headers to compile.
#include <tt/concepts.h>
#include <tt/exception.h>
#include <tt/scalar.h>
#include <tt/shape.h>
#include <tt/tensor.h>

#include "tensor/backend/cuda/data_types.cuh"
#include "tensor/backend/cuda/matmul.h"
#include "tensor/backend/cuda/storage_cuda.h"

#include <cstddef>
#include <memory>
#include <string>
#include <type_traits>
#include <variant>

#include "../../include/ttb.h"

namespace tinytensor::cuda {

auto batched_matmul_runner(const Tensor &lhs, const Tensor &rhs) -> Tensor {
    if (lhs.dim() != 3 || rhs.dim() != 3) {
        TT_EXCEPTION("batched_matmul expects rank-3 operands");
    }
    // The caller guarantees equal dtypes and devices and matching inner dims
    // (tensor.cpp:2390-2472); the batch sizes are checked by the library.
    const int B = lhs.size(0);
    const int N = lhs.size(1);
    const int M = rhs.size(2);
    const int device_id = lhs.device().id;
    const auto res_shape = Shape({B, N, M});
    const auto res_device = lhs.device();

    return std::visit(
        [&](auto &&lhs_mem) -> Tensor {
            using DT = std::remove_cvref_t<decltype(lhs_mem)>;
            using T = template_parameter_t<DT>;
            const auto &rhs_mem = std::get<DT>(rhs.template get_storage<StorageCUDA>().dev_memory);

            ttb_view lv{};
            lv.data = lhs_mem.data_ptr();
            lv.offset = lhs.offset();
            ttb_view rv{};
            rv.data = rhs_mem.data_ptr();
            rv.offset = rhs.offset();
            for (int d = 0; d < 3; ++d) {
                lv.size[d] = lhs.size(d);
                lv.stride[d] = lhs.stride()[d];
                rv.size[d] = rhs.size(d);
                rv.stride[d] = rhs.stride()[d];
            }
            if (lv.size[0] != rv.size[0] || lv.size[2] != rv.size[1]) {
                TT_EXCEPTION("batched_matmul: operand shapes do not agree");
            }
            auto res = DeviceMemory<T>::AllocateElements(
                device_id, static_cast<std::size_t>(B) * static_cast<std::size_t>(N) * static_cast<std::size_t>(M)
            );
            const int rc = ttb_batched_matmul(
                &lv, &rv, res.data_ptr(), static_cast<int>(lhs.dtype()), device_id, /*stream=*/nullptr
            );
            if (rc != TTB_OK) {
                TT_EXCEPTION(std::string("ttb_batched_matmul: ") + ttb_last_error());
            }
            return {std::make_unique<StorageCUDA>(std::move(res)), lhs.dtype(), res_shape, res_device};
        },
        lhs.template get_storage<StorageCUDA>().dev_memory
    );
}

}    // namespace tinytensor::cuda
