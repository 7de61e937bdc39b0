// tt_conv_shim.cu -- the tinytensor-side adapter for conv2d: defines
// tinytensor::cuda::batched_conv2d_forward_runner and batched_conv2d_backward_runner with the
// signatures declared in tinytensor/tensor/backend/cuda/conv.h:16-30, so BackendCUDA::conv2d and
// conv2d_backward need no change.  Compile it into the tinytensor CUDA backend next to conv.cu
// with the two conv2d runners removed from that file (the pooling runners stay), and link
// libttb.so.
//
// Allocation goes through DeviceMemory<T>::AllocateElements like the reference
// (conv.cu:96-101, :248-257), so tinytensor's byte counters stay truthful; the kernels run on
// the legacy default stream (kernel_launch.cuh:24).  The bias gradient is computed by the
// library instead of three tensor reductions (conv.cu:396-399).
//
// This file is not part of libttb.so; it needs tinytensor's headers to compile.
#include <tt/concepts.h>
#include <tt/exception.h>
#include <tt/scalar.h>
#include <tt/shape.h>
#include <tt/tensor.h>

#include "tensor/backend/cuda/data_types.cuh"
#include "tensor/backend/cuda/storage_cuda.h"

#include <cstddef>
#include <memory>
#include <optional>
#include <string>
#include <tuple>
#include <type_traits>
#include <variant>

#include "../../include/ttb.h"

namespace tinytensor::cuda {

namespace {
ttb_conv2d_desc describe(const Tensor &input, const Tensor &weight, int stride, int padding) {
    if (input.dim() != 4 || weight.dim() != 4 || input.size(1) != weight.size(1) ||
        weight.size(2) != weight.size(3)) {
        TT_EXCEPTION("conv2d: input [B,C_in,H,W] and weight [C_out,C_in,K,K] expected");
    }
    ttb_conv2d_desc d{};
    d.batch = input.size(0);
    d.c_in = input.size(1);
    d.h_in = input.size(2);
    d.w_in = input.size(3);
    d.c_out = weight.size(0);
    d.kernel = weight.size(2);
    d.stride = stride;
    d.padding = padding;
    return d;
}
}    // namespace

auto batched_conv2d_forward_runner(
    const Tensor &input,
    const Tensor &weight,
    const std::optional<Tensor> &bias,
    int stride,
    int padding
) -> Tensor {
    const ttb_conv2d_desc d = describe(input, weight, stride, padding);
    const int H_out = static_cast<int>((d.h_in + 2 * d.padding - d.kernel) / d.stride + 1);
    const int W_out = static_cast<int>((d.w_in + 2 * d.padding - d.kernel) / d.stride + 1);
    const auto res_shape = Shape({static_cast<int>(d.batch), static_cast<int>(d.c_out), H_out, W_out});
    const int device_id = input.device().id;
    const Tensor x = input.contiguous();     // conv.cu:77
    const Tensor w = weight.contiguous();    // reshape of the weight needs it, conv.cu:74
    std::optional<Tensor> b;
    if (bias) {
        b = bias->contiguous();
    }
    return std::visit(
        [&](auto &&x_mem) -> Tensor {
            using DT = std::remove_cvref_t<decltype(x_mem)>;
            using T = template_parameter_t<DT>;
            const T *xp = x_mem.data_ptr() + x.offset();
            const T *wp = std::get<DT>(w.template get_storage<StorageCUDA>().dev_memory).data_ptr() + w.offset();
            const T *bp = nullptr;
            if (b) {
                bp = std::get<DT>(b->template get_storage<StorageCUDA>().dev_memory).data_ptr() + b->offset();
            }
            auto res = DeviceMemory<T>::AllocateElements(device_id, static_cast<std::size_t>(res_shape.numel()));
            const int rc = ttb_conv2d_forward(
                xp, wp, bp, res.data_ptr(), &d, static_cast<int>(input.dtype()), device_id, /*stream=*/nullptr
            );
            if (rc != TTB_OK) {
                TT_EXCEPTION(std::string("ttb_conv2d_forward: ") + ttb_last_error());
            }
            return {std::make_unique<StorageCUDA>(std::move(res)), input.dtype(), res_shape, input.device()};
        },
        x.template get_storage<StorageCUDA>().dev_memory
    );
}

auto batched_conv2d_backward_runner(
    const Tensor &grad_output,
    const Tensor &input,
    const Tensor &weight,
    const std::optional<Tensor> &bias,
    int stride,
    int padding
) -> std::tuple<Tensor, Tensor, std::optional<Tensor>> {
    const ttb_conv2d_desc d = describe(input, weight, stride, padding);
    const int device_id = input.device().id;
    const Tensor x = input.contiguous();
    const Tensor w = weight.contiguous();
    const Tensor g = grad_output.contiguous();
    return std::visit(
        [&](auto &&x_mem) -> std::tuple<Tensor, Tensor, std::optional<Tensor>> {
            using DT = std::remove_cvref_t<decltype(x_mem)>;
            using T = template_parameter_t<DT>;
            const T *xp = x_mem.data_ptr() + x.offset();
            const T *wp = std::get<DT>(w.template get_storage<StorageCUDA>().dev_memory).data_ptr() + w.offset();
            const T *gp = std::get<DT>(g.template get_storage<StorageCUDA>().dev_memory).data_ptr() + g.offset();
            auto gx = DeviceMemory<T>::AllocateElements(device_id, static_cast<std::size_t>(input.numel()));
            auto gw = DeviceMemory<T>::AllocateElements(device_id, static_cast<std::size_t>(weight.numel()));
            std::optional<DeviceMemory<T>> gb;
            if (bias) {
                gb = DeviceMemory<T>::AllocateElements(device_id, static_cast<std::size_t>(d.c_out));
            }
            const int rc = ttb_conv2d_backward(
                gp, xp, wp, gx.data_ptr(), gw.data_ptr(), gb ? gb->data_ptr() : nullptr, &d,
                static_cast<int>(input.dtype()), device_id, /*stream=*/nullptr
            );
            if (rc != TTB_OK) {
                TT_EXCEPTION(std::string("ttb_conv2d_backward: ") + ttb_last_error());
            }
            Tensor grad_input(std::make_unique<StorageCUDA>(std::move(gx)), input.dtype(), input.shape(), input.device());
            Tensor grad_w(std::make_unique<StorageCUDA>(std::move(gw)), input.dtype(), weight.shape(), weight.device());
            std::optional<Tensor> grad_b;
            if (gb) {
                grad_b = Tensor(
                    std::make_unique<StorageCUDA>(std::move(*gb)),
                    input.dtype(),
                    Shape({static_cast<int>(d.c_out)}),
                    input.device()
                );
            }
            return {grad_input, grad_w, grad_b};
        },
        x.template get_storage<StorageCUDA>().dev_memory
    );
}

}    // namespace tinytensor::cuda
