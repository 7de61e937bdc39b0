// tt_to_device_shim.cpp -- the tinytensor-side adapter for Tensor::to(Device): defines
// tinytensor::autograd::TensorToDevice::forward / backward (declared in
// tinytensor/autograd/unary_ops.h:29-33).
//
// The reference moves a tensor between devices through the host: to_vec<T>() (a blocking
// device-to-host copy into a std::vector) and a fresh tensor built from that vector on the
// target (tinytensor/autograd/unary_ops.cpp:67-83).  Between two CUDA devices this adapter
// makes one peer copy instead (ttb_copy_device_to_device: direct over NVLink where the
// devices can map each other), into storage allocated through
// DeviceMemory<T>::AllocateElements so tinytensor's byte counters stay truthful.  Every
// other pair of devices (CPU involved) keeps the reference's behaviour.
//
// Build: compile tinytensor/autograd/unary_ops.cpp with -DTensorToDevice=<unused name> so it
// no longer defines these two members, and add this file.  Not part of libttb.so; it needs
// tinytensor's headers.
#include <tt/autograd.h>
#include <tt/device.h>
#include <tt/exception.h>
#include <tt/scalar.h>
#include <tt/tensor.h>

#include "autograd/unary_ops.h"
#include "tensor/backend/common/dispatch.h"
#include "tensor/backend/cuda/data_types.cuh"
#include "tensor/backend/cuda/storage_cuda.h"

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <type_traits>
#include <variant>

#include <cuda_runtime_api.h>

#include "../../include/ttb.h"

namespace tinytensor::autograd {

namespace {
// Waits for the legacy default stream of `device_id` (the stream all tinytensor kernels use).
void sync_default_stream(int device_id) {
    int previous = 0;
    cudaError_t e = cudaGetDevice(&previous);
    if (e == cudaSuccess) {
        e = cudaSetDevice(device_id);
    }
    if (e == cudaSuccess) {
        e = cudaStreamSynchronize(cudaStreamLegacy);
    }
    (void)cudaSetDevice(previous);
    if (e != cudaSuccess) {
        TT_EXCEPTION(std::string("Tensor::to(Device): ") + cudaGetErrorString(e));
    }
}

// One device-to-device copy of a contiguous CUDA tensor onto another CUDA device.  The
// default streams of two devices are not ordered with each other, so the source's work is
// waited for before the copy and the copy before returning (the source tensor may be freed,
// stream-ordered on ITS device, right after); the reference's host bounce blocks likewise.
auto peer_copy(const Tensor &tensor, Device device) -> Tensor {
    using cuda::DeviceMemory;
    using cuda::StorageCUDA;
    const Tensor src = tensor.contiguous();
    const auto n = static_cast<std::size_t>(src.numel());
    sync_default_stream(src.device().id);
    Tensor result = std::visit(
        [&](auto &&src_mem) -> Tensor {
            using DT = std::remove_cvref_t<decltype(src_mem)>;
            using T = template_parameter_t<DT>;
            auto dst = DeviceMemory<T>::AllocateElements(device.id, n);
            const int rc = ttb_copy_device_to_device(
                dst.data_ptr(), device.id, src_mem.data_ptr() + src.offset(), src.device().id,
                static_cast<std::uint64_t>(n) * sizeof(T), /*stream=*/nullptr
            );
            if (rc != TTB_OK) {
                TT_EXCEPTION(std::string("ttb_copy_device_to_device: ") + ttb_last_error());
            }
            return {std::make_unique<StorageCUDA>(std::move(dst)), src.dtype(), src.shape(), device};
        },
        src.template get_storage<StorageCUDA>().dev_memory
    );
    sync_default_stream(device.id);
    return result;
}
}    // namespace

auto TensorToDevice::forward(
    [[maybe_unused]] AutogradStorage &storage,
    [[maybe_unused]] bool is_grad_required,
    const Tensor &tensor,
    Device device
) -> Tensor {
    if (is_grad_required) {
        storage["device"] = tensor.device();
    }
    if (tensor.device().backend == Backend::cuda && device.backend == Backend::cuda) {
        if (device.id < 0 || device.id >= get_device_count(Backend::cuda)) {
            TT_EXCEPTION("Device id " + std::to_string(device.id) + " is out of range");
        }
        return peer_copy(tensor, device);
    }
    // CPU on either side: the host vector IS the transfer, as in the reference.
    if (tensor.dtype() == kBool) {
        return {tensor.to_vec<bool>(), tensor.shape(), device};
    }
    return DISPATCH_ALL_TYPES(tensor.dtype(), "Tensor::to", [&]() -> Tensor {
        return {tensor.to_vec<scalar_t>(), tensor.shape(), device};
    });
}

auto TensorToDevice::backward(const AutogradStorage &storage, const Tensor &grad_output) -> GradList {
    return {grad_output.to(std::get<Device>(storage.at("device")))};
}

}    // namespace tinytensor::autograd
