// tt_alloc_shim.h -- moves tinytensor's DeviceMemory<T> onto libttb.so's stream-ordered
// memory pool without editing tinytensor's sources.
//
// DeviceMemory<T> is the one place tinytensor's CUDA backend allocates and frees device
// memory: cudaMalloc at tinytensor/tensor/backend/cuda/data_types.cu:44 and cudaFree at
// :109, each right after a cudaSetDevice(device_id).  Compile THAT translation unit (and no
// other) with this header force-included (nvcc -include tt_alloc_shim.h): the two calls then
// resolve to ttb_device_alloc / ttb_device_free on the current device and the legacy default
// stream, the stream every tinytensor kernel runs on (kernel_launch.cuh:24).  The pool caches
// freed blocks, so a result tensor costs neither cudaMalloc's nor cudaFree's device-wide
// synchronisation; tinytensor's own byte counters (storage_cuda.h:66-67) are untouched.  Blocks
// are handed out zero-filled (see pool_malloc).
//
// This header is not part of libttb.so.
#ifndef TTB_TT_ALLOC_SHIM_H_
#define TTB_TT_ALLOC_SHIM_H_

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdio>
#include <cstdlib>

#include "../../include/ttb.h"

namespace ttb_dropin {

// TTB_DROPIN_TRACE=1 in the environment lists every allocation and release on stderr.
inline bool trace() {
    static const bool on = std::getenv("TTB_DROPIN_TRACE") != nullptr;
    return on;
}

inline cudaError_t pool_malloc(void **p, std::size_t bytes) {
    int device = 0;
    const cudaError_t st = cudaGetDevice(&device);
    if (st != cudaSuccess) {
        return st;
    }
    if (ttb_device_alloc(p, bytes, device, /*stream=*/nullptr) != TTB_OK) {
        std::fprintf(stderr, "tinytensor DeviceMemory: %s\n", ttb_last_error());    // the status code alone says little
        return cudaErrorMemoryAllocation;
    }
    if (trace()) std::fprintf(stderr, "tinytensor DeviceMemory: alloc %p %zu bytes on device %d\n", *p, bytes, device);
    // tinytensor's pooling backward adds into its freshly allocated grad_input without clearing it
    // (backend/cuda/conv.cu:526-527, kernel/conv.cuh:216 and :252): that holds only while every
    // block comes zero-filled from the driver, as new cudaMalloc pages do.  The pool hands back
    // used blocks, so each one is cleared here, in stream order (a write at HBM speed; still far
    // cheaper than the cudaMalloc / cudaFree pair it replaces).
    return bytes ? cudaMemsetAsync(*p, 0, bytes, /*stream=*/nullptr) : cudaSuccess;
}

inline cudaError_t pool_free(void *p) {
    int device = 0;
    const cudaError_t st = cudaGetDevice(&device);
    if (st != cudaSuccess) {
        return st;
    }
    if (trace()) std::fprintf(stderr, "tinytensor DeviceMemory: free  %p on device %d\n", p, device);
    if (ttb_device_free(p, device, /*stream=*/nullptr) != TTB_OK) {
        std::fprintf(stderr, "tinytensor DeviceMemory: %s\n", ttb_last_error());
        return cudaErrorInvalidValue;
    }
    return cudaSuccess;
}

}    // namespace ttb_dropin

// After cuda_runtime.h has been read (its include guard keeps it from being read again), so
// only the calls written in the translation unit itself are redirected.
#define cudaMalloc(pp, bytes) ::ttb_dropin::pool_malloc(reinterpret_cast<void **>(pp), (bytes))
#define cudaFree(p)           ::ttb_dropin::pool_free(p)

#endif    // TTB_TT_ALLOC_SHIM_H_
