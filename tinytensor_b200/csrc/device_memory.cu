// device_memory.cu -- stream-ordered cached device allocations and device-to-device copies.
//
// The reference allocates every tensor with cudaMalloc and releases it with cudaFree
// (DeviceMemory<T>, backend/cuda/data_types.cu:38-50 and :102-116): both synchronise the whole
// device, so each matmul result costs two device-wide stalls, and a tensor changes device by
// being read back into a host vector and uploaded again (autograd/unary_ops.cpp:67-83).
// Here an allocation comes from one explicit CUDA memory pool per device whose release
// threshold is "never": a freed block stays in the pool and the next request of that size on the
// same stream gets it back without a driver call, in stream order (no synchronisation; blocks
// move between streams only behind the event dependencies the pool tracks).  The byte counters
// mirror StorageCUDA::current_bytes_allocated / total_bytes_allocated.  A copy between devices
// is one cudaMemcpyPeerAsync, direct over NVLink once peer access is on (enabled on first use
// for that pair, pool included), staged by the driver otherwise.
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace ttb {
namespace {

constexpr int kMaxDevices = 64;

struct PoolState {
    cudaMemPool_t pool = nullptr;
    std::unordered_map<void *, uint64_t> live;  // pointer -> bytes, for the counters
    uint64_t current = 0;                       // bytes handed out and not yet freed
    uint64_t total = 0;                         // bytes ever handed out
    bool peer_on[kMaxDevices] = {};             // the pair (this device -> that device) has been set up
    bool peer_direct[kMaxDevices] = {};         // ... and that device can map this device's memory
};

std::mutex g_mem_mutex;
PoolState g_pools[kMaxDevices];

int check_device(int device, const char *who) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceCount");
    if (device < 0 || device >= n || device >= kMaxDevices) {
        set_error("%s: device %d out of range (%d devices)", who, device, n);
        return TTB_EDEVICE;
    }
    return TTB_OK;
}

// These entry points serve any device from any thread: they switch the calling thread to the
// device they work on and put its previous device back when they return.
struct DeviceGuard {
    int prev = -1;
    DeviceGuard() {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) (void)cudaSetDevice(prev);
    }
};

// The device's pool, created on first use.  Caller holds g_mem_mutex.
int pool_of(int device, PoolState **out) {
    PoolState &ps = g_pools[device];
    if (ps.pool == nullptr) {
        cudaMemPoolProps props{};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = device;
        cudaError_t e = cudaMemPoolCreate(&ps.pool, &props);
        if (e != cudaSuccess) {
            ps.pool = nullptr;
            return cuda_fail(e, "cudaMemPoolCreate");
        }
        uint64_t keep = UINT64_MAX;  // freed blocks stay cached until ttb_device_trim
        e = cudaMemPoolSetAttribute(ps.pool, cudaMemPoolAttrReleaseThreshold, &keep);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemPoolSetAttribute");
        // devices that were given peer access before this pool existed
        for (int d = 0; d < kMaxDevices; ++d) {
            if (!ps.peer_direct[d]) continue;
            cudaMemAccessDesc access{};
            access.location.type = cudaMemLocationTypeDevice;
            access.location.id = d;
            access.flags = cudaMemAccessFlagsProtReadWrite;
            e = cudaMemPoolSetAccess(ps.pool, &access, 1);
            if (e != cudaSuccess) return cuda_fail(e, "cudaMemPoolSetAccess");
        }
    }
    *out = &ps;
    return TTB_OK;
}

}  // namespace
}  // namespace ttb

using namespace ttb;

TTB_API int ttb_device_alloc(void **ptr, uint64_t bytes, int device_id, void *stream) {
    if (ptr == nullptr) {
        set_error("ttb_device_alloc: ptr is null");
        return TTB_EINVAL;
    }
    *ptr = nullptr;
    int rc = check_device(device_id, "ttb_device_alloc");
    if (rc != TTB_OK) return rc;
    if (bytes == 0) return TTB_OK;  // like cudaMalloc(0): success, null pointer
    DeviceGuard guard;
    std::lock_guard<std::mutex> lock(g_mem_mutex);
    PoolState *ps;
    rc = pool_of(device_id, &ps);
    if (rc != TTB_OK) return rc;
    void *p = nullptr;
    cudaError_t e = cudaSetDevice(device_id);  // a NULL stream means this device's default stream
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    e = cudaMallocFromPoolAsync(&p, bytes, ps->pool, static_cast<cudaStream_t>(stream));
    if (e == cudaErrorMemoryAllocation) {
        (void)cudaGetLastError();
        set_error("ttb_device_alloc: out of memory asking for %llu bytes on device %d (%llu in use here)",
                  static_cast<unsigned long long>(bytes), device_id, static_cast<unsigned long long>(ps->current));
        return TTB_ENOMEM;
    }
    if (e != cudaSuccess) return cuda_fail(e, "cudaMallocFromPoolAsync");
    ps->live[p] = bytes;
    ps->current += bytes;
    ps->total += bytes;
    *ptr = p;
    return TTB_OK;
}

TTB_API int ttb_device_free(void *ptr, int device_id, void *stream) {
    if (ptr == nullptr) return TTB_OK;
    int rc = check_device(device_id, "ttb_device_free");
    if (rc != TTB_OK) return rc;
    DeviceGuard guard;
    std::lock_guard<std::mutex> lock(g_mem_mutex);
    PoolState &ps = g_pools[device_id];
    auto it = ps.live.find(ptr);
    if (it == ps.live.end()) {
        set_error("ttb_device_free: %p was not allocated by ttb_device_alloc on device %d (or was freed already)", ptr,
                  device_id);
        return TTB_EINVAL;
    }
    cudaError_t e = cudaSetDevice(device_id);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    e = cudaFreeAsync(ptr, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "cudaFreeAsync");
    ps.current -= it->second;
    ps.live.erase(it);
    return TTB_OK;
}

TTB_API int ttb_device_memory_stats(int device_id, uint64_t *current_bytes, uint64_t *total_bytes,
                                    uint64_t *reserved_bytes) {
    int rc = check_device(device_id, "ttb_device_memory_stats");
    if (rc != TTB_OK) return rc;
    std::lock_guard<std::mutex> lock(g_mem_mutex);
    PoolState &ps = g_pools[device_id];
    if (current_bytes) *current_bytes = ps.current;
    if (total_bytes) *total_bytes = ps.total;
    if (reserved_bytes) {
        uint64_t reserved = 0;
        if (ps.pool != nullptr) {
            cudaError_t e = cudaMemPoolGetAttribute(ps.pool, cudaMemPoolAttrReservedMemCurrent, &reserved);
            if (e != cudaSuccess) return cuda_fail(e, "cudaMemPoolGetAttribute");
        }
        *reserved_bytes = reserved;
    }
    return TTB_OK;
}

TTB_API int ttb_device_trim(int device_id) {
    int rc = check_device(device_id, "ttb_device_trim");
    if (rc != TTB_OK) return rc;
    DeviceGuard guard;
    std::lock_guard<std::mutex> lock(g_mem_mutex);
    PoolState &ps = g_pools[device_id];
    if (ps.pool == nullptr) return TTB_OK;
    // Frees are stream-ordered: let them land, then give every cached block back to the driver.
    cudaError_t e = cudaSetDevice(device_id);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSynchronize");
    e = cudaMemPoolTrimTo(ps.pool, 0);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemPoolTrimTo");
    return TTB_OK;
}

TTB_API int ttb_copy_device_to_device(void *dst, int dst_device, const void *src, int src_device, uint64_t bytes,
                                      void *stream) {
    if (bytes == 0) return TTB_OK;
    if (dst == nullptr || src == nullptr) {
        set_error("ttb_copy_device_to_device: null pointer");
        return TTB_EINVAL;
    }
    int rc = check_device(dst_device, "ttb_copy_device_to_device");
    if (rc != TTB_OK) return rc;
    rc = check_device(src_device, "ttb_copy_device_to_device");
    if (rc != TTB_OK) return rc;
    DeviceGuard guard;
    cudaError_t e;
    if (dst_device != src_device) {
        std::lock_guard<std::mutex> lock(g_mem_mutex);
        PoolState &sp = g_pools[src_device];
        if (!sp.peer_on[dst_device]) {
            int can = 0;
            e = cudaDeviceCanAccessPeer(&can, dst_device, src_device);
            if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceCanAccessPeer");
            if (can) {
                e = cudaSetDevice(dst_device);
                if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
                e = cudaDeviceEnablePeerAccess(src_device, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) {
                    (void)cudaGetLastError();
                    e = cudaSuccess;
                }
                if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceEnablePeerAccess");
                sp.peer_direct[dst_device] = true;
                if (sp.pool != nullptr) {
                    cudaMemAccessDesc access{};
                    access.location.type = cudaMemLocationTypeDevice;
                    access.location.id = dst_device;
                    access.flags = cudaMemAccessFlagsProtReadWrite;
                    e = cudaMemPoolSetAccess(sp.pool, &access, 1);
                    if (e != cudaSuccess) return cuda_fail(e, "cudaMemPoolSetAccess");
                }
            }
            // without peer access the driver stages the copy; either way the pair is settled
            sp.peer_on[dst_device] = true;
        }
    }
    e = cudaSetDevice(dst_device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    if (dst_device == src_device) {
        // a plain device copy (also what a stream capture accepts)
        e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync");
        return TTB_OK;
    }
    e = cudaMemcpyPeerAsync(dst, dst_device, src, src_device, bytes, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyPeerAsync");
    return TTB_OK;
}
