// tma_desc.cu -- stride -> TMA tensor-map builder (host side).
#include "tma_desc.cuh"

#include <cstdio>
#include <mutex>

namespace ttb {

namespace {
using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up through the runtime, so the library does
// not link against libcuda directly.
EncodeFn get_encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
        if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeFn>(p);
    });
    return fn;
}

// Cache of encoded tensor maps.  A map is a pure function of (first element, extents, strides,
// element type and size, box, major); products that come back with the same views -- a training
// loop's weights and activations, a captured sequence replayed call by call -- would otherwise
// pay three driver encodes per call.  Direct-mapped and per thread: no lock, a collision just
// re-encodes.  (A freed and re-allocated buffer at the same address with the same shape gives
// the same map, which is still the right one.)
struct MapKey {
    const void *ptr;
    int64_t mn, k, batch, s_mn, s_k, s_b;
    int32_t major, dt, es, box_inner, box_mn_rows, box_k_rows;
    bool operator==(const MapKey &o) const {
        return ptr == o.ptr && mn == o.mn && k == o.k && batch == o.batch && s_mn == o.s_mn && s_k == o.s_k &&
               s_b == o.s_b && major == o.major && dt == o.dt && es == o.es && box_inner == o.box_inner &&
               box_mn_rows == o.box_mn_rows && box_k_rows == o.box_k_rows;
    }
};
struct MapEntry {
    bool valid = false;
    MapKey key{};
    int batch_mul = 0;
    CUtensorMap map;
};
constexpr int kMapCacheSlots = 256;
thread_local MapEntry g_map_cache[kMapCacheSlots];
thread_local uint64_t g_map_hits = 0, g_map_misses = 0;

uint32_t map_slot(const MapKey &k) {
    uint64_t h = reinterpret_cast<uintptr_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
    auto mix = [&](uint64_t v) { h = (h ^ v) * 0xBF58476D1CE4E5B9ull; h ^= h >> 29; };
    mix(static_cast<uint64_t>(k.mn));
    mix(static_cast<uint64_t>(k.k));
    mix(static_cast<uint64_t>(k.batch));
    mix(static_cast<uint64_t>(k.s_mn));
    mix(static_cast<uint64_t>(k.s_k));
    mix(static_cast<uint64_t>(k.s_b));
    mix((static_cast<uint64_t>(k.major) << 40) ^ (static_cast<uint64_t>(k.dt) << 32) ^ (static_cast<uint64_t>(k.es) << 24) ^
        (static_cast<uint64_t>(k.box_inner) << 16) ^ (static_cast<uint64_t>(k.box_mn_rows) << 8) ^
        static_cast<uint64_t>(k.box_k_rows));
    return static_cast<uint32_t>(h >> 40) % kMapCacheSlots;
}
}  // namespace

void tensor_map_cache_stats(uint64_t *hits, uint64_t *misses) {
    if (hits) *hits = g_map_hits;
    if (misses) *misses = g_map_misses;
}

OperandMajor classify_operand(const OperandView &v, size_t es, char *why, int why_len) {
    auto fail = [&](const char *msg) {
        if (why && why_len > 0) snprintf(why, why_len, "%s", msg);
        return kMajorNone;
    };
    if (reinterpret_cast<uintptr_t>(v.ptr) % 16 != 0) return fail("first element is not 16-byte aligned");
    if (v.mn > 0xFFFFFFFFLL || v.k > 0xFFFFFFFFLL || v.batch > 0xFFFFFFFFLL) return fail("extent above 2^32");
    const int64_t lim = (1LL << 40);
    auto outer_ok = [&](int64_t stride, int64_t extent) {
        if (extent == 1) return true;  // never stepped
        return stride > 0 && (stride * static_cast<int64_t>(es)) % 16 == 0 &&
               stride * static_cast<int64_t>(es) < lim;
    };
    if (v.batch > 1 && v.s_b != 0 && !outer_ok(v.s_b, v.batch)) return fail("batch stride is not a multiple of 16 bytes");
    // Prefer K-major when both dims qualify (e.g. an extent-1 dim).
    if ((v.s_k == 1 || v.k == 1) && outer_ok(v.s_mn, v.mn)) return kMajorK;
    if ((v.s_mn == 1 || v.mn == 1) && outer_ok(v.s_k, v.k)) return kMajorMN;
    if (v.s_k != 1 && v.s_mn != 1) return fail("neither matrix dim has unit stride");
    return fail("outer stride is zero or not a multiple of 16 bytes");
}

int encode_operand_tmap(CUtensorMap *map, const OperandView &v, OperandMajor major, CUtensorMapDataType dt,
                        size_t es, int box_inner, int box_mn_rows, int box_k_rows, int *batch_mul, char *why,
                        int why_len) {
    const MapKey key{v.ptr, v.mn, v.k, v.batch, v.s_mn, v.s_k, v.s_b, static_cast<int32_t>(major),
                     static_cast<int32_t>(dt), static_cast<int32_t>(es), box_inner, box_mn_rows, box_k_rows};
    MapEntry &slot = g_map_cache[map_slot(key)];
    if (slot.valid && slot.key == key) {
        *map = slot.map;
        *batch_mul = slot.batch_mul;
        ++g_map_hits;
        return 0;
    }
    ++g_map_misses;
    EncodeFn fn = get_encode_fn();
    if (!fn) {
        if (why) snprintf(why, why_len, "cuTensorMapEncodeTiled entry point not found");
        return 1;
    }
    const bool bcast = (v.batch == 1) || (v.s_b == 0);
    *batch_mul = bcast ? 0 : 1;
    cuuint64_t gdim[3];
    cuuint64_t gstr[2];
    cuuint32_t box[3];
    const cuuint32_t estr[3] = {1, 1, 1};
    // A dim of extent 1 is never stepped; its stride only has to satisfy the
    // encoder (multiple of 16, non-zero), so a safe dummy is used.
    auto stride_bytes = [&](int64_t stride, int64_t extent, uint64_t dummy) -> cuuint64_t {
        if (extent == 1 || stride == 0) return dummy;
        return static_cast<cuuint64_t>(stride) * es;
    };
    if (major == kMajorK) {
        gdim[0] = static_cast<cuuint64_t>(v.k);
        gdim[1] = static_cast<cuuint64_t>(v.mn);
        const uint64_t row_dummy = ((static_cast<uint64_t>(v.k) * es + 15) / 16) * 16;
        gstr[0] = stride_bytes(v.s_mn, v.mn, row_dummy);
        box[0] = static_cast<cuuint32_t>(box_inner);
        box[1] = static_cast<cuuint32_t>(box_mn_rows);
    } else {
        gdim[0] = static_cast<cuuint64_t>(v.mn);
        gdim[1] = static_cast<cuuint64_t>(v.k);
        const uint64_t row_dummy = ((static_cast<uint64_t>(v.mn) * es + 15) / 16) * 16;
        gstr[0] = stride_bytes(v.s_k, v.k, row_dummy);
        box[0] = static_cast<cuuint32_t>(box_inner);
        box[1] = static_cast<cuuint32_t>(box_k_rows);
    }
    gdim[2] = bcast ? 1 : static_cast<cuuint64_t>(v.batch);
    gstr[1] = bcast ? gstr[0] * gdim[1] : static_cast<cuuint64_t>(v.s_b) * es;
    box[2] = 1;
    // K-major tiles use the ordinary 128-byte swizzle (16-byte chunks).  MN-major tiles of
    // 32-bit elements must use the 128-byte swizzle with 32-byte chunks: it is the only
    // shared-memory layout tcgen05.mma accepts for MN-major tf32 operands.
    const CUtensorMapSwizzle swz =
        (major == kMajorMN && es == 4) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
    CUresult r = fn(map, dt, 3, const_cast<void *>(v.ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        if (why)
            snprintf(why, why_len, "cuTensorMapEncodeTiled failed with %d (dims %llu,%llu,%llu strides %llu,%llu)",
                     static_cast<int>(r), (unsigned long long)gdim[0], (unsigned long long)gdim[1],
                     (unsigned long long)gdim[2], (unsigned long long)gstr[0], (unsigned long long)gstr[1]);
        return 1;
    }
    slot.valid = true;
    slot.key = key;
    slot.batch_mul = *batch_mul;
    slot.map = *map;
    return 0;
}

}  // namespace ttb
