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
}  // namespace

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
    return 0;
}

}  // namespace ttb
