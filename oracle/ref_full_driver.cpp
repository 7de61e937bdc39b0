// ref_full_driver.cpp -- C entry points around the REFERENCE's own public API, CPU backend.
//
// TEST INFRASTRUCTURE ONLY.  No arithmetic of its own: it is linked against the unmodified
// reference library (oracle/_ref/tt_cpu/libtinytensor.a, built by oracle/dropin.mk from the
// reference tree where it lies) and calls
//   tinytensor::matmul            (tinytensor/tensor/tensor.cpp:2390-2484): rank plumbing,
//                                 dtype promotion, bool rejection, shape errors;
//   Tensor::backward              (tensor.cpp:1192-1209) through TensorBatchedMatmul::backward
//                                 (tinytensor/autograd/binary_ops.cpp:173-179): the gradients;
//   Generator, uniform_real, normal, uniform_int (tinytensor/tensor/random.cpp:26-59,
//                                 include/tt/tensor.h:1964-2003, :2204-2210): seeded inputs.
// The result, oracle/_ref/libttref_full.so, pins the Python mirror of the rank plumbing and
// of the gradients, and the restated input generator, to the reference itself.
#include <tt/grad_mode.h>
#include <tt/tensor.h>
#include <tt/tinytensor.h>

#include <cstdint>
#include <cstring>
#include <optional>
#include <string>
#include <vector>

using namespace tinytensor;

namespace {
constexpr int kOk = 0;
constexpr int kThrew = 1;       // a TTException, message in `err`
constexpr int kBadArg = 2;      // misuse of this driver

void put_error(char *err, int errlen, const std::string &msg) {
    if (err != nullptr && errlen > 0) {
        std::strncpy(err, msg.c_str(), static_cast<std::size_t>(errlen - 1));
        err[errlen - 1] = '\0';
    }
}

template <typename F>
auto by_dtype(int dtype, F &&f) {
    switch (static_cast<ScalarType>(dtype)) {
    case kBool: return f.template operator()<bool>();
    case kU8: return f.template operator()<uint8_t>();
    case kI16: return f.template operator()<int16_t>();
    case kI32: return f.template operator()<int32_t>();
    case kI64: return f.template operator()<int64_t>();
    case kF32: return f.template operator()<float>();
    default: return f.template operator()<double>();
    }
}

// A contiguous tensor of `shape` from raw host data.  bool data arrives as one byte per element.
Tensor make(int dtype, const void *data, int ndim, const int *shape, bool requires_grad) {
    std::vector<int> dims(shape, shape + ndim);
    int64_t n = 1;
    for (int d : dims) n *= d;
    Tensor t = by_dtype(dtype, [&]<typename T>() -> Tensor {
        if constexpr (std::is_same_v<T, bool>) {
            const auto *p = static_cast<const uint8_t *>(data);
            std::vector<bool> v(static_cast<std::size_t>(n));
            for (int64_t i = 0; i < n; ++i) v[static_cast<std::size_t>(i)] = p[i] != 0;
            return Tensor(v, Shape(dims), kCPU, false);
        } else {
            const auto *p = static_cast<const T *>(data);
            return Tensor(std::vector<T>(p, p + n), Shape(dims), kCPU, requires_grad);
        }
    });
    return t;
}

// The view Tensor::permute makes (shape and stride entries swapped, no copy); null = as is.
Tensor view_of(const Tensor &t, int ndim, const int *perm) {
    if (perm == nullptr) return t;
    return t.permute(std::vector<int>(perm, perm + ndim));
}

void copy_out(const Tensor &t, void *out) {
    by_dtype(static_cast<int>(t.dtype()), [&]<typename T>() {
        if constexpr (std::is_same_v<T, bool>) {
            const auto v = t.to_vec<bool>();
            auto *p = static_cast<uint8_t *>(out);
            for (std::size_t i = 0; i < v.size(); ++i) p[i] = v[i] ? 1 : 0;
        } else {
            const auto v = t.to_vec<T>();
            std::memcpy(out, v.data(), v.size() * sizeof(T));
        }
    });
}
}    // namespace

#define EXPORT extern "C" __attribute__((visibility("default")))

// out = matmul(view(a), view(b)).  `out` must hold out_capacity bytes; the result's rank,
// shape and dtype come back through out_ndim / out_shape[<=3] / out_dtype.
EXPORT int ttref_full_matmul(int a_dtype, const void *a, int a_ndim, const int *a_shape, const int *a_perm,
                             int b_dtype, const void *b, int b_ndim, const int *b_shape, const int *b_perm,
                             void *out, int64_t out_capacity, int *out_ndim, int *out_shape, int *out_dtype,
                             char *err, int errlen) {
    try {
        const autograd::NoGradGuard guard;
        const Tensor ta = make(a_dtype, a, a_ndim, a_shape, false);
        const Tensor tb = make(b_dtype, b, b_ndim, b_shape, false);
        const Tensor r = matmul(view_of(ta, a_ndim, a_perm), view_of(tb, b_ndim, b_perm));
        const int64_t bytes = static_cast<int64_t>(r.numel()) *
                              by_dtype(static_cast<int>(r.dtype()), []<typename T>() -> int64_t { return sizeof(T); });
        if (bytes > out_capacity || r.dim() > 3) {
            put_error(err, errlen, "output buffer too small");
            return kBadArg;
        }
        *out_ndim = r.dim();
        for (int d = 0; d < r.dim(); ++d) out_shape[d] = r.size(d);
        *out_dtype = static_cast<int>(r.dtype());
        copy_out(r, out);
        return kOk;
    } catch (const TTException &e) {
        put_error(err, errlen, e.what());
        return kThrew;
    }
}

// r = matmul(view(a), view(b)); r.backward(grad_out); grad_a, grad_b = a.grad, b.grad in the
// leaves' own (unpermuted, contiguous) layout.  One floating-point dtype for all tensors.
EXPORT int ttref_full_matmul_backward(int dtype, const void *a, int a_ndim, const int *a_shape, const int *a_perm,
                                      const void *b, int b_ndim, const int *b_shape, const int *b_perm,
                                      const void *grad_out, void *grad_a, void *grad_b, char *err, int errlen) {
    try {
        Tensor ta = make(dtype, a, a_ndim, a_shape, true);
        Tensor tb = make(dtype, b, b_ndim, b_shape, true);
        Tensor r = matmul(view_of(ta, a_ndim, a_perm), view_of(tb, b_ndim, b_perm));
        std::vector<int> rs;
        for (int d = 0; d < r.dim(); ++d) rs.push_back(r.size(d));
        if (rs.empty()) rs.push_back(1);
        const Tensor g = make(dtype, grad_out, static_cast<int>(rs.size()), rs.data(), false).reshape(r.shape());
        r.backward(g);
        if (!ta.grad() || !tb.grad()) {
            put_error(err, errlen, "no gradient was produced");
            return kBadArg;
        }
        copy_out(*ta.grad(), grad_a);
        copy_out(*tb.grad(), grad_b);
        return kOk;
    } catch (const TTException &e) {
        put_error(err, errlen, e.what());
        return kThrew;
    }
}

// ---- the reference's Generator and the three distributions the benchmark inputs use ----
EXPORT void *ttref_gen_new(uint64_t seed) { return new Generator(seed); }
EXPORT void ttref_gen_free(void *gen) { delete static_cast<Generator *>(gen); }
EXPORT uint64_t ttref_gen_next(void *gen) { return (*static_cast<Generator *>(gen))(); }

namespace {
template <typename F>
int draw(void *out, int dtype, char *err, int errlen, F &&f) {
    try {
        const autograd::NoGradGuard guard;
        const Tensor t = f();
        if (static_cast<int>(t.dtype()) != dtype) {    // the reference promoted the request
            put_error(err, errlen, "result dtype " + to_string(t.dtype()) + " differs from the requested one");
            return kBadArg;
        }
        copy_out(t, out);
        return kOk;
    } catch (const TTException &e) {
        put_error(err, errlen, e.what());
        return kThrew;
    }
}
}    // namespace

EXPORT int ttref_uniform_real(void *gen, double lo, double hi, int n, int dtype, void *out, char *err, int errlen) {
    return draw(out, dtype, err, errlen, [&] {
        return uniform_real(lo, hi, Shape({n}), TensorOptions().dtype(static_cast<ScalarType>(dtype)),
                            *static_cast<Generator *>(gen));
    });
}
EXPORT int ttref_normal(void *gen, double mu, double sd, int n, int dtype, void *out, char *err, int errlen) {
    return draw(out, dtype, err, errlen, [&] {
        return normal(mu, sd, Shape({n}), TensorOptions().dtype(static_cast<ScalarType>(dtype)),
                      *static_cast<Generator *>(gen));
    });
}
EXPORT int ttref_uniform_int(void *gen, int64_t lo, int64_t hi, int n, int dtype, void *out, char *err, int errlen) {
    return draw(out, dtype, err, errlen, [&] {
        return uniform_int(lo, hi, Shape({n}), TensorOptions().dtype(static_cast<ScalarType>(dtype)),
                           *static_cast<Generator *>(gen));
    });
}
