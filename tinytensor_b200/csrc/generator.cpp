// generator.cpp -- host-side restatement of tinytensor's seeded input generator, so that
// benchmarks and tests draw exactly the operands a tinytensor program would draw.
//
// Follows the reference's CPU backend:
//   Generator(seed): state = splitmix64(seed); operator() = xorshift64 (13, 7, 17)
//                                              tinytensor/tensor/random.cpp:17-59
//   a distribution call on N elements first takes N successive outputs of the caller's
//   generator, one per element in flat row-major order, and samples element i from a fresh
//   generator whose state is the i-th output     backend/cpu/distribution.cpp:31-38,
//                                              backend/cpu/kernel/distribution.hpp:27-31
//   uniform_real: mantissa bits of one draw, (bits | exponent of 1.0) - 1, scaled in T
//   normal: Box-Muller from two such draws (sqrt(-2 log1p(-u1)) * sin(2 pi u2)), in T
//   uniform_int: Lemire's multiply-shift rejection on 64-bit draws, in T
//                                              backend/common/kernel/distribution.hpp:63-129, :234-245
// The floating-point expressions are written the way the reference writes them and compiled
// with the same contraction setting as its release build, and use the same libm calls
// (log1p, sin, sqrt in T), so the values are bit-identical to the reference library built on
// the same toolchain (pinned by tests against the reference itself and by golden vectors).
// Host memory only; nothing here touches a device.
#include <algorithm>
#include <bit>
#include <cmath>
#include <cstdint>
#include <limits>
#include <numbers>
#include <thread>
#include <type_traits>
#include <vector>

#include "../../include/ttb.h"

namespace {

uint64_t splitmix64(uint64_t seed) {
    uint64_t r = seed + 0x9E3779B97f4A7C15ull;
    r = (r ^ (r >> 30)) * 0xBF58476D1CE4E5B9ull;
    r = (r ^ (r >> 27)) * 0x94D049BB133111EBull;
    return r ^ (r >> 31);
}

inline uint64_t xorshift64(uint64_t &state) {
    uint64_t x = state;
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    state = x;
    return x;
}

template <typename T>
struct FloatBits;
template <>
struct FloatBits<float> {
    using U = uint32_t;
    static constexpr U one = static_cast<U>(127) << 23;
    static constexpr int shift = 9;
};
template <>
struct FloatBits<double> {
    using U = uint64_t;
    static constexpr U one = static_cast<U>(1023) << 52;
    static constexpr int shift = 12;
};

template <typename T>
inline T uniform_sample(T low, T high, uint64_t &state) {
    using U = typename FloatBits<T>::U;
    const T r = std::bit_cast<T>(static_cast<U>((static_cast<U>(xorshift64(state)) >> FloatBits<T>::shift) |
                                                FloatBits<T>::one)) -
                static_cast<T>(1.0);
    return r * (high - low) + low;
}

template <typename T>
inline T normal_sample(T mu, T sd, uint64_t &state) {
    const T u1 = uniform_sample(static_cast<T>(0), static_cast<T>(1), state);
    const T u2 = uniform_sample(static_cast<T>(0), static_cast<T>(1), state);
    const T r = std::sqrt(static_cast<T>(-2) * std::log1p(-u1));
    const T theta = static_cast<T>(2) * std::numbers::pi_v<T> * u2;
    const T z1 = r * std::sin(theta);
    return sd * z1 + mu;
}

inline uint64_t rand_in_range(uint64_t s, uint64_t &state) {
    __uint128_t m = static_cast<__uint128_t>(xorshift64(state)) * static_cast<__uint128_t>(s);
    auto l = static_cast<uint64_t>(m);
    if (l < s) {
        const uint64_t t = -s % s;
        while (l < t) {
            m = static_cast<__uint128_t>(xorshift64(state)) * static_cast<__uint128_t>(s);
            l = static_cast<uint64_t>(m);
        }
    }
    return static_cast<uint64_t>(m >> 64);
}

template <typename T>
inline T int_sample(T low, T high, uint64_t &state) {
    const auto range = static_cast<uint64_t>(high - low);
    const auto x = static_cast<T>(rand_in_range(range, state));
    return static_cast<T>(x + low);
}

// Element i is sampled from the i-th output of the caller's generator; the outputs are taken
// sequentially, the sampling runs over a few host threads.
template <typename T, typename F>
void fill(uint64_t *state, int64_t n, T *out, F &&sample) {
    std::vector<uint64_t> states(static_cast<std::size_t>(n));
    uint64_t s = *state;
    for (int64_t i = 0; i < n; ++i) states[static_cast<std::size_t>(i)] = xorshift64(s);
    *state = s;
    const int64_t grain = 1 << 16;
    const int threads = static_cast<int>(std::clamp<int64_t>(
        std::min<int64_t>(n / grain, std::thread::hardware_concurrency()), 1, 16));
    auto work = [&](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) {
            uint64_t st = states[static_cast<std::size_t>(i)];
            out[i] = sample(st);
        }
    };
    if (threads == 1) {
        work(0, n);
        return;
    }
    std::vector<std::thread> pool;
    const int64_t per = (n + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        const int64_t lo = t * per, hi = std::min<int64_t>(n, lo + per);
        if (lo < hi) pool.emplace_back(work, lo, hi);
    }
    for (auto &th : pool) th.join();
}

bool bad(const uint64_t *state, int64_t n, const void *out) { return state == nullptr || out == nullptr || n < 0; }

}    // namespace

extern "C" {

TTB_API uint64_t ttb_generator_seed(uint64_t seed) { return splitmix64(seed); }

TTB_API uint64_t ttb_generator_next(uint64_t *state) { return state ? xorshift64(*state) : 0; }

TTB_API int ttb_generator_uniform_real(uint64_t *state, double low, double high, int64_t n, int dtype, void *out) {
    if (bad(state, n, out) || !(low < high)) return TTB_EINVAL;
    if (dtype == TTB_F64) {
        fill(state, n, static_cast<double *>(out), [=](uint64_t &st) { return uniform_sample<double>(low, high, st); });
    } else if (dtype == TTB_F32) {
        const float lo = static_cast<float>(low), hi = static_cast<float>(high);
        fill(state, n, static_cast<float *>(out), [=](uint64_t &st) { return uniform_sample<float>(lo, hi, st); });
    } else {
        return TTB_EDTYPE;
    }
    return TTB_OK;
}

TTB_API int ttb_generator_normal(uint64_t *state, double mu, double sd, int64_t n, int dtype, void *out) {
    if (bad(state, n, out)) return TTB_EINVAL;
    if (dtype == TTB_F64) {
        fill(state, n, static_cast<double *>(out), [=](uint64_t &st) { return normal_sample<double>(mu, sd, st); });
    } else if (dtype == TTB_F32) {
        const float m = static_cast<float>(mu), s = static_cast<float>(sd);
        fill(state, n, static_cast<float *>(out), [=](uint64_t &st) { return normal_sample<float>(m, s, st); });
    } else {
        return TTB_EDTYPE;
    }
    return TTB_OK;
}

TTB_API int ttb_generator_uniform_int(uint64_t *state, int64_t low, int64_t high, int64_t n, int dtype, void *out) {
    if (bad(state, n, out) || !(low < high)) return TTB_EINVAL;
    // The reference promotes u8 / i16 requests to i32 (the result type is the promotion of the
    // bounds' type with its default integer type, tinytensor/tensor/tensor.cpp:1803-1819), so
    // only the two types it really samples in exist here; a caller narrows afterwards.
    switch (dtype) {
    case TTB_I32: {
        const auto lo = static_cast<int32_t>(low), hi = static_cast<int32_t>(high);
        fill(state, n, static_cast<int32_t *>(out), [=](uint64_t &st) { return int_sample<int32_t>(lo, hi, st); });
        break;
    }
    case TTB_I64:
        fill(state, n, static_cast<int64_t *>(out), [=](uint64_t &st) { return int_sample<int64_t>(low, high, st); });
        break;
    default:
        return TTB_EDTYPE;
    }
    return TTB_OK;
}

}    // extern "C"
