// conv2d.cu -- conv2d forward / backward on top of the batched matmul path.
//
// The reference runs, per batch item, an unroll (im2col) kernel, matmul_kernel<T> and a
// separate bias add (backend/cuda/conv.cu:37-197), and for backward an unroll-transpose, two
// matmuls, an accumulation kernel and a col2im whose threads add into shared pixels
// (conv.cu:199-403, kernel/conv.cuh:93-133).  Here the whole batch is unrolled by one launch
// into columns[B][C_in*K*K][H_out*W_out] and each of the three products is ONE batched matmul
// through the same dispatch as ttb_batched_matmul (tcgen05 for f32, DMMA for f64, the CUDA-core
// kernel for integers):
//   forward : out[b]      = W[C_out, CKK] . columns[b]            + bias (fused row addend)
//   grad_w  : part[b]     = g_out[b][C_out, HW] . columns[b]^T    (a permuted view, no transpose
//                           kernel), then summed over b in ascending order like the reference
//   grad_x  : columns[b]  = W^T[CKK, C_out] . g_out[b]            (permuted view of W), then a
//                           col2im in gather form: one thread per input pixel adds its <= K*K
//                           contributions in (p, q) order, the order the reference's CPU loop
//                           adds them in, without atomics or races.
// All kernels here are HBM-bound copies / short sums; their algorithmic bytes are the tensors
// they read and write once.
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "common.cuh"

namespace ttb {

int workspace_slot(int device, cudaStream_t stream, int slot, size_t bytes, void **out);
int dispatch_problem(const Problem &p);
size_t conv_columns_budget();

namespace {

struct ConvGeom {
    int C_in, H_in, W_in, C_out, K, S, P, H_out, W_out;
    long long rows;   // C_in * K * K
    long long hw;     // H_out * W_out
    long long pitch;  // row pitch of the columns buffer, elements (hw rounded up)
};

// Unsigned type of the same width for wrap-around integer sums; floats add as themselves.
template <typename T, bool FP = std::is_floating_point_v<T>>
struct SumOf {
    using type = T;
};
template <typename T>
struct SumOf<T, false> {
    using type = std::make_unsigned_t<T>;
};

// Four elements moved as one (16 bytes for 4-byte types; 8-byte types take two 16-byte stores).
template <typename U>
struct alignas(sizeof(U) * 4 <= 16 ? sizeof(U) * 4 : 16) Vec4 {
    U v[4];
};

// columns[bz][c*K*K + p*K + q][hw] = x[b0 + bz][c][S*h + p - P][S*w + q - P] or 0 outside the
// image.  grid: (blocks of 256 x 4 output pixels, C_in, batch items of this group).  A thread owns
// four consecutive output pixels: it derives their (h, w) once, then walks the K*K rows of its
// channel, writing one aligned vector per row (the row pitch is a multiple of 32 elements, so
// the vector never crosses a row; pixels past H_out*W_out land in the pitch padding as zeros).
// Pure data movement, so it is instantiated per element size only.
template <typename U>
__global__ void __launch_bounds__(256) im2col_kernel(const U *__restrict__ x, U *__restrict__ cols, ConvGeom g,
                                                     long long b0) {
    const long long hw0 = (static_cast<long long>(blockIdx.x) * 256 + threadIdx.x) * 4;
    if (hw0 >= g.hw) return;
    int hs[4], ws[4];
    bool live[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const long long hw = hw0 + j;
        live[j] = hw < g.hw;
        hs[j] = static_cast<int>(hw / g.W_out) * g.S - g.P;
        ws[j] = static_cast<int>(hw % g.W_out) * g.S - g.P;
    }
    const int c = blockIdx.y;
    const long long bz = blockIdx.z;
    const U *xc = x + ((b0 + bz) * g.C_in + c) * static_cast<long long>(g.H_in) * g.W_in;
    U *cr = cols + (bz * g.rows + static_cast<long long>(c) * g.K * g.K) * g.pitch + hw0;
    for (int p = 0; p < g.K; ++p) {
        for (int q = 0; q < g.K; ++q) {
            Vec4<U> out;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int h_in = hs[j] + p, w_in = ws[j] + q;
                const bool inside = live[j] && h_in >= 0 && w_in >= 0 && h_in < g.H_in && w_in < g.W_in;
                out.v[j] = inside ? xc[static_cast<long long>(h_in) * g.W_in + w_in] : U(0);
            }
            *reinterpret_cast<Vec4<U> *>(cr) = out;
            cr += g.pitch;
        }
    }
}

// grad_x[b][c][hi][wi] = sum over (p, q), ascending, of columns[b][c*KK + p*K + q][h*W_out + w]
// with S*h + p - P == hi and S*w + q - P == wi.  UNIT: stride 1 (no division per tap); KT: the
// kernel size when it is one of the usual ones (3, 5), else 0 and the taps are walked in a loop.
template <typename T, bool UNIT, int KT>
__global__ void __launch_bounds__(256) col2im_kernel(const T *__restrict__ cols, T *__restrict__ gx, ConvGeom g,
                                                     long long b0) {
    using A = typename SumOf<T>::type;
    const int pix = blockIdx.x * 256 + threadIdx.x;  // grid: (pixel blocks, C_in, batch items of this group)
    if (pix >= g.H_in * g.W_in) return;
    const int hi = pix / g.W_in, wi = pix % g.W_in;
    const int c = blockIdx.y;
    const long long bz = blockIdx.z;
    const T *cb = cols + (bz * g.rows + static_cast<long long>(c) * g.K * g.K) * g.pitch;
    A s = A(0);
    if constexpr (KT > 0) {
        // Kernel size known at compile time: all K*K loads are issued before the first add (a
        // thread keeps K*K requests in flight instead of one), then added in (p, q) order.
        T v[KT > 0 ? KT * KT : 1];
        bool ok[KT > 0 ? KT * KT : 1];
#pragma unroll
        for (int p = 0; p < KT; ++p) {
            const int hh = hi + g.P - p;
            const int h = UNIT ? hh : hh / g.S;
            const bool row_ok = hh >= 0 && (UNIT || hh % g.S == 0) && h < g.H_out;
#pragma unroll
            for (int q = 0; q < KT; ++q) {
                const int ww = wi + g.P - q;
                const int w = UNIT ? ww : ww / g.S;
                const bool take = row_ok && ww >= 0 && (UNIT || ww % g.S == 0) && w < g.W_out;
                ok[p * KT + q] = take;
                v[p * KT + q] = take ? cb[static_cast<long long>(p * KT + q) * g.pitch + static_cast<long long>(h) * g.W_out + w]
                                     : T(0);
            }
        }
#pragma unroll
        for (int t = 0; t < KT * KT; ++t)
            if (ok[t]) s = s + static_cast<A>(v[t]);
        gx[(((b0 + bz) * g.C_in + c) * g.H_in + hi) * static_cast<long long>(g.W_in) + wi] = static_cast<T>(s);
        return;
    }
    for (int p = 0; p < g.K; ++p) {
        const int hh = hi + g.P - p;
        if (hh < 0) break;  // larger p only lowers hh
        int h = hh;
        if (!UNIT) {
            if (hh % g.S != 0) continue;
            h = hh / g.S;
        }
        if (h >= g.H_out) continue;
        const T *row = cb + static_cast<long long>(p) * g.K * g.pitch + static_cast<long long>(h) * g.W_out;
        for (int q = 0; q < g.K; ++q) {
            const int ww = wi + g.P - q;
            if (ww < 0) break;
            int w = ww;
            if (!UNIT) {
                if (ww % g.S != 0) continue;
                w = ww / g.S;
            }
            if (w >= g.W_out) continue;
            s = s + static_cast<A>(row[static_cast<long long>(q) * g.pitch + w]);
        }
    }
    gx[(((b0 + bz) * g.C_in + c) * g.H_in + hi) * static_cast<long long>(g.W_in) + wi] = static_cast<T>(s);
}

// out[i] = (accumulate ? out[i] : 0) + part[0][i] + part[1][i] + ... in that order.
template <typename T>
__global__ void __launch_bounds__(256) sum_parts_kernel(const T *__restrict__ part, T *__restrict__ out, long long n,
                                                        int parts, int accumulate) {
    using A = typename SumOf<T>::type;
    const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= n) return;
    A s = accumulate ? static_cast<A>(out[i]) : A(0);
    for (int b = 0; b < parts; ++b) s = s + static_cast<A>(part[b * n + i]);
    out[i] = static_cast<T>(s);
}

// part[b][m] = sum over h, w of g_out[b][m][h][w]: one CTA per (channel, batch item); the batch
// items are then added in ascending order by sum_parts_kernel.  Integers wrap; a float row is
// summed in double and rounded once.
template <typename T>
__global__ void __launch_bounds__(256) channel_sum_kernel(const T *__restrict__ go, T *__restrict__ part,
                                                          long long C_out, long long hw) {
    using A = std::conditional_t<std::is_floating_point_v<T>, double, typename SumOf<T>::type>;
    __shared__ A red[256];
    const long long m = blockIdx.x, b = blockIdx.y;
    const T *src = go + (b * C_out + m) * hw;
    A s = A(0);
    for (long long i = threadIdx.x; i < hw; i += 256) s = s + static_cast<A>(src[i]);
    red[threadIdx.x] = s;
    __syncthreads();
    for (int step = 128; step > 0; step >>= 1) {
        if (threadIdx.x < step) red[threadIdx.x] = red[threadIdx.x] + red[threadIdx.x + step];
        __syncthreads();
    }
    if (threadIdx.x == 0) part[b * C_out + m] = static_cast<T>(red[0]);
}

// dst[r][0..cols) = src[r][0..cols), row pitch `pitch` (>= cols); the padding is zeroed.
template <typename U>
__global__ void __launch_bounds__(256) pad_rows_kernel(const U *__restrict__ src, U *__restrict__ dst, long long rows,
                                                       long long cols, long long pitch) {
    const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= rows * pitch) return;
    const long long r = i / pitch, c = i % pitch;
    dst[i] = c < cols ? src[r * cols + c] : U(0);
}

template <typename U>
int launch_im2col(const void *x, void *cols, const ConvGeom &g, long long b0, long long nb, cudaStream_t st) {
    dim3 grid(static_cast<unsigned>((g.hw + 1023) / 1024), static_cast<unsigned>(g.C_in), static_cast<unsigned>(nb));
    im2col_kernel<U><<<grid, 256, 0, st>>>(static_cast<const U *>(x), static_cast<U *>(cols), g, b0);
    cudaError_t e = cudaGetLastError();
    note_launch(-1, 1);
    return e == cudaSuccess ? TTB_OK : cuda_fail(e, "im2col_kernel launch");
}

int im2col(const void *x, void *cols, const ConvGeom &g, long long b0, long long nb, size_t es, cudaStream_t st) {
    switch (es) {
        case 1: return launch_im2col<uint8_t>(x, cols, g, b0, nb, st);
        case 2: return launch_im2col<uint16_t>(x, cols, g, b0, nb, st);
        case 4: return launch_im2col<uint32_t>(x, cols, g, b0, nb, st);
        default: return launch_im2col<uint64_t>(x, cols, g, b0, nb, st);
    }
}

template <typename T>
int typed_col2im(const void *cols, void *gx, const ConvGeom &g, long long b0, long long nb, cudaStream_t st) {
    dim3 grid(static_cast<unsigned>((static_cast<long long>(g.H_in) * g.W_in + 255) / 256),
              static_cast<unsigned>(g.C_in), static_cast<unsigned>(nb));
    const T *src = static_cast<const T *>(cols);
    T *dst = static_cast<T *>(gx);
    if (g.S == 1) {
        if (g.K == 3)
            col2im_kernel<T, true, 3><<<grid, 256, 0, st>>>(src, dst, g, b0);
        else if (g.K == 5)
            col2im_kernel<T, true, 5><<<grid, 256, 0, st>>>(src, dst, g, b0);
        else
            col2im_kernel<T, true, 0><<<grid, 256, 0, st>>>(src, dst, g, b0);
    } else {
        if (g.K == 3)
            col2im_kernel<T, false, 3><<<grid, 256, 0, st>>>(src, dst, g, b0);
        else if (g.K == 5)
            col2im_kernel<T, false, 5><<<grid, 256, 0, st>>>(src, dst, g, b0);
        else
            col2im_kernel<T, false, 0><<<grid, 256, 0, st>>>(src, dst, g, b0);
    }
    cudaError_t e = cudaGetLastError();
    note_launch(-1, 1);
    return e == cudaSuccess ? TTB_OK : cuda_fail(e, "col2im_kernel launch");
}

template <typename T>
int typed_sum_parts(const void *part, void *out, long long n, int parts, int accumulate, cudaStream_t st) {
    sum_parts_kernel<T><<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(static_cast<const T *>(part),
                                                                                static_cast<T *>(out), n, parts,
                                                                                accumulate);
    cudaError_t e = cudaGetLastError();
    note_launch(-1, 1);
    return e == cudaSuccess ? TTB_OK : cuda_fail(e, "sum_parts_kernel launch");
}

template <typename T>
int typed_channel_sum(const void *go, void *part, long long B, long long C_out, long long hw, cudaStream_t st) {
    dim3 grid(static_cast<unsigned>(C_out), static_cast<unsigned>(B));
    channel_sum_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T *>(go), static_cast<T *>(part), C_out, hw);
    cudaError_t e = cudaGetLastError();
    note_launch(-1, 1);
    return e == cudaSuccess ? TTB_OK : cuda_fail(e, "channel_sum_kernel launch");
}

#define TTB_BY_DTYPE(dtype, fn, ...)                                     \
    ((dtype) == TTB_U8    ? fn<uint8_t>(__VA_ARGS__)                     \
     : (dtype) == TTB_I16 ? fn<int16_t>(__VA_ARGS__)                     \
     : (dtype) == TTB_I32 ? fn<int32_t>(__VA_ARGS__)                     \
     : (dtype) == TTB_I64 ? fn<int64_t>(__VA_ARGS__)                     \
     : (dtype) == TTB_F32 ? fn<float>(__VA_ARGS__)                       \
                          : fn<double>(__VA_ARGS__))

// Checks the description and derives the geometry.
int make_geom(const ttb_conv2d_desc *d, int dtype, ConvGeom *g, size_t *es) {
    if (!d) {
        set_error("conv2d: null description");
        return TTB_EINVAL;
    }
    *es = dtype_size(dtype);
    if (dtype == TTB_BOOL8 || *es == 0) {
        set_error("conv2d: unsupported dtype %d", dtype);
        return TTB_EDTYPE;
    }
    if (d->batch < 1 || d->c_in < 1 || d->c_out < 1 || d->h_in < 1 || d->w_in < 1 || d->kernel < 1 ||
        d->stride < 1 || d->padding < 0) {
        set_error("conv2d: sizes must be >= 1 (stride >= 1, padding >= 0)");
        return TTB_ESHAPE;
    }
    const long long h_out = (d->h_in + 2 * d->padding - d->kernel) / d->stride + 1;
    const long long w_out = (d->w_in + 2 * d->padding - d->kernel) / d->stride + 1;
    if (d->h_in + 2 * d->padding < d->kernel || d->w_in + 2 * d->padding < d->kernel || h_out < 1 || w_out < 1) {
        set_error("conv2d: kernel %lld does not fit the padded %lldx%lld image", static_cast<long long>(d->kernel),
                  static_cast<long long>(d->h_in + 2 * d->padding), static_cast<long long>(d->w_in + 2 * d->padding));
        return TTB_ESHAPE;
    }
    // The reference indexes every tensor with `int` (kernel/conv.cuh:27-46).
    const long double lim = 2147483647.0L;
    if (static_cast<long double>(d->batch) * d->c_in * d->h_in * d->w_in > lim ||
        static_cast<long double>(d->batch) * d->c_out * h_out * w_out > lim ||
        static_cast<long double>(d->c_in) * d->kernel * d->kernel * h_out * w_out > lim) {
        set_error("conv2d: tensor sizes beyond 2^31 - 1 elements");
        return TTB_ELIMIT;
    }
    if (d->c_in > 65535 || d->c_out > 65535) {
        set_error("conv2d: more than 65535 channels");
        return TTB_ELIMIT;
    }
    g->C_in = static_cast<int>(d->c_in);
    g->H_in = static_cast<int>(d->h_in);
    g->W_in = static_cast<int>(d->w_in);
    g->C_out = static_cast<int>(d->c_out);
    g->K = static_cast<int>(d->kernel);
    g->S = static_cast<int>(d->stride);
    g->P = static_cast<int>(d->padding);
    g->H_out = static_cast<int>(h_out);
    g->W_out = static_cast<int>(w_out);
    g->rows = static_cast<long long>(d->c_in) * d->kernel * d->kernel;
    g->hw = h_out * w_out;
    g->pitch = (g->hw + 31) / 32 * 32;  // 128-byte rows for f32: every row start is TMA- and vector-aligned
    return TTB_OK;
}

// Batch items per chunk so that the columns buffer stays within the workspace budget (option
// "conv_columns_mb", 2 GiB by default; one batch item is always allowed).
long long chunk_batches(const ConvGeom &g, long long B, size_t es) {
    const size_t per = static_cast<size_t>(g.rows) * g.pitch * es;
    long long nb = static_cast<long long>(conv_columns_budget() / (per ? per : 1));
    if (nb < 1) nb = 1;
    if (nb > 65535) nb = 65535;  // batch items of a group are grid.z of the unroll kernels
    return nb < B ? nb : B;
}

int select_device(int device) {
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceCount");
    if (device < 0 || device >= ndev) {
        set_error("device id %d out of range (have %d)", device, ndev);
        return TTB_EDEVICE;
    }
    e = cudaSetDevice(device);
    return e == cudaSuccess ? TTB_OK : cuda_fail(e, "cudaSetDevice");
}

// Weight rows for the tensor-core path: TMA needs a 16-byte row pitch, so an f32 weight
// matrix whose row length C_in*K*K is not a multiple of 4 is copied once into padded rows.
int weight_rows(const void *weight, const ConvGeom &g, int dtype, int device, cudaStream_t st, const void **w,
                long long *w_pitch) {
    *w = weight;
    *w_pitch = g.rows;
    if (dtype != TTB_F32 || (g.rows & 3) == 0) return TTB_OK;
    const long long pitch = (g.rows + 3) / 4 * 4;
    void *buf = nullptr;
    int rc = workspace_slot(device, st, 3, static_cast<size_t>(g.C_out) * pitch * 4, &buf);
    if (rc != TTB_OK) return rc;
    const long long n = static_cast<long long>(g.C_out) * pitch;
    pad_rows_kernel<uint32_t><<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(
        static_cast<const uint32_t *>(weight), static_cast<uint32_t *>(buf), g.C_out, g.rows, pitch);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "pad_rows_kernel launch");
    note_launch(-1, 1);
    *w = buf;
    *w_pitch = pitch;
    return TTB_OK;
}

}  // namespace
}  // namespace ttb

using namespace ttb;

extern "C" TTB_API int ttb_conv2d_forward(const void *input, const void *weight, const void *bias, void *out,
                                          const ttb_conv2d_desc *desc, int dtype, int device_id, void *stream) {
    ConvGeom g{};
    size_t es = 0;
    int rc = make_geom(desc, dtype, &g, &es);
    if (rc != TTB_OK) return rc;
    if (!input || !weight || !out) {
        set_error("conv2d forward: null pointer");
        return TTB_EINVAL;
    }
    rc = select_device(device_id);
    if (rc != TTB_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long B = desc->batch;
    const long long nb_max = chunk_batches(g, B, es);
    void *cols = nullptr;
    rc = workspace_slot(device_id, st, 1, static_cast<size_t>(nb_max) * g.rows * g.pitch * es, &cols);
    if (rc != TTB_OK) return rc;
    const void *w = nullptr;
    long long w_pitch = 0;
    rc = weight_rows(weight, g, dtype, device_id, st, &w, &w_pitch);
    if (rc != TTB_OK) return rc;
    for (long long b0 = 0; b0 < B; b0 += nb_max) {
        const long long nb = b0 + nb_max <= B ? nb_max : B - b0;
        rc = im2col(input, cols, g, b0, nb, es, st);
        if (rc != TTB_OK) return rc;
        Problem p{};
        p.a = w;  // the same weight matrix for every batch item: batch stride 0
        p.a_sb = 0;
        p.a_si = w_pitch;
        p.a_sk = 1;
        p.b = cols;
        p.b_sb = g.rows * g.pitch;
        p.b_sk = g.pitch;
        p.b_sj = 1;
        p.c = static_cast<char *>(out) + static_cast<size_t>(b0) * g.C_out * g.hw * es;
        p.c_sb = g.C_out * g.hw;
        p.c_si = g.hw;
        p.c_sj = 1;
        p.B = nb;
        p.N = g.C_out;
        p.K = g.rows;
        p.M = g.hw;
        p.dtype = dtype;
        p.device = device_id;
        p.stream = st;
        if (bias) {  // one value per output channel = per row of the product
            p.d = bias;
            p.d_sb = 0;
            p.d_si = 1;
            p.d_sj = 0;
        }
        rc = dispatch_problem(p);
        if (rc != TTB_OK) return rc;
    }
    return TTB_OK;
}

extern "C" TTB_API int ttb_conv2d_backward(const void *grad_out, const void *input, const void *weight,
                                           void *grad_input, void *grad_weight, void *grad_bias,
                                           const ttb_conv2d_desc *desc, int dtype, int device_id, void *stream) {
    ConvGeom g{};
    size_t es = 0;
    int rc = make_geom(desc, dtype, &g, &es);
    if (rc != TTB_OK) return rc;
    if (!grad_out || !input || !weight || !grad_input || !grad_weight) {
        set_error("conv2d backward: null pointer");
        return TTB_EINVAL;
    }
    rc = select_device(device_id);
    if (rc != TTB_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long B = desc->batch;
    const long long nb_max = chunk_batches(g, B, es);
    void *cols = nullptr, *parts = nullptr;
    rc = workspace_slot(device_id, st, 1, static_cast<size_t>(nb_max) * g.rows * g.pitch * es, &cols);
    if (rc != TTB_OK) return rc;
    const long long wn = static_cast<long long>(g.C_out) * g.rows;
    // also holds the per-item channel sums of grad_bias afterwards
    const long long parts_elems = nb_max * wn > B * g.C_out ? nb_max * wn : B * g.C_out;
    rc = workspace_slot(device_id, st, 2, static_cast<size_t>(parts_elems) * es, &parts);
    if (rc != TTB_OK) return rc;
    const void *w = nullptr;
    long long w_pitch = 0;
    rc = weight_rows(weight, g, dtype, device_id, st, &w, &w_pitch);
    if (rc != TTB_OK) return rc;
    for (long long b0 = 0; b0 < B; b0 += nb_max) {
        const long long nb = b0 + nb_max <= B ? nb_max : B - b0;
        const char *go = static_cast<const char *>(grad_out) + static_cast<size_t>(b0) * g.C_out * g.hw * es;
        // grad_w partials: g_out[b][C_out, HW] . columns[b]^T[HW, CKK]
        rc = im2col(input, cols, g, b0, nb, es, st);
        if (rc != TTB_OK) return rc;
        Problem p{};
        p.dtype = dtype;
        p.device = device_id;
        p.stream = st;
        p.B = nb;
        p.a = go;
        p.a_sb = g.C_out * g.hw;
        p.a_si = g.hw;
        p.a_sk = 1;
        p.b = cols;
        p.b_sb = g.rows * g.pitch;
        p.b_sk = 1;        // columns^T: k walks along a row of the columns buffer,
        p.b_sj = g.pitch;  // j from row to row
        p.c = parts;
        p.c_sb = wn;
        p.c_si = g.rows;
        p.c_sj = 1;
        p.N = g.C_out;
        p.K = g.hw;
        p.M = g.rows;
        rc = dispatch_problem(p);
        if (rc != TTB_OK) return rc;
        rc = TTB_BY_DTYPE(dtype, typed_sum_parts, parts, grad_weight, wn, static_cast<int>(nb), b0 > 0 ? 1 : 0, st);
        if (rc != TTB_OK) return rc;
        // grad_x columns: W^T[CKK, C_out] . g_out[b][C_out, HW], overwriting the columns buffer
        Problem q{};
        q.dtype = dtype;
        q.device = device_id;
        q.stream = st;
        q.B = nb;
        q.a = w;
        q.a_sb = 0;
        q.a_si = 1;  // W^T as a permuted view of W[C_out, CKK]
        q.a_sk = w_pitch;
        q.b = go;
        q.b_sb = g.C_out * g.hw;
        q.b_sk = g.hw;
        q.b_sj = 1;
        q.c = cols;
        q.c_sb = g.rows * g.pitch;
        q.c_si = g.pitch;
        q.c_sj = 1;
        q.N = g.rows;
        q.K = g.C_out;
        q.M = g.hw;
        rc = dispatch_problem(q);
        if (rc != TTB_OK) return rc;
        rc = TTB_BY_DTYPE(dtype, typed_col2im, cols, grad_input, g, b0, nb, st);
        if (rc != TTB_OK) return rc;
    }
    if (grad_bias) {
        rc = TTB_BY_DTYPE(dtype, typed_channel_sum, grad_out, parts, B, static_cast<long long>(g.C_out), g.hw, st);
        if (rc != TTB_OK) return rc;
        rc = TTB_BY_DTYPE(dtype, typed_sum_parts, parts, grad_bias, static_cast<long long>(g.C_out), static_cast<int>(B),
                          0, st);
        if (rc != TTB_OK) return rc;
    }
    return TTB_OK;
}
