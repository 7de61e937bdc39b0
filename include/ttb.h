/* ttb.h -- C ABI of the B200 (sm_100a) matmul backend for tinytensor.
 *
 * Every entry point takes plain pointers and sizes; nothing here depends on
 * tinytensor, torch or C++.  The library (libttb.so) is what a tinytensor
 * build links in place of its CUDA matmul translation unit
 * (tinytensor/tensor/backend/cuda/matmul.cu); the C++ shim that adapts
 * `Tensor` to these calls lives in tinytensor_b200/csrc/tt_runner_shim.cu.
 *
 * Naming follows the reference: lhs[B,N,K] . rhs[B,K,M] -> out[B,N,M]
 * (tinytensor/autograd/binary_ops.cpp:162-164).
 */
#ifndef TTB_H_
#define TTB_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define TTB_API __attribute__((visibility("default")))
#else
#define TTB_API
#endif

/* Element types.  Values equal tinytensor::ScalarType (include/tt/scalar.h:21-29)
 * so the shim can pass `static_cast<int>(tensor.dtype())` straight through.
 * bool8 (0) never reaches the backend (tinytensor/tensor/tensor.cpp:2395-2397)
 * and is rejected with TTB_EDTYPE. */
enum ttb_dtype {
    TTB_BOOL8 = 0,
    TTB_U8 = 1,
    TTB_I16 = 2,
    TTB_I32 = 3,
    TTB_I64 = 4,
    TTB_F32 = 5,
    TTB_F64 = 6
};

/* Status codes.  0 is success; negatives are errors with a message in
 * ttb_last_error().  The reference throws TTException for user errors
 * (include/tt/exception.h:15-25) and exits on launch failure
 * (backend/cuda/kernel_launch.cuh:25-28); the shim maps any non-zero status to
 * TT_EXCEPTION. */
enum ttb_status {
    TTB_OK = 0,
    TTB_EINVAL = -1,       /* null pointer, negative stride/offset, bad option */
    TTB_ESHAPE = -2,       /* rank/inner-dim/batch mismatch, size < 1, overflow */
    TTB_EDTYPE = -3,       /* bool8 or unknown dtype */
    TTB_EDEVICE = -4,      /* device id out of range */
    TTB_ECUDA = -5,        /* a CUDA runtime/driver call failed */
    TTB_ETIMEOUT = -6,     /* a bounded device-side wait gave up */
    TTB_ENOMEM = -7,       /* workspace allocation failed */
    TTB_EUNSUPPORTED = -8, /* forced kernel variant cannot take these views */
    TTB_ELIMIT = -9        /* size beyond a documented fixed limit */
};

/* A strided rank-3 view, exactly the fields tinytensor's Tensor carries
 * (include/tt/tensor.h:1570-1577): element offset into the storage, shape and
 * element strides (0 allowed, negative never -- tinytensor/tensor/index.cpp:21-25).
 * `data` is the storage base (DeviceMemory<T>::data_ptr(),
 * backend/cuda/matmul.cu:54-57); the first element is data + offset. */
typedef struct ttb_view {
    const void *data;
    int64_t offset;
    int64_t size[3];
    int64_t stride[3];
} ttb_view;

/* Kernel variants, reported by ttb_last_variant() and forced by the
 * "force_variant" option. */
enum ttb_variant {
    TTB_VARIANT_AUTO = 0,
    TTB_VARIANT_SIMT = 1,         /* CUDA-core register-tiled kernel, any dtype/stride */
    TTB_VARIANT_TCGEN05_3XTF32 = 2, /* f32: tcgen05 + TMEM + TMA, split precision, one CTA per tile */
    TTB_VARIANT_DMMA_F64 = 3,     /* f64: FP64 tensor-core (DMMA) kernel */
    TTB_VARIANT_SIMT_SPLITK = 4,  /* SIMT with K split over CTAs + scratch reduce */
    TTB_VARIANT_TCGEN05_2CTA = 5, /* f32: tcgen05 cta_group::2 (CTA pairs) */
    TTB_VARIANT_TCGEN05_I8LIMB = 6, /* i32: exact mod 2^32 from ten u8 x u8 tcgen05 products of byte planes */
    TTB_VARIANT_SIMT_SKINNY = 7   /* one dim <= 16: streaming CUDA-core kernels (reported only; not forceable) */
};

/* ---- the hot path -------------------------------------------------------
 *
 * ttb_batched_matmul: out[b] = lhs[b] . rhs[b] on device `device_id`, queued
 * on `stream` (a cudaStream_t; NULL = the legacy default stream, which is what
 * the reference launches on, backend/cuda/kernel_launch.cuh:24).  All pointers
 * are device pointers.  `out` receives a contiguous row-major [B,N,M] result
 * with offset 0, the layout the reference allocates (backend/cuda/matmul.cu:50,74).
 * Views may be arbitrarily strided; no contiguous copy is made.
 * Replaces: tinytensor::cuda::batched_matmul_runner's contiguous()+launch
 * (backend/cuda/matmul.cu:26-78) and matmul_kernel<T>
 * (backend/cuda/kernel/matmul.cuh:27-151).
 * Does not synchronise (neither does the reference). */
TTB_API int ttb_batched_matmul(const ttb_view *lhs, const ttb_view *rhs, void *out,
                               int dtype, int device_id, void *stream);

/* Same product, but the result goes to a strided destination
 * out[b*out_stride[0] + i*out_stride[1] + j*out_stride[2]] (+ out_offset).
 * Used by the multi-GPU partitioner to write an output-column block straight
 * into its place in the full row-major C.  No counterpart in the reference
 * (its output is always fresh and contiguous). */
TTB_API int ttb_batched_matmul_strided_out(const ttb_view *lhs, const ttb_view *rhs,
                                           void *out, int64_t out_offset,
                                           const int64_t out_stride[3], int dtype,
                                           int device_id, void *stream);

/* Activations of the fused form below. */
enum ttb_activation {
    TTB_ACT_NONE = 0,
    TTB_ACT_RELU = 1   /* max(x, 0) as the reference's OpReLU (backend/common/kernel/unary.hpp:403-407):
                          NaN and -0.0 pass through; floating-point dtypes only, as there */
};

/* Product with a fused epilogue: out = act(lhs . rhs + addend), written to the
 * strided destination like ttb_batched_matmul_strided_out.  `addend` (NULL = none)
 * is a [B,N,M] view of the same dtype; any of its strides may be 0, so it can be
 *   - a bias over output columns, stride {0,0,1}: tinytensor's Linear,
 *     `matmul(x, w) + bias.expand(...)` (nn/linear.cpp:45-48), in one kernel instead
 *     of a matmul, an expand and a binary add kernel;
 *   - a bias over output rows, stride {0,1,0}: the per-channel bias of conv2d's
 *     GEMM (backend/cuda/conv.cu:149-183);
 *   - the destination itself (same pointer, offset and strides): accumulation
 *     out += lhs . rhs, what backward's add_grad does with a second kernel
 *     (tensor/tensor.cpp:1137-1160).  Each element is read and written by the
 *     same thread, so this in-place form is safe; any other overlap of `addend`
 *     with `out` is not.
 * Integers wrap exactly as a separate add in T would; for floats the addend is
 * added to the fp32 / fp64 sum before the one rounding of the store.
 * `activation` is a ttb_activation; TTB_ACT_RELU needs a floating-point dtype
 * (the reference's relu on integers yields floats, backend/common/unary.h:187). */
TTB_API int ttb_batched_matmul_fused(const ttb_view *lhs, const ttb_view *rhs, void *out,
                                     int64_t out_offset, const int64_t out_stride[3],
                                     const ttb_view *addend, int activation, int dtype,
                                     int device_id, void *stream);

/* Product fused with an all-gather of the result over NVLink (f32, tensor-core
 * kernel only).  Computes lhs . rhs into the strided destination `out` on this GPU
 * like ttb_batched_matmul_strided_out, and stores every finished tile into the
 * same place (same out_offset, same strides) of each of the `n_peers` buffers
 * peer_out[i]: device pointers to the other GPUs' C that are mapped into this
 * process (peer access, symmetric memory, IPC).  The peer stores are plain
 * st.global issued by dedicated warps of the GEMM kernel, so the exchange
 * overlaps the math tile by tile.  When the kernel has completed on every
 * rank, and the ranks have then synchronised with each other (the caller's
 * job: e.g. a symmetric-memory or NCCL barrier on the same stream), every
 * rank holds the complete C.  n_peers == 0 degenerates to the plain product.
 * Every peer_out[i] must be aligned like `out` modulo 16 bytes (TTB_EINVAL otherwise).
 * Ordering across ranks is the caller's: besides the barrier AFTER the product, no rank
 * may start the next product into the same C while another rank still reads the
 * previous result from its copy (a barrier before the launch, or two C buffers used in
 * turn -- tinytensor_b200/partition.py does the latter).
 * No counterpart in the reference (single-device matmul, host-bounce copies
 * between devices, autograd/unary_ops.cpp:67-83). */
TTB_API int ttb_matmul_allgather(const ttb_view *lhs, const ttb_view *rhs, void *out,
                                 int64_t out_offset, const int64_t out_stride[3],
                                 void *const *peer_out, int n_peers, int dtype,
                                 int device_id, void *stream);

/* The same fused product + all-gather through NVSwitch multicast.  `multicast_out` is
 * the multicast address of C: a virtual address bound (cuMulticastBindMem / a
 * symmetric-memory allocator) to the C buffers of ALL participating GPUs, laid out like
 * `out` (same out_offset and strides).  The kernel stores every finished tile once, with
 * multimem.st, to that address; the switch delivers it to every GPU, this one included,
 * so a GPU sends each byte of its block once instead of once per peer.  `out` (this
 * GPU's own mapping of C) is only used to describe the layout.  Needs row-contiguous,
 * 16-byte-aligned rows of C and a column count that is a multiple of 4; otherwise
 * TTB_EUNSUPPORTED (use ttb_matmul_allgather).  Completion as there: kernel done on
 * every rank, then a cross-rank barrier.  No counterpart in the reference. */
TTB_API int ttb_matmul_allgather_multicast(const ttb_view *lhs, const ttb_view *rhs, void *out,
                                           int64_t out_offset, const int64_t out_stride[3],
                                           void *multicast_out, int dtype, int device_id,
                                           void *stream);

/* Host-buffer form: lhs/rhs `data` and `out` are HOST pointers (pinned memory
 * makes the copies asynchronous).  Copies the operands' storage spans to the
 * device, runs ttb_batched_matmul on `device_id`, copies the contiguous result
 * back and synchronises.  Device staging buffers are cached per device and
 * grown on demand.  Large products are pipelined over three streams so that
 * upload, product and download overlap: a single product (B == 1, rhs rows
 * contiguous) in up to 8 blocks of output columns, a batched one (B >= 4,
 * batch-major operands) in groups of batches.  Calls for one device are serialised
 * (a second host thread waits until the first call has returned).  This is the call a CPU-resident caller makes, the
 * equivalent of tinytensor's `matmul(a.to(cuda), b.to(cuda)).to(cpu)`
 * (autograd/unary_ops.cpp:67-83 + backend/cuda/matmul.cu:26-78). */
TTB_API int ttb_batched_matmul_host(const ttb_view *lhs, const ttb_view *rhs, void *out,
                                    int dtype, int device_id);

/* The same product for callers that must not allocate device memory.
 * Has no counterpart in the reference, whose runner allocates on every call
 * (backend/cuda/matmul.cu:50).
 *
 * Some programs cannot let a library call cudaMalloc: they have given all
 * device memory to an allocator of their own or run under a fixed memory
 * budget, so an allocation from in here would fail or break that budget; or
 * they sit in a latency-critical loop and cannot take the device-wide
 * synchronisation that cudaMalloc and cudaFree bring.  The other entry points
 * may grow a cached workspace when they split K; this one never allocates
 * (no cudaMalloc, cudaFree or allocating library routine): it always runs the
 * CUDA-core kernel with K split over thread blocks and keeps the partial sums
 * in a 16 MiB array that is part of the library's device image (every GPU
 * on which the image is loaded holds those 16 MiB until the process exits).
 *
 * Limit: 2 * B * N * M * sizeof(element) must not exceed 16 MiB, otherwise
 * TTB_ELIMIT with a message naming both sizes; nothing is launched then.
 * All dtypes and all strides are accepted; `out` is contiguous [B,N,M].
 *
 * The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress), which also makes the driver load the library's
 * device image there -- the moment the 16 MiB are taken from that GPU.  So
 * make that first call early: before the program hands the remaining device
 * memory to its own allocator (afterwards the image might not fit), and
 * before starting any stream capture.  All calls on a device share the one
 * array: two calls whose kernels may overlap on the GPU (different streams,
 * no ordering between them) race on it and give wrong results -- keep calls
 * on one stream or order them with events.  The array keeps whatever the
 * last call left in it; no clearing is needed, because a call overwrites
 * every partial sum it later reads.  The calling thread's current device is
 * left as it was. */
TTB_API int ttb_batched_matmul_static_scratch(const ttb_view *lhs, const ttb_view *rhs,
                                              void *out, int dtype, int device_id,
                                              void *stream);

/* ---- conv2d on the matmul path -------------------------------------------
 *
 * The other caller of the reference's matmul kernel: conv2d forward and backward
 * (backend/cuda/conv.cu:37-197 and :199-403) unroll one batch item at a time and run
 * matmul_kernel<T> on it.  These two entry points replace
 * tinytensor::cuda::batched_conv2d_forward_runner / batched_conv2d_backward_runner
 * (backend/cuda/conv.h:16-30): the whole batch is unrolled by one kernel and each
 * product is one batched matmul through the same dispatch as ttb_batched_matmul
 * (bias fused into the forward product's epilogue).
 *
 * Tensors are contiguous, as the reference requires (it calls contiguous() on the
 * input, conv.cu:77): input [batch, c_in, h_in, w_in], weight [c_out, c_in, kernel,
 * kernel], bias [c_out] or NULL, out / grad_out [batch, c_out, h_out, w_out] with
 * h_out = (h_in + 2*padding - kernel) / stride + 1 (likewise w_out).  All device
 * pointers to the first element, one dtype (any but bool8).  Integers wrap like the
 * reference's; f32 / f64 meet the matmul tolerances.  The unrolled columns live in a
 * cached workspace (at most 2 GiB; larger batches are processed in groups of batch
 * items).  Neither call synchronises. */
typedef struct ttb_conv2d_desc {
    int64_t batch, c_in, h_in, w_in;
    int64_t c_out, kernel, stride, padding;
} ttb_conv2d_desc;

TTB_API int ttb_conv2d_forward(const void *input, const void *weight, const void *bias, void *out,
                               const ttb_conv2d_desc *desc, int dtype, int device_id, void *stream);

/* grad_input [batch, c_in, h_in, w_in] and grad_weight [c_out, c_in, kernel, kernel] are
 * overwritten; grad_bias [c_out] is written when not NULL (the reference returns it only
 * when the forward had a bias, conv.cu:396-399). */
TTB_API int ttb_conv2d_backward(const void *grad_out, const void *input, const void *weight,
                                void *grad_input, void *grad_weight, void *grad_bias,
                                const ttb_conv2d_desc *desc, int dtype, int device_id, void *stream);

/* ---- multi-GPU partitioner (host logic only; no communication) ----------
 *
 * Splits lhs[B,N,K].rhs[B,K,M] over `world` GPUs the way the partitioner
 * does: B > 1 -> contiguous batch ranges (no exchange step); B == 1 ->
 * output-column blocks of rhs/out rounded to `col_align` columns (an
 * all-gather of C follows).  Writes this rank's half-open range to
 * [*begin, *end) and returns 0 for batch sharding, 1 for column sharding,
 * or a negative status.  Ranks past the end of the work get an empty range.
 * No counterpart in the reference (single-device matmul only). */
TTB_API int ttb_partition(int64_t B, int64_t N, int64_t K, int64_t M, int world, int rank,
                          int64_t col_align, int64_t *begin, int64_t *end);

/* ---- device memory ------------------------------------------------------ */

/* Stream-ordered cached allocation: replaces the cudaMalloc / cudaFree pair of
 * DeviceMemory<T> (backend/cuda/data_types.cu:38-50, 102-116), each of which
 * synchronises the whole device.  Blocks come from one CUDA memory pool per
 * device that never shrinks by itself, so a freed block is handed to the next
 * request on that stream without a driver call or a synchronisation.  `*ptr`
 * may be used by work enqueued on `stream` after this call; use on another
 * stream needs the usual event ordering.  bytes == 0 gives a null pointer and
 * TTB_OK.  `stream` is a cudaStream_t of `device_id` (NULL = legacy default).
 * TTB_ENOMEM when the device is out of memory. */
TTB_API int ttb_device_alloc(void **ptr, uint64_t bytes, int device_id, void *stream);
/* Returns the block to the pool once the work already enqueued on `stream` has
 * finished.  NULL is a no-op; a pointer this library did not hand out (or a
 * second free) is TTB_EINVAL. */
TTB_API int ttb_device_free(void *ptr, int device_id, void *stream);
/* Byte counters of ttb_device_alloc on `device_id`, mirroring
 * StorageCUDA::current_bytes_allocated / total_bytes_allocated
 * (backend/cuda/storage_cuda.h:66-67): bytes handed out and not yet freed, bytes ever
 * handed out, and what the pool holds from the driver (live + cached).  Any
 * out-pointer may be NULL. */
TTB_API int ttb_device_memory_stats(int device_id, uint64_t *current_bytes, uint64_t *total_bytes,
                                    uint64_t *reserved_bytes);
/* Synchronises `device_id` and gives all cached (free) blocks back to the driver. */
TTB_API int ttb_device_trim(int device_id);
/* dst[0..bytes) on `dst_device` = src[0..bytes) on `src_device`, enqueued on
 * `stream` (a stream of dst_device, NULL = legacy default): one peer copy,
 * direct over NVLink where the devices can map each other (peer access is
 * switched on at the first copy of a pair), instead of the reference's
 * device -> host vector -> device bounce of Tensor::to(Device)
 * (autograd/unary_ops.cpp:67-83).  Same device: a plain device copy.
 * The copy is ordered on `stream` only: work of src_device that produces `src`
 * on another stream must be ordered before it by the caller (an event).
 * Like the other device-memory calls it leaves the calling thread's current
 * device as it found it. */
TTB_API int ttb_copy_device_to_device(void *dst, int dst_device, const void *src, int src_device, uint64_t bytes,
                                      void *stream);

/* ---- seeded inputs (host only) ------------------------------------------
 *
 * tinytensor's own random generator, restated so that a benchmark or test
 * draws exactly the operands a tinytensor program would draw from
 * Generator(seed) (tinytensor/tensor/random.cpp:17-59: splitmix64 of the seed
 * gives the state, xorshift64 the outputs).  `*state` is the generator; it
 * advances by n outputs per distribution call, as the reference's does: a call
 * on n elements takes n successive outputs, one per element in flat row-major
 * order, and samples element i from a fresh generator whose state is the i-th
 * output (backend/cpu/distribution.cpp:31-38, backend/cpu/kernel/distribution.hpp:27-31).
 * The three distributions are the reference's uniform_real(low, high, shape),
 * normal(mu, std, shape) and uniform_int(low, high, shape) on its CPU backend
 * (include/tt/tensor.h:1964-2003, :2204-2210; kernels
 * backend/common/kernel/distribution.hpp:63-129, :234-245): [low, high) in both
 * uniform forms.  `out` is HOST memory for n elements of `dtype` (f32 / f64 for
 * the real-valued ones; i32 / i64 for uniform_int, the reference promotes narrower
 * integer requests to i32, tensor.cpp:1803-1819).  Values are
 * bit-identical to the reference library built with the same compiler and libm. */
TTB_API uint64_t ttb_generator_seed(uint64_t seed);
TTB_API uint64_t ttb_generator_next(uint64_t *state);
TTB_API int ttb_generator_uniform_real(uint64_t *state, double low, double high, int64_t n, int dtype, void *out);
TTB_API int ttb_generator_normal(uint64_t *state, double mu, double sd, int64_t n, int dtype, void *out);
TTB_API int ttb_generator_uniform_int(uint64_t *state, int64_t low, int64_t high, int64_t n, int dtype, void *out);

/* ---- introspection / control ------------------------------------------- */

/* Message of the last failing call on this thread ("" if none). */
TTB_API const char *ttb_last_error(void);
/* Variant the last successful ttb_batched_matmul on this thread launched. */
TTB_API int ttb_last_variant(void);
/* Number of kernels this library has launched on this thread since load. */
TTB_API int64_t ttb_launch_count(void);
TTB_API const char *ttb_variant_name(int variant);
/* Workspaces.  The CUDA-core kernels' K-split partial sums and conv2d's unrolled columns,
 * weight-gradient partials and padded weights live in cached buffers keyed by
 * (device, stream), grown with cudaMalloc on demand; calls on different streams never
 * share one.  A call that would have to grow its buffer while its stream is being
 * captured into a CUDA graph is refused (TTB_EUNSUPPORTED): make the same call once
 * before the capture.  Buffers a captured launch has used are never freed. */

/* Options: "force_variant" (enum ttb_variant; AUTO restores dispatch),
 * "tf32_terms" (how the f32 tensor-core kernel reaches fp32-class accuracy:
 * 2 = hybrid split, default: one TF32 product of the operands' high parts plus
 * two bf16 products that add the low-part corrections; 3 = classic 3xTF32;
 * 1 = a single TF32 pass, test only -- it misses the 1e-5 gate),
 * "k_chunk" (32-element K blocks accumulated inside the tensor core before the
 * partial sum is folded into fp32 registers; 0 = default of 8, -1 = whole K,
 * test only), "two_cta" (automatic dispatch: -1 = pick the CTA-pair kernel by
 * shape, default; 0 = never; 1 = always),
 * "splitk" (0 = never split K in the SIMT kernel), "mask_big" (test only),
 * "tc_profile" (1 = record wait-cycle counters, see ttb_tc_profile; 2 = the CTA lifetimes only, which
 *              costs the kernel nothing),
 * "streamk" (f32 tensor-core kernel: deal the K blocks of all tiles out evenly
 * over the SMs instead of whole tiles; -1 = when whole tiles would leave SMs
 * idle, default; 0 = never; 1 = whenever possible),
 * "int_tensor" (1, default: large TMA-eligible i32 products run on the int8
 * tensor cores as ten byte-plane products, exact mod 2^32; 0 = always the
 * CUDA-core kernel), "conv_columns_mb" (budget in MiB of conv2d's unrolled
 * columns workspace, default 2048; larger batches are processed in groups),
 * "peer_tma" (1, default: ttb_matmul_allgather reaches the peers with bulk
 * tensor stores issued by the epilogue; 0: dedicated warps copy finished tiles
 * with st.global),
 * "a_tmem" (0, default; 1: the f32 kernel's correction products read their A operands from
 * tensor memory, where the converters put them, instead of shared memory -- measured: no
 * faster, the pair form then has room for one accumulator only),
 * "extra_conv" (1, default: the two spare warps of the f32 pair kernel convert 5/8 of every
 * rhs tile; 0: converter warpgroup only),
 * "sk_pair" (-1, default: with a fused all-gather; 0 never; 1 whenever stream-K cuts tiles and every
 * unit's range is a tile long: odd units walk their K-block range backwards and the two units
 * that share a tile settle by ticket which of them adds the other's sums and stores, so half
 * as many tiles complete at the very end of the kernel, where the fused all-gather has nothing
 * left to hide their exchange behind -- measured at 8 GPUs: 0.568 instead of 0.671 ms per step),
 * "pieces" (-1 / 0, default: off; n >= 2: the f32 tensor-core kernel cuts every tile's K range into
 * the largest power of two of equal parts not above n and deals the parts out round-robin, so
 * that tiles complete all through the kernel; the part that arrives last adds all parts in part
 * order, so results do not depend on timing -- measured: the hand-overs cost 15 % and more, so
 * nothing selects it by itself),
 * "tc_debug" (bit mask of timing / fault-handling experiments of the f32
 * tensor-core kernel, test only: results are wrong or absent when set).
 * Returns TTB_EINVAL for an unknown key or value. */
TTB_API int ttb_set_option(const char *key, int64_t value);
TTB_API int64_t ttb_get_option(const char *key);
/* Number of visible CUDA devices, or a negative status. */
TTB_API int ttb_device_count(void);
/* Reads and clears the device-side error word of `device_id` (set when a
 * bounded wait inside a kernel gave up).  Synchronises the device.
 * Returns TTB_OK, TTB_ETIMEOUT, or another negative status. */
TTB_API int ttb_check_device(int device_id);
/* Tracing aid for the f32 tensor-core kernel.  With the "tc_profile" option
 * set to 1, every CTA of that kernel records eight cycle counters: time its
 * TMA producer waited for a free shared-memory slot, its MMA thread for a
 * free accumulator and for converted tiles, its first converter thread for a
 * free small-tile slot, for TMA data, and spent converting, its first epilogue
 * warp for a finished accumulator, and the CTA's lifetime.  Copies the
 * counters of the first `ctas` CTAs (8 values each) of the last such launch
 * into `out`; synchronises the device.  The reference has no tracing at all
 * (only a Graphviz dump of the autograd graph, tensor.cpp:3225). */
TTB_API int ttb_tc_profile(int device_id, int64_t *out, int ctas);
/* 1 if this view can be fed to the tensor-core kernels through a TMA
 * descriptor (16-byte aligned base, unit stride on one matrix dim, other
 * byte strides multiples of 16), else 0; `operand` 0 = lhs, 1 = rhs.
 * Host-only, touches no device. */
TTB_API int ttb_view_tma_eligible(const ttb_view *v, int dtype, int operand);
/* Tensor maps (TMA descriptors) are built from a view's pointer, extents and strides and kept
 * in a per-thread cache keyed by exactly those, so a product that comes back with the same
 * views encodes nothing.  Hits and misses of the calling thread since load; either may be NULL.
 * The reference has no descriptors (its kernel takes contiguous operands only). */
TTB_API void ttb_tensor_map_cache_stats(uint64_t *hits, uint64_t *misses);
/* Measures the FP64 tensor-core (DMMA) rate of `device_id` with a register-only loop of the
 * f64 kernel's own MMA instruction (no memory traffic) and returns it in TFLOP/s: the ceiling
 * the f64 kernel's roofline fraction is quoted against.  Takes a few milliseconds and
 * synchronises.  The reference has no such probe (it publishes no performance figures). */
TTB_API int ttb_measure_fp64_tensor_peak(int device_id, double *tflops);
TTB_API int ttb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* TTB_H_ */
