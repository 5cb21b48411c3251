/*
 * dwim_b200 — the block-quantized matrix product of the dwim inference engine,
 * hand-written for NVIDIA B200 (sm_100a), behind a flat C ABI.
 *
 * The entry points map one to one onto the hot-path methods of the engine's
 * `trait Device` (gpu/mod.rs:176-401): a Rust `impl Device for B200` binds
 * them with `extern "C"` and nothing else.  Each declaration names the trait
 * method or reference function it replaces.
 *
 * Conventions
 *   - Every function returns 0 on success and a negative DWIM_B200_E* code on
 *     failure; the message is kept per context (dwim_b200_last_error).  No
 *     exception crosses this boundary and nothing aborts.  (The trait's
 *     methods are infallible and panic on misuse, gpu/cuda/mod.rs:485-500: a
 *     binding turns a non-zero code into a panic.)
 *   - A context is driven by one host thread at a time, as the reference's
 *     device is (gpu/cuda/mod.rs:5-9).  All work of a context runs in order
 *     on one CUDA stream; only read, sync, dequantize and quantize wait.
 *   - Weights are GGUF blocks, row-major: rows * dwim_b200_row_bytes(fmt,
 *     cols) bytes.  Activations are f32, one row of `cols` per token;
 *     results are token-major, out[t * rows + r] (gpu/cpu.rs:144-148).
 *   - There is no CPU fallback: without a CUDA device dwim_b200_open fails.
 */
#ifndef DWIM_B200_H
#define DWIM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DWIM_B200_API __attribute__((visibility("default")))
#else
#define DWIM_B200_API
#endif

/* Weight formats, numbered as GGUF numbers its tensor types
 * (inference/gguf.rs:28-33 knows 8 and 14; 12 is new to the engine). */
enum {
    DWIM_B200_Q8_0 = 8,  /* 32 weights: f16 d, 32 x i8            (34 B)  */
    DWIM_B200_Q4_K = 12, /* 256 weights: f16 d, dmin, 12 B of 6-bit scales/mins, 128 B of nibbles (144 B) */
    DWIM_B200_Q6_K = 14, /* 256 weights: ql[128] qh[64] i8 scales[16] f16 d (210 B) */
    DWIM_B200_BF16 = 30  /* plain bf16 weights, 2 B each (Tensor::Bf16, gpu/mod.rs:46-50): the small gate matrices */
};

enum {
    DWIM_B200_OK = 0,
    DWIM_B200_EINVAL = -1,  /* a null handle, a bad shape or a bad length */
    DWIM_B200_EFORMAT = -2, /* an unknown weight format, or cols not whole blocks */
    DWIM_B200_ENOMEM = -3,  /* out of device memory */
    DWIM_B200_ECUDA = -4,   /* the CUDA runtime reported an error */
    DWIM_B200_ENODEV = -5,  /* no usable device (not sm_100) */
    DWIM_B200_ETIMEOUT = -6 /* a bounded device-side wait gave up; see dwim_b200_status */
};

typedef struct dwim_b200_ctx dwim_b200_ctx;
typedef struct dwim_b200_buffer dwim_b200_buffer;
typedef struct dwim_b200_weight dwim_b200_weight;

/* ---- the device ------------------------------------------------------- */

/* Cuda::new (gpu/cuda/mod.rs:210-238): opens device `device`, creates the
 * context's stream.  Fails with ENODEV on anything but compute capability 10.x. */
DWIM_B200_API int dwim_b200_open(int device, dwim_b200_ctx **out);
/* The same, on a stream the caller owns (a cudaStream_t; it is neither
 * synchronized against others nor destroyed here).  The reference's device runs
 * everything on one in-order stream (gpu/cuda/mod.rs:5-9, 238): an engine that
 * keeps its other operators (norms, attention, rope ...) on its own CUDA device
 * opens this library on that device's stream, and the two sets of kernels are
 * ordered as if they were one device's.  Without it, work of the caller that
 * touches a buffer of this library must be fenced against dwim_b200_stream()
 * with events. */
DWIM_B200_API int dwim_b200_open_on_stream(int device, void *cuda_stream, dwim_b200_ctx **out);
DWIM_B200_API int dwim_b200_close(dwim_b200_ctx *ctx);

/* The message of the last failure on this context ("" if none).  With a null
 * context: the last failure of dwim_b200_open on this thread. */
DWIM_B200_API const char *dwim_b200_last_error(const dwim_b200_ctx *ctx);

/* Device::name (gpu/mod.rs:188-189). */
DWIM_B200_API int dwim_b200_name(const dwim_b200_ctx *ctx, char *buf, size_t cap);
/* Device::memory (gpu/mod.rs:191-194): bytes free on the device. */
DWIM_B200_API int dwim_b200_memory(const dwim_b200_ctx *ctx, uint64_t *free_bytes);
/* Device::batch (gpu/mod.rs:196-204; 512 for the reference's CUDA device,
 * gpu/cuda/mod.rs:47-48): most tokens one matmul should be given. */
DWIM_B200_API size_t dwim_b200_batch(const dwim_b200_ctx *ctx);
/* Waits for everything queued on the context (the reference has no such
 * method: reading a buffer is its only wait, gpu/cuda/mod.rs:995-1000).
 * Returns ETIMEOUT if a kernel's bounded wait gave up since the last call. */
DWIM_B200_API int dwim_b200_sync(dwim_b200_ctx *ctx);
/* The context's cudaStream_t, for callers that record their own events. */
DWIM_B200_API void *dwim_b200_stream(const dwim_b200_ctx *ctx);
/* The status word kernels write when a bounded wait runs out: 0 = none. */
DWIM_B200_API int dwim_b200_status(dwim_b200_ctx *ctx, uint32_t *status);
/* Number of kernels this context has launched since it was opened. */
DWIM_B200_API uint64_t dwim_b200_launches(const dwim_b200_ctx *ctx);

/* Timing on the context's own stream: begin records an event, end records a
 * second one, waits for it and returns the milliseconds between them. */
DWIM_B200_API int dwim_b200_timer_begin(dwim_b200_ctx *ctx);
DWIM_B200_API int dwim_b200_timer_end(dwim_b200_ctx *ctx, float *ms);

/* ---- activations -------------------------------------------------------- */

/* Device::alloc (gpu/mod.rs:209-210): a zeroed buffer of `len` f32. */
DWIM_B200_API int dwim_b200_alloc(dwim_b200_ctx *ctx, size_t len, dwim_b200_buffer **out);
/* A buffer over device memory the caller owns (`len` f32 at `device_ptr`),
 * e.g. the receive side of an NCCL collective.  Freeing the handle leaves
 * the memory alone.  No counterpart in the reference (it is single-GPU). */
DWIM_B200_API int dwim_b200_wrap(dwim_b200_ctx *ctx, float *device_ptr, size_t len, dwim_b200_buffer **out);
/* Device::resize (gpu/mod.rs:216-219; gpu/cuda/mod.rs:986-993): sets the
 * length, up to the allocated one; never reallocates. */
DWIM_B200_API int dwim_b200_resize(dwim_b200_ctx *ctx, dwim_b200_buffer *buf, size_t len);
/* "Someone else wrote this buffer."  A buffer caches the 16-bit operand form
 * of its contents between products (after `Form`, gpu/cuda/mod.rs:108-126,
 * which the reference invalidates in its own write paths, :313-384).  This
 * library drops the cache whenever one of its own calls writes the buffer; a
 * write it cannot see (a kernel of the caller's through dwim_b200_buffer_ptr, a
 * collective into a wrapped buffer) must be followed by touch before the next
 * product reads the buffer, or that product multiplies the old contents.  It
 * also forgets that the contents were exact in 16 bits (write_bf16). */
DWIM_B200_API int dwim_b200_touch(dwim_b200_ctx *ctx, dwim_b200_buffer *buf);
/* The same, where the caller vouches that every value it wrote is exactly a
 * bf16 (the output of a bf16 kernel widened to f32): the next product then
 * carries a token as one 16-bit column instead of two, as after write_bf16.
 * A value that is not a bf16 would be rounded to f16's 11 bits, silently. */
DWIM_B200_API int dwim_b200_touch_bf16(dwim_b200_ctx *ctx, dwim_b200_buffer *buf);
/* How f32 activations reach the tensor-core kernels (products of more than
 * eight tokens; the small-M kernel's digit planes are exact either way).
 * EXACT, the default: a token travels as two f16 columns, value and rounding
 * remainder, and the product's error stays near 2e-6 of its rms; twice the
 * tensor-core work of a bf16-exact buffer.  F16: one column, the activation
 * rounded to f16 after the token's power-of-two scaling, which is the
 * precision of the reference's own CUDA device (`halves`,
 * gpu/cuda/mod.rs:313-384): rms error about 3e-4 of the result's magnitude,
 * the worst element about 3e-3 -- inside that device's gate (1e-3 and 1e-2,
 * gpu/tests.rs:198-211), outside this library's 1e-3 on the worst element --
 * at twice the rate. */
#define DWIM_B200_ACT_EXACT 0
#define DWIM_B200_ACT_F16 1
DWIM_B200_API int dwim_b200_activation_precision(dwim_b200_ctx *ctx, int mode);
/* Device::write (gpu/mod.rs:224-225): `len` must equal the buffer's length. */
DWIM_B200_API int dwim_b200_write(dwim_b200_ctx *ctx, dwim_b200_buffer *buf, const float *data, size_t len);
/* As write, from bf16 bits (gpu/float.rs:5-8): the buffer holds the same
 * values as f32 and remembers that they are exact in 16 bits. */
DWIM_B200_API int dwim_b200_write_bf16(dwim_b200_ctx *ctx, dwim_b200_buffer *buf, const uint16_t *data, size_t len);
/* Device::read (gpu/mod.rs:221-222): waits for the queued work. */
DWIM_B200_API int dwim_b200_read(dwim_b200_ctx *ctx, const dwim_b200_buffer *buf, float *out, size_t len);
DWIM_B200_API int dwim_b200_buffer_free(dwim_b200_ctx *ctx, dwim_b200_buffer *buf);
DWIM_B200_API size_t dwim_b200_buffer_len(const dwim_b200_buffer *buf);
/* The device address of the buffer's f32 data. */
DWIM_B200_API float *dwim_b200_buffer_ptr(const dwim_b200_buffer *buf);

/* ---- weights ------------------------------------------------------------ */

/* Bytes of one row of `cols` weights in GGUF layout, 0 if the format is
 * unknown or cols is not whole blocks (inference/gguf.rs:36-53). */
DWIM_B200_API size_t dwim_b200_row_bytes(int fmt, size_t cols);

/* Device::upload (gpu/mod.rs:206-207; gpu/cuda/mod.rs:905-951): copies a
 * [rows, cols] matrix of GGUF blocks to the device; the host memory is not
 * kept.  `bytes` must be rows * row_bytes. */
DWIM_B200_API int dwim_b200_upload(dwim_b200_ctx *ctx, int fmt, size_t rows, size_t cols,
                                   const void *blocks, size_t bytes, dwim_b200_weight **out);
DWIM_B200_API int dwim_b200_weight_free(dwim_b200_ctx *ctx, dwim_b200_weight *w);
DWIM_B200_API int dwim_b200_weight_shape(const dwim_b200_weight *w, int *fmt, size_t *rows, size_t *cols);

/* Tensor::dequantize (gpu/mod.rs:138-168), run on the device: `len` =
 * rows * cols f32, row-major, to host memory.  Bit-exact with the reference's
 * decoders (inference/quants.rs:59-104) — the tests' ground truth. */
DWIM_B200_API int dwim_b200_dequantize(dwim_b200_ctx *ctx, const dwim_b200_weight *w, float *out, size_t len);

/* Quantizes a host f32 [rows, cols] matrix to GGUF blocks in host memory, on
 * the device.  Q8_0 follows quantize_q8_0_row (gpu/quant.rs:31-46, 154-180);
 * the Q4_K and Q6_K quantizers have no reference counterpart. */
DWIM_B200_API int dwim_b200_quantize(dwim_b200_ctx *ctx, int fmt, size_t rows, size_t cols,
                                     const float *weights, void *blocks, size_t bytes);

/* ---- the product -------------------------------------------------------- */

/* Device::matmul (gpu/mod.rs:251-254): out[t] = w . x[t] for each of the
 * n = len(x)/cols rows of x; len(out) must be n * rows. */
DWIM_B200_API int dwim_b200_matmul(dwim_b200_ctx *ctx, dwim_b200_buffer *out,
                                   const dwim_b200_weight *w, dwim_b200_buffer *x);
/* Device::matmul_add (gpu/mod.rs:256-268): x += w . input.  `scratch` is as
 * long as x and is left undefined (it may be null: the sum is fused). */
DWIM_B200_API int dwim_b200_matmul_add(dwim_b200_ctx *ctx, dwim_b200_buffer *x, const dwim_b200_weight *w,
                                       dwim_b200_buffer *input, dwim_b200_buffer *scratch);
/* Device::swiglu (gpu/mod.rs:270-285): out = silu(gate . x) * (up . x).
 * `scratch` is as long as out and is left undefined. */
DWIM_B200_API int dwim_b200_swiglu(dwim_b200_ctx *ctx, dwim_b200_buffer *out, const dwim_b200_weight *gate,
                                   const dwim_b200_weight *up, dwim_b200_buffer *x, dwim_b200_buffer *scratch);

/* Device::normalize (gpu/mod.rs:290-305; Cuda::normalize, gpu/cuda/mod.rs:1177-1198,
 * rmsnorm.cu:11-58): out = rmsnorm(x[0..len]) * weight, rows of len(weight);
 * len(out) must be `len`.  The reference's CUDA device writes the f16 copy its
 * tile kernels read; here the same launch writes the f32 result and, where rows
 * are whole 256-weight units, the 16-bit operand form the next product of `out`
 * will read (int8 digit planes for up to eight rows, the tensor-core kernel's
 * f16 rows, means and scales above sixteen), so that no activation prologue
 * runs before that product. */
DWIM_B200_API int dwim_b200_normalize(dwim_b200_ctx *ctx, dwim_b200_buffer *out, const dwim_b200_buffer *x,
                                      const dwim_b200_buffer *weight, size_t len, float eps);
/* The first index of the largest of each of the n rows of `len` logits in
 * `logits` (n * len f32), to host memory; waits.  Replaces reading the logits
 * back and scanning them on the host (inference/qwen35/mod.rs:702-710,
 * 1066-1068: 608 KB per drafted token); NaNs never win. */
DWIM_B200_API int dwim_b200_argmax(dwim_b200_ctx *ctx, const dwim_b200_buffer *logits, size_t len, uint32_t *out,
                                   size_t n);

/* No counterpart in the reference.  out[t] = w . x[t] for n <= 8 token rows,
 * like dwim_b200_matmul, but without allocating anything: `out` (n * rows f32)
 * and `x` (n * cols f32) are device pointers the caller owns, and the 16-bit
 * operand form of x goes to a fixed 1 MiB array inside the library instead of
 * a buffer allocated on first use.  For callers whose device memory is an
 * arena sized once, or that run where cudaMalloc is not allowed.  Sizes whose
 * operand form does not fit the array are refused with EINVAL: with `units` =
 * cols / 256 rounded up, n * units may be at most 949 for one or two tokens
 * (1104 bytes of int8 digit planes per token and unit: about 243 000
 * activations per call) and 1266 for three to eight (828 bytes: about 324 000).
 * bf16 weights are not taken.  The array is shared by all calls on
 * a GPU: calls that overlap there race; calls on one context are ordered.  Its
 * device address is looked up (cudaGetSymbolAddress) when the context is
 * opened, so dwim_b200_open is the call that should come before any stream
 * capture; no call of matmul_static sets anything up. */
DWIM_B200_API int dwim_b200_matmul_static(dwim_b200_ctx *ctx, float *out, const dwim_b200_weight *w, const float *x,
                                          size_t n);

/* ---- sharding across GPUs (no counterpart in the reference) -------------- */

/* A buffer of `len` f32 that the ranks of a group (one process per GPU) share:
 * every rank allocates its copy with shared_alloc, which also writes the
 * copy's inter-process handle (dwim_b200_peer_handle_bytes() bytes); the
 * handles are exchanged by the caller's own means and given, in rank order
 * and `handle_bytes` apart, to shared_connect, which maps the peers' copies
 * (a world of 1 needs no handles).  Freed with dwim_b200_buffer_free. */
DWIM_B200_API int dwim_b200_shared_alloc(dwim_b200_ctx *ctx, size_t len, dwim_b200_buffer **out, void *handle,
                                         size_t handle_bytes);
DWIM_B200_API int dwim_b200_shared_connect(dwim_b200_ctx *ctx, dwim_b200_buffer *buf, int world, int rank,
                                           const void *handles, size_t handle_bytes);
/* The same for ranks that live in one process (one host thread driving several
 * GPUs, as the reference's server would): `copies[r]` is rank r's buffer of
 * dwim_b200_shared_alloc, of the same length (copies[rank] is ignored); the
 * pointers are used as they are, so peer access between the devices must be
 * enabled by the caller.  Ranks on one GPU may share results this way, but
 * must not call dwim_b200_shared_barrier: kernels that wait for one another
 * cannot be relied on to run together on one device. */
DWIM_B200_API int dwim_b200_shared_connect_local(dwim_b200_ctx *ctx, dwim_b200_buffer *buf, int world, int rank,
                                                 dwim_b200_buffer *const *copies);
/* The row-sharded product with the all-gather fused into it: `w` holds rows
 * [row_begin, row_begin + rows(w)) of a matrix of `total_rows`; the kernel's
 * epilogue stores out[t * total_rows + row_begin + r] = w[r] . x[t] into EVERY
 * rank's copy of the shared buffer `out` (n * total_rows f32), the peers'
 * copies by plain stores over NVLink while other tiles still multiply.  When
 * every rank has made the call and passed dwim_b200_shared_barrier(out), every
 * copy holds the full token-major result.  A copy must not be written again
 * (the next matmul_gather into it, by any rank) before its owner has finished
 * reading it: alternate two shared buffers, as a barrier lets a rank run at
 * most one step ahead of its peers. */
DWIM_B200_API int dwim_b200_matmul_gather(dwim_b200_ctx *ctx, dwim_b200_buffer *out, const dwim_b200_weight *w,
                                          dwim_b200_buffer *x, size_t row_begin, size_t total_rows);
/* One small kernel on the context's stream: tells every rank that this rank's
 * stores into the shared buffer (everything queued before the call) have
 * landed, and waits, on the device and bounded by the library's wait limit,
 * until every rank has said so.  Every rank must call it the same number of
 * times.  The barrier's count lives in device memory, so the call may be
 * captured in a CUDA graph and replayed. */
DWIM_B200_API int dwim_b200_shared_barrier(dwim_b200_ctx *ctx, dwim_b200_buffer *buf);

/* The K-sharded product with the reduction's first half fused into it: `w` holds
 * this rank's K slice of a [rows, K] matrix (all rows), `x` this rank's slice of
 * the activations; rows are owned by ranks in slices of per = ceil(rows / world).
 * The kernel's epilogue stores every partial sum into its row's owner: slot
 * `rank` of the owner's copy of the shared buffer `slots` (world * n * per f32,
 * laid out [source rank][token][row of the slice]).  After every rank's call
 * and dwim_b200_shared_barrier(slots), reduce_gather adds this rank's own rows
 * over the slots in rank order and stores the sums into every rank's copy of
 * the shared result `out` (n * rows f32, token-major); after
 * dwim_b200_shared_barrier(out) every copy holds the full sum, the same bits on
 * every rank.  Replaces an all-reduce of the n * rows partial sums. */
DWIM_B200_API int dwim_b200_matmul_scatter(dwim_b200_ctx *ctx, dwim_b200_buffer *slots, const dwim_b200_weight *w,
                                           dwim_b200_buffer *x);
DWIM_B200_API int dwim_b200_reduce_gather(dwim_b200_ctx *ctx, dwim_b200_buffer *out, const dwim_b200_buffer *slots,
                                          size_t n, size_t rows);

/* The rows rank `rank` of `world` holds when a matrix is split by output
 * rows at multiples of `align`: [*begin, *end). */
DWIM_B200_API int dwim_b200_shard_rows(size_t rows, int rank, int world, size_t align,
                                       size_t *begin, size_t *end);
/* Re-assembles an all-gathered result: `parts` holds, for each rank in turn,
 * that rank's [n, rows_of_rank] slice; `out` gets the token-major [n, rows]. */
DWIM_B200_API int dwim_b200_gather_rows(dwim_b200_ctx *ctx, dwim_b200_buffer *out, const dwim_b200_buffer *parts,
                                        size_t n, size_t rows, int world, size_t align);

/* ---- a small all-reduce over peer memory ------------------------------------
 * New (the reference engine is single-GPU): the sum of the ranks' partial
 * results of a K-sharded product (the down projection of a tensor-parallel
 * feed-forward block) for a few tokens, where a library collective's latency
 * exceeds the product's time.  One process per GPU.  peer_create allocates this
 * rank's mailbox (slots of `cap` floats) and writes its inter-process handle
 * (dwim_b200_peer_handle_bytes() bytes) to `handle`; the caller exchanges the
 * handles by its own means and passes all `world` of them, in rank order and
 * `handle_bytes` apart, to peer_connect.  peer_allreduce then replaces the first
 * n floats of `buf` on every rank by their sum over the ranks, added in rank
 * order (the same bits everywhere).  Every rank must make the same calls in the
 * same order; a rank that waits for its peers longer than the library's wait
 * limit gives up, and the next sync reports DWIM_B200_ETIMEOUT.  The call's
 * epoch is a launch argument: peer_allreduce refuses (EINVAL) while the
 * context's stream is being captured into a CUDA graph. */
DWIM_B200_API size_t dwim_b200_peer_handle_bytes(void);
DWIM_B200_API int dwim_b200_peer_create(dwim_b200_ctx *ctx, int world, int rank, size_t cap, void *handle,
                                        size_t handle_bytes);
DWIM_B200_API int dwim_b200_peer_connect(dwim_b200_ctx *ctx, const void *handles, size_t handle_bytes);
DWIM_B200_API int dwim_b200_peer_allreduce(dwim_b200_ctx *ctx, dwim_b200_buffer *buf, size_t n);

#ifdef __cplusplus
}
#endif
#endif /* DWIM_B200_H */
