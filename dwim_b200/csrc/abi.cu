// The C ABI: contexts, buffers, weights and the operator entry points.
// Declarations and their reference counterparts: include/dwim_b200.h.
#include <new>

#include "common.cuh"

using namespace dwim;

static thread_local char g_open_error[512] = "";

#define REQUIRE(ctx, cond, code, ...)                      \
    do {                                                   \
        if (!(cond)) return dwim::fail(ctx, code, __VA_ARGS__); \
    } while (0)

// Extra bytes behind every weight array: the small-M kernel's copies run in
// whole 256-weight units and may read past the last row's end.
static constexpr size_t WEIGHT_SLACK = 1024;


namespace dwim {
// gemm.cu
bool gemm_supports(const WeightView &w);
int gemm_large(dwim_b200_ctx *ctx, const WeightView &w, const __half *operand, size_t n, int split, const OutSpec &out,
               const float *aux, int epilogue);
void gemm_release(dwim_b200_ctx *ctx);
}  // namespace dwim

extern "C" {

static int open_impl(int device, cudaStream_t adopt, bool adopting, dwim_b200_ctx **out) {
    if (!out) return DWIM_B200_EINVAL;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        snprintf(g_open_error, sizeof g_open_error, "no CUDA device: %s",
                 e == cudaSuccess ? "none present" : cudaGetErrorString(e));
        return DWIM_B200_ENODEV;
    }
    if (device < 0 || device >= count) {
        snprintf(g_open_error, sizeof g_open_error, "device %d of %d does not exist", device, count);
        return DWIM_B200_ENODEV;
    }
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) {
        snprintf(g_open_error, sizeof g_open_error, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
        return DWIM_B200_ECUDA;
    }
    if (prop.major != 10) {
        snprintf(g_open_error, sizeof g_open_error, "%s is compute capability %d.%d; this library is sm_100a only",
                 prop.name, prop.major, prop.minor);
        return DWIM_B200_ENODEV;
    }
    if ((e = cudaSetDevice(device)) != cudaSuccess) {
        snprintf(g_open_error, sizeof g_open_error, "cudaSetDevice: %s", cudaGetErrorString(e));
        return DWIM_B200_ECUDA;
    }
    dwim_b200_ctx *ctx = new (std::nothrow) dwim_b200_ctx();
    if (!ctx) return DWIM_B200_ENOMEM;
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    snprintf(ctx->name, sizeof ctx->name, "%s", prop.name);
    bool ok = true;
    if (adopting) {
        ctx->stream = adopt;
        ctx->stream_owned = false;
    } else {
        ok = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) == cudaSuccess;
    }
    ok = ok && cudaEventCreate(&ctx->ev0) == cudaSuccess && cudaEventCreate(&ctx->ev1) == cudaSuccess &&
         cudaMalloc(&ctx->status, sizeof(uint32_t)) == cudaSuccess &&
         cudaMallocHost(&ctx->status_host, sizeof(uint32_t)) == cudaSuccess &&
         cudaMemset(ctx->status, 0, sizeof(uint32_t)) == cudaSuccess &&
         // the fixed scratch array of dwim_b200_matmul_static: its device address is looked up here,
         // with the device current and before anything could be capturing the stream
         static_scratch_prepare(ctx) == 0;
    if (!ok) {
        cudaError_t last = cudaGetLastError();
        if (last != cudaSuccess || !ctx->err[0])
            snprintf(g_open_error, sizeof g_open_error, "creating the context: %s", cudaGetErrorString(last));
        else
            snprintf(g_open_error, sizeof g_open_error, "creating the context: %s", ctx->err);
        dwim_b200_close(ctx);
        return DWIM_B200_ECUDA;
    }
    *out = ctx;
    return 0;
}

int dwim_b200_open(int device, dwim_b200_ctx **out) { return open_impl(device, nullptr, false, out); }

int dwim_b200_open_on_stream(int device, void *cuda_stream, dwim_b200_ctx **out) {
    return open_impl(device, static_cast<cudaStream_t>(cuda_stream), true, out);
}

int dwim_b200_close(dwim_b200_ctx *ctx) {
    DWIM_DEVICE(ctx);
    if (!ctx) return DWIM_B200_EINVAL;
    cudaSetDevice(ctx->device);
    if (ctx->stream || !ctx->stream_owned) cudaStreamSynchronize(ctx->stream);
    peer_release(ctx);
    gemm_release(ctx);
    if (ctx->ev0) cudaEventDestroy(ctx->ev0);
    if (ctx->ev1) cudaEventDestroy(ctx->ev1);
    if (ctx->argmax_dev) cudaFree(ctx->argmax_dev);
    if (ctx->argmax_host) cudaFreeHost(ctx->argmax_host);
    if (ctx->status) cudaFree(ctx->status);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    if (ctx->stream && ctx->stream_owned) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return 0;
}

const char *dwim_b200_last_error(const dwim_b200_ctx *ctx) { return ctx ? ctx->err : g_open_error; }

int dwim_b200_name(const dwim_b200_ctx *ctx, char *buf, size_t cap) {
    DWIM_DEVICE(ctx);
    if (!ctx || !buf || cap == 0) return DWIM_B200_EINVAL;
    snprintf(buf, cap, "%s", ctx->name);
    return 0;
}

int dwim_b200_memory(const dwim_b200_ctx *ctx, uint64_t *free_bytes) {
    DWIM_DEVICE(ctx);
    if (!ctx || !free_bytes) return DWIM_B200_EINVAL;
    size_t f = 0, t = 0;
    cudaSetDevice(ctx->device);
    if (cudaMemGetInfo(&f, &t) != cudaSuccess) return DWIM_B200_ECUDA;
    *free_bytes = f;
    return 0;
}

size_t dwim_b200_batch(const dwim_b200_ctx *ctx) { return ctx ? 2048 : 0; }

static int check_status(dwim_b200_ctx *ctx) {
    DWIM_CUDA(ctx, cudaMemcpyAsync(ctx->status_host, ctx->status, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    DWIM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (*ctx->status_host != 0) {
        uint32_t s = *ctx->status_host;
        cudaMemsetAsync(ctx->status, 0, sizeof(uint32_t), ctx->stream);
        return fail(ctx, DWIM_B200_ETIMEOUT, "a device-side wait gave up (status 0x%x); results are undefined", s);
    }
    return 0;
}

int dwim_b200_sync(dwim_b200_ctx *ctx) {
    DWIM_DEVICE(ctx);
    if (!ctx) return DWIM_B200_EINVAL;
    return check_status(ctx);
}

void *dwim_b200_stream(const dwim_b200_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

int dwim_b200_status(dwim_b200_ctx *ctx, uint32_t *status) {
    DWIM_DEVICE(ctx);
    if (!ctx || !status) return DWIM_B200_EINVAL;
    DWIM_CUDA(ctx, cudaMemcpyAsync(ctx->status_host, ctx->status, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    DWIM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    *status = *ctx->status_host;
    return 0;
}

uint64_t dwim_b200_launches(const dwim_b200_ctx *ctx) { return ctx ? ctx->launches : 0; }

int dwim_b200_timer_begin(dwim_b200_ctx *ctx) {
    DWIM_DEVICE(ctx);
    if (!ctx) return DWIM_B200_EINVAL;
    DWIM_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
    return 0;
}

int dwim_b200_timer_end(dwim_b200_ctx *ctx, float *ms) {
    DWIM_DEVICE(ctx);
    if (!ctx || !ms) return DWIM_B200_EINVAL;
    DWIM_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
    DWIM_CUDA(ctx, cudaEventSynchronize(ctx->ev1));
    DWIM_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev0, ctx->ev1));
    return 0;
}

// ---- buffers ----------------------------------------------------------------

int dwim_b200_alloc(dwim_b200_ctx *ctx, size_t len, dwim_b200_buffer **out) {
    DWIM_DEVICE(ctx);
    if (!ctx || !out) return DWIM_B200_EINVAL;
    *out = nullptr;
    dwim_b200_buffer *b = new (std::nothrow) dwim_b200_buffer();
    REQUIRE(ctx, b, DWIM_B200_ENOMEM, "out of host memory");
    b->len = b->cap = len;
    if (len) {
        cudaError_t e = cudaMalloc(&b->data, len * sizeof(float));
        if (e == cudaSuccess) e = cudaMemsetAsync(b->data, 0, len * sizeof(float), ctx->stream);
        if (e != cudaSuccess) {
            if (b->data) cudaFree(b->data);
            delete b;
            cudaGetLastError();
            return fail(ctx, e == cudaErrorMemoryAllocation ? DWIM_B200_ENOMEM : DWIM_B200_ECUDA,
                        "allocating %zu floats: %s", len, cudaGetErrorString(e));
        }
    }
    *out = b;
    return 0;
}

int dwim_b200_wrap(dwim_b200_ctx *ctx, float *device_ptr, size_t len, dwim_b200_buffer **out) {
    DWIM_DEVICE(ctx);
    if (!ctx || !out) return DWIM_B200_EINVAL;
    *out = nullptr;
    REQUIRE(ctx, device_ptr || len == 0, DWIM_B200_EINVAL, "wrap: null device pointer");
    REQUIRE(ctx, (reinterpret_cast<uintptr_t>(device_ptr) & 15) == 0, DWIM_B200_EINVAL, "wrap: pointer not 16-byte aligned");
    dwim_b200_buffer *b = new (std::nothrow) dwim_b200_buffer();
    REQUIRE(ctx, b, DWIM_B200_ENOMEM, "out of host memory");
    b->data = device_ptr;
    b->len = b->cap = len;
    b->owned = false;
    *out = b;
    return 0;
}

int dwim_b200_resize(dwim_b200_ctx *ctx, dwim_b200_buffer *buf, size_t len) {
    DWIM_DEVICE(ctx);
    if (!ctx || !buf) return DWIM_B200_EINVAL;
    REQUIRE(ctx, len <= buf->cap, DWIM_B200_EINVAL, "resize to %zu beyond the %zu allocated", len, buf->cap);
    buf->len = len;
    buf->shadow_kind = SHADOW_NONE;
    return 0;
}

int dwim_b200_touch(dwim_b200_ctx *ctx, dwim_b200_buffer *buf) {
    DWIM_DEVICE(ctx);
    if (!ctx || !buf) return DWIM_B200_EINVAL;
    buf->shadow_kind = SHADOW_NONE;
    buf->bf16_exact = false;
    return 0;
}

int dwim_b200_activation_precision(dwim_b200_ctx *ctx, int mode) {
    DWIM_DEVICE(ctx);
    if (!ctx) return DWIM_B200_EINVAL;
    REQUIRE(ctx, mode == DWIM_B200_ACT_EXACT || mode == DWIM_B200_ACT_F16, DWIM_B200_EINVAL, "activation precision %d", mode);
    ctx->act_f16 = mode == DWIM_B200_ACT_F16;
    return 0;
}

int dwim_b200_touch_bf16(dwim_b200_ctx *ctx, dwim_b200_buffer *buf) {
    DWIM_DEVICE(ctx);
    if (!ctx || !buf) return DWIM_B200_EINVAL;
    buf->shadow_kind = SHADOW_NONE;
    buf->bf16_exact = true;
    return 0;
}

int dwim_b200_write(dwim_b200_ctx *ctx, dwim_b200_buffer *buf, const float *data, size_t len) {
    DWIM_DEVICE(ctx);
    if (!ctx || !buf || (!data && len)) return DWIM_B200_EINVAL;
    REQUIRE(ctx, len == buf->len, DWIM_B200_EINVAL, "write of %zu floats to a buffer of %zu", len, buf->len);
    if (len) DWIM_CUDA(ctx, cudaMemcpyAsync(buf->data, data, len * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    buf->shadow_kind = SHADOW_NONE;
    buf->bf16_exact = false;
    return 0;
}

__global__ void bf16_to_f32_kernel(const uint16_t *__restrict__ in, size_t n, float *__restrict__ out) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __uint_as_float((uint32_t)in[i] << 16);   // gpu/float.rs:5-8
}

int dwim_b200_write_bf16(dwim_b200_ctx *ctx, dwim_b200_buffer *buf, const uint16_t *data, size_t len) {
    DWIM_DEVICE(ctx);
    if (!ctx || !buf || (!data && len)) return DWIM_B200_EINVAL;
    REQUIRE(ctx, len == buf->len, DWIM_B200_EINVAL, "write of %zu values to a buffer of %zu", len, buf->len);
    buf->shadow_kind = SHADOW_NONE;
    buf->bf16_exact = true;
    if (!len) return 0;
    uint16_t *staging = nullptr;
    DWIM_CUDA(ctx, cudaMallocAsync((void **)&staging, len * sizeof(uint16_t), ctx->stream));
    cudaError_t e = cudaMemcpyAsync(staging, data, len * sizeof(uint16_t), cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) {
        size_t blocks = (len + 255) / 256, cap = (size_t)ctx->sm_count * 8;
        bf16_to_f32_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, ctx->stream>>>(staging, len, buf->data);
        ctx->launches++;
        e = cudaGetLastError();
    }
    cudaFreeAsync(staging, ctx->stream);
    if (e != cudaSuccess) return fail(ctx, DWIM_B200_ECUDA, "write_bf16: %s", cudaGetErrorString(e));
    return 0;
}

int dwim_b200_read(dwim_b200_ctx *ctx, const dwim_b200_buffer *buf, float *out, size_t len) {
    DWIM_DEVICE(ctx);
    if (!ctx || !buf || (!out && len)) return DWIM_B200_EINVAL;
    REQUIRE(ctx, len == buf->len, DWIM_B200_EINVAL, "read of %zu floats from a buffer of %zu", len, buf->len);
    if (len) DWIM_CUDA(ctx, cudaMemcpyAsync(out, buf->data, len * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    return check_status(ctx);
}

int dwim_b200_buffer_free(dwim_b200_ctx *ctx, dwim_b200_buffer *buf) {
    DWIM_DEVICE(ctx);
    if (!ctx || !buf) return DWIM_B200_EINVAL;
    cudaStreamSynchronize(ctx->stream);
    if (buf->sh_world) shared_release(buf);
    if (buf->owned && buf->data) cudaFree(buf->data);
    if (buf->shadow) cudaFree(buf->shadow);
    delete buf;
    return 0;
}

size_t dwim_b200_buffer_len(const dwim_b200_buffer *buf) { return buf ? buf->len : 0; }
float *dwim_b200_buffer_ptr(const dwim_b200_buffer *buf) { return buf ? buf->data : nullptr; }

// ---- weights ------------------------------------------------------------------

size_t dwim_b200_row_bytes(int fmt, size_t cols) { return file_row_bytes(fmt, cols); }

int dwim_b200_upload(dwim_b200_ctx *ctx, int fmt, size_t rows, size_t cols, const void *blocks, size_t bytes,
                     dwim_b200_weight **out) {
    DWIM_DEVICE(ctx);
    if (!ctx || !out) return DWIM_B200_EINVAL;
    *out = nullptr;
    REQUIRE(ctx, fmt == Q8_0 || fmt == Q4_K || fmt == Q6_K || fmt == BF16, DWIM_B200_EFORMAT, "unknown weight format %d", fmt);
    size_t rb = file_row_bytes(fmt, cols);
    REQUIRE(ctx, cols > 0 && rb > 0, DWIM_B200_EFORMAT, "%zu columns are not whole blocks of %d weights", cols,
            block_weights(fmt));
    REQUIRE(ctx, cols % 8 == 0, DWIM_B200_EFORMAT, "cols must be a multiple of 8");
    REQUIRE(ctx, bytes == rows * rb, DWIM_B200_EINVAL, "a [%zu, %zu] matrix is %zu bytes, not %zu", rows, cols, rows * rb,
            bytes);
    REQUIRE(ctx, blocks || bytes == 0, DWIM_B200_EINVAL, "null blocks");
    REQUIRE(ctx, rows < (size_t)1 << 31 && cols < (size_t)1 << 31, DWIM_B200_EINVAL, "matrix too large");
    dwim_b200_weight *w = new (std::nothrow) dwim_b200_weight();
    REQUIRE(ctx, w, DWIM_B200_ENOMEM, "out of host memory");
    w->v.fmt = fmt;
    w->v.rows = rows;
    w->v.cols = cols;
    w->v.qrow = dev_quant_row_bytes(fmt, cols);
    w->v.qpitch = dev_quant_pitch(fmt, cols);
    w->v.srow = dev_scale_row_elems(fmt, cols);
    uint8_t *staging = nullptr;
    cudaError_t e = cudaMalloc(&w->quants_alloc, rows * w->v.qpitch + WEIGHT_SLACK);
    // the padding between rows is read by the bulk copies: keep it defined
    if (e == cudaSuccess && w->v.qpitch != w->v.qrow)
        e = cudaMemsetAsync(w->quants_alloc, 0, rows * w->v.qpitch, ctx->stream);
    if (e == cudaSuccess && w->v.srow) e = cudaMalloc(&w->scales_alloc, rows * w->v.srow * sizeof(__half) + WEIGHT_SLACK);
    if (e == cudaSuccess) e = cudaMemsetAsync((uint8_t *)w->quants_alloc + rows * w->v.qpitch, 0, WEIGHT_SLACK, ctx->stream);
    int rc = 0;
    if (e == cudaSuccess && bytes) {
        if (fmt == Q4_K || fmt == BF16) {
            e = cudaMemcpy2DAsync(w->quants_alloc, w->v.qpitch, blocks, rb, rb, rows, cudaMemcpyHostToDevice, ctx->stream);
        } else {
            e = cudaMalloc(&staging, bytes);
            if (e == cudaSuccess) e = cudaMemcpyAsync(staging, blocks, bytes, cudaMemcpyHostToDevice, ctx->stream);
            if (e == cudaSuccess) {
                rc = repack_to_device(ctx, fmt, rows, cols, staging, (uint8_t *)w->quants_alloc, (__half *)w->scales_alloc);
                ctx->weights_written = true;
            }
        }
    }
    // The host memory is the caller's again when this returns.
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (staging) cudaFree(staging);
    if (e != cudaSuccess || rc != 0) {
        if (w->quants_alloc) cudaFree(w->quants_alloc);
        if (w->scales_alloc) cudaFree(w->scales_alloc);
        delete w;
        cudaGetLastError();
        if (rc != 0) return rc;
        return fail(ctx, e == cudaErrorMemoryAllocation ? DWIM_B200_ENOMEM : DWIM_B200_ECUDA, "upload: %s",
                    cudaGetErrorString(e));
    }
    w->v.quants = (const uint8_t *)w->quants_alloc;
    w->v.scales = (const __half *)w->scales_alloc;
    *out = w;
    return 0;
}

int dwim_b200_weight_free(dwim_b200_ctx *ctx, dwim_b200_weight *w) {
    DWIM_DEVICE(ctx);
    if (!ctx || !w) return DWIM_B200_EINVAL;
    cudaStreamSynchronize(ctx->stream);
    if (w->quants_alloc) cudaFree(w->quants_alloc);
    if (w->scales_alloc) cudaFree(w->scales_alloc);
    delete w;
    return 0;
}

int dwim_b200_weight_shape(const dwim_b200_weight *w, int *fmt, size_t *rows, size_t *cols) {
    if (!w) return DWIM_B200_EINVAL;
    if (fmt) *fmt = w->v.fmt;
    if (rows) *rows = w->v.rows;
    if (cols) *cols = w->v.cols;
    return 0;
}

int dwim_b200_dequantize(dwim_b200_ctx *ctx, const dwim_b200_weight *w, float *out, size_t len) {
    DWIM_DEVICE(ctx);
    if (!ctx || !w || (!out && len)) return DWIM_B200_EINVAL;
    REQUIRE(ctx, len == w->v.rows * w->v.cols, DWIM_B200_EINVAL, "dequantize: %zu floats for a [%zu, %zu] matrix", len,
            w->v.rows, w->v.cols);
    if (!len) return 0;
    float *dev = nullptr;
    DWIM_CUDA(ctx, cudaMalloc(&dev, len * sizeof(float)));
    int rc = dequantize_device(ctx, w->v, dev);
    cudaError_t e = cudaSuccess;
    if (rc == 0) e = cudaMemcpyAsync(out, dev, len * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(dev);
    if (rc) return rc;
    if (e != cudaSuccess) return fail(ctx, DWIM_B200_ECUDA, "dequantize: %s", cudaGetErrorString(e));
    return 0;
}

int dwim_b200_quantize(dwim_b200_ctx *ctx, int fmt, size_t rows, size_t cols, const float *weights, void *blocks,
                       size_t bytes) {
    DWIM_DEVICE(ctx);
    if (!ctx) return DWIM_B200_EINVAL;
    REQUIRE(ctx, fmt == Q8_0 || fmt == Q4_K || fmt == Q6_K, DWIM_B200_EFORMAT, "unknown weight format %d", fmt);
    size_t rb = file_row_bytes(fmt, cols);
    REQUIRE(ctx, cols > 0 && rb > 0, DWIM_B200_EFORMAT, "%zu columns are not whole blocks of %d weights", cols,
            block_weights(fmt));
    REQUIRE(ctx, bytes == rows * rb, DWIM_B200_EINVAL, "a [%zu, %zu] matrix is %zu bytes, not %zu", rows, cols, rows * rb,
            bytes);
    if (!bytes) return 0;
    REQUIRE(ctx, weights && blocks, DWIM_B200_EINVAL, "null pointer");
    float *wdev = nullptr;
    uint8_t *bdev = nullptr;
    cudaError_t e = cudaMalloc(&wdev, rows * cols * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&bdev, bytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(wdev, weights, rows * cols * sizeof(float), cudaMemcpyHostToDevice, ctx->stream);
    int rc = 0;
    if (e == cudaSuccess) rc = quantize_device(ctx, fmt, rows, cols, wdev, bdev);
    if (e == cudaSuccess && rc == 0) e = cudaMemcpyAsync(blocks, bdev, bytes, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (wdev) cudaFree(wdev);
    if (bdev) cudaFree(bdev);
    if (rc) return rc;
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, e == cudaErrorMemoryAllocation ? DWIM_B200_ENOMEM : DWIM_B200_ECUDA, "quantize: %s",
                    cudaGetErrorString(e));
    }
    return 0;
}

// ---- the product ----------------------------------------------------------------

// Makes sure `x` has a shadow of the given kind for K = cols, (re)building it
// if the buffer was written since.
static int ensure_shadow(dwim_b200_ctx *ctx, dwim_b200_buffer *x, int kind, size_t cols, int split) {
    if (x->shadow_kind == kind && x->shadow_cols == cols && x->shadow_split == split) return 0;
    size_t n = x->len / cols;
    size_t need = kind == SHADOW_GEMM ? gemm_operand_bytes(cols, n, split) : panel_i8_bytes(cols, n);
    if (need > x->shadow_cap) {
        if (x->shadow) {
            DWIM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            cudaFree(x->shadow);
            x->shadow = nullptr;
            x->shadow_cap = 0;
        }
        DWIM_CUDA(ctx, cudaMalloc(&x->shadow, need));
        x->shadow_cap = need;
    }
    x->shadow_kind = SHADOW_NONE;
    int rc = kind == SHADOW_GEMM ? build_gemm_operand(ctx, x->data, n, cols, split, (__half *)x->shadow)
                                 : build_panels_i8(ctx, x->data, n, cols, (uint8_t *)x->shadow);
    if (rc) return rc;
    x->shadow_kind = kind;
    x->shadow_cols = cols;
    x->shadow_split = split;
    return 0;
}

static int product(dwim_b200_ctx *ctx, const OutSpec &out, size_t out_len, const dwim_b200_weight *w, dwim_b200_buffer *x,
                   const float *aux, int epilogue, const char *what) {
    const WeightView &v = w->v;
    REQUIRE(ctx, x->len % v.cols == 0, DWIM_B200_EINVAL, "%s: input of %zu floats is not rows of %zu", what, x->len, v.cols);
    size_t n = x->len / v.cols;
    REQUIRE(ctx, out_len == n * out.pitch, DWIM_B200_EINVAL, "%s: output of %zu floats for %zu tokens of %zu rows", what,
            out_len, n, out.pitch);
    if (n == 0 || v.rows == 0) return 0;
    REQUIRE(ctx, out.dst[0] != x->data, DWIM_B200_EINVAL, "%s: output aliases input", what);
    // bf16 weights (the small gate matrices): f32 activations as they are, fp32 throughout
    if (v.fmt == BF16) return matmul_bf16(ctx, v, x->data, n, out, aux, epilogue);
    // bf16 activations are exact in one f16 column; f32 ones travel as two
    // (value and rounding remainder), summed again in the epilogue.
    // Up to eight tokens: the small-M kernel's int8 routines.  Above: the tensor-core kernels -- Q4_K
    // from nine tokens on (measured on B200 at [17408, 5120]: 26 us at nine to sixteen tokens, against
    // 57 us for sixteen through two small-M launches); Q6_K and Q8_0, whose dense path first decodes
    // the matrix (3.7 ms for the [151936, 5120] head at 64 tokens, against eight small-M launches of
    // 0.31 ms), from 65 on, and in groups of eight through the small-M kernel below that.
    const bool dense = gemm_supports(v) && n > (v.fmt == Q4_K ? (size_t)I8_MAX_TOKENS : (size_t)64);
    if (dense) {
        // bf16 activations are exact in one f16 column; f32 ones travel as two
        // (value and rounding remainder), summed again in the epilogue.
        int split = x->bf16_exact || ctx->act_f16 ? 0 : 1;
        int rc = ensure_shadow(ctx, x, SHADOW_GEMM, v.cols, split);
        if (rc) return rc;
        return gemm_large(ctx, v, (const __half *)x->shadow, n, split, out, aux, epilogue);
    }
    if (!gemv_takes_i8(v, n < (size_t)I8_MAX_TOKENS ? n : (size_t)I8_MAX_TOKENS))
        return fail(ctx, DWIM_B200_EFORMAT, "%s: no kernel takes format %d with %zu columns", what, v.fmt, v.cols);
    if (n <= (size_t)I8_MAX_TOKENS) {
        int rc = ensure_shadow(ctx, x, SHADOW_PANEL_I8, v.cols, 0);
        if (rc) return rc;
        return gemv_small_i8(ctx, v, (const uint8_t *)x->shadow, (int)n, 0, out, aux, epilogue);
    }
    // groups of eight tokens, each with its own digit planes (the buffer's shadow holds one group at a time)
    const size_t need = panel_i8_bytes(v.cols, I8_MAX_TOKENS);
    if (need > x->shadow_cap) {
        if (x->shadow) {
            DWIM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            cudaFree(x->shadow);
            x->shadow = nullptr;
            x->shadow_cap = 0;
        }
        DWIM_CUDA(ctx, cudaMalloc(&x->shadow, need));
        x->shadow_cap = need;
    }
    x->shadow_kind = SHADOW_NONE;
    for (size_t t0 = 0; t0 < n; t0 += I8_MAX_TOKENS) {
        const size_t nt = n - t0 < (size_t)I8_MAX_TOKENS ? n - t0 : (size_t)I8_MAX_TOKENS;
        int rc = build_panels_i8(ctx, x->data + t0 * v.cols, nt, v.cols, (uint8_t *)x->shadow);
        if (rc == 0) rc = gemv_small_i8(ctx, v, (const uint8_t *)x->shadow, (int)nt, t0, out, aux, epilogue);
        if (rc) return rc;
    }
    return 0;
}

}  // extern "C"

namespace dwim {
// For the sharded forms in peer.cu: a plain product into destinations described by `out`.
int product_into(dwim_b200_ctx *ctx, const OutSpec &out, size_t out_len, const dwim_b200_weight *w, dwim_b200_buffer *x,
                 const char *what) {
    return product(ctx, out, out_len, w, x, nullptr, EPI_STORE, what);
}
}  // namespace dwim

extern "C" {

int dwim_b200_matmul(dwim_b200_ctx *ctx, dwim_b200_buffer *out, const dwim_b200_weight *w, dwim_b200_buffer *x) {
    DWIM_DEVICE(ctx);
    if (!ctx || !out || !w || !x) return DWIM_B200_EINVAL;
    int rc = product(ctx, out_local(out->data, w->v.rows), out->len, w, x, nullptr, EPI_STORE, "matmul");
    out->shadow_kind = SHADOW_NONE;
    out->bf16_exact = false;
    return rc;
}

int dwim_b200_matmul_gather(dwim_b200_ctx *ctx, dwim_b200_buffer *out, const dwim_b200_weight *w, dwim_b200_buffer *x,
                            size_t row_begin, size_t total_rows) {
    DWIM_DEVICE(ctx);
    if (!ctx || !out || !w || !x) return DWIM_B200_EINVAL;
    REQUIRE(ctx, out->sh_world >= 1, DWIM_B200_EINVAL, "matmul_gather: the output is not a connected shared buffer");
    REQUIRE(ctx, row_begin + w->v.rows <= total_rows, DWIM_B200_EINVAL, "matmul_gather: rows [%zu, %zu) of %zu", row_begin,
            row_begin + w->v.rows, total_rows);
    OutSpec o{};
    o.world = out->sh_world;
    o.pitch = total_rows;
    o.row0 = row_begin;
    // this rank's copy first: the fused add / SwiGLU forms read it; the peers' follow
    o.dst[0] = out->data;
    // the peers in ring order from this rank on: at any moment the ranks' stores head for different GPUs
    for (int k = 1; k < out->sh_world; k++) o.dst[k] = out->sh_peer[(out->sh_rank + k) % out->sh_world];
    int rc = product(ctx, o, out->len, w, x, nullptr, EPI_STORE, "matmul_gather");
    out->shadow_kind = SHADOW_NONE;
    out->bf16_exact = false;
    return rc;
}

int dwim_b200_matmul_add(dwim_b200_ctx *ctx, dwim_b200_buffer *x, const dwim_b200_weight *w, dwim_b200_buffer *input,
                         dwim_b200_buffer *scratch) {
    DWIM_DEVICE(ctx);
    if (!ctx || !x || !w || !input) return DWIM_B200_EINVAL;
    if (scratch) REQUIRE(ctx, scratch->len == x->len, DWIM_B200_EINVAL, "matmul_add: scratch of %zu for x of %zu", scratch->len, x->len);
    int rc = product(ctx, out_local(x->data, w->v.rows), x->len, w, input, nullptr, EPI_ADD, "matmul_add");
    x->shadow_kind = SHADOW_NONE;
    x->bf16_exact = false;
    return rc;
}

int dwim_b200_swiglu(dwim_b200_ctx *ctx, dwim_b200_buffer *out, const dwim_b200_weight *gate, const dwim_b200_weight *up,
                     dwim_b200_buffer *x, dwim_b200_buffer *scratch) {
    DWIM_DEVICE(ctx);
    if (!ctx || !out || !gate || !up || !x || !scratch) return DWIM_B200_EINVAL;
    REQUIRE(ctx, gate->v.rows == up->v.rows && gate->v.cols == up->v.cols, DWIM_B200_EINVAL,
            "swiglu: gate is [%zu, %zu] but up is [%zu, %zu]", gate->v.rows, gate->v.cols, up->v.rows, up->v.cols);
    REQUIRE(ctx, scratch->len == out->len, DWIM_B200_EINVAL, "swiglu: scratch of %zu for out of %zu", scratch->len, out->len);
    REQUIRE(ctx, scratch->data != out->data, DWIM_B200_EINVAL, "swiglu: scratch aliases out");
    int rc;
    const size_t n = gate->v.cols ? x->len / gate->v.cols : 0;
    if (gate->v.fmt == up->v.fmt && gate->v.qpitch == up->v.qpitch && gemv_takes_i8(gate->v, n) &&
        x->len == n * gate->v.cols && out->len == n * gate->v.rows && out->data != x->data && gate->v.rows) {
        // one and two tokens: both matrices in one launch, the activation applied where the two sums meet
        rc = ensure_shadow(ctx, x, SHADOW_PANEL_I8, gate->v.cols, 0);
        if (rc == 0)
            rc = gemv_small_i8(ctx, gate->v, (const uint8_t *)x->shadow, (int)n, 0, out_local(out->data, gate->v.rows), nullptr, EPI_STORE, &up->v);
    } else {
        // up . x into scratch, then gate . x with the activation fused into the
        // epilogue, as the reference's CUDA device does (gpu/cuda/mod.rs:1148-1175).
        rc = product(ctx, out_local(scratch->data, up->v.rows), scratch->len, up, x, nullptr, EPI_STORE, "swiglu");
        if (rc == 0) rc = product(ctx, out_local(out->data, gate->v.rows), out->len, gate, x, scratch->data, EPI_SWIGLU, "swiglu");
    }
    out->shadow_kind = scratch->shadow_kind = SHADOW_NONE;
    out->bf16_exact = scratch->bf16_exact = false;
    return rc;
}

// ---- sharding ---------------------------------------------------------------------

int dwim_b200_shard_rows(size_t rows, int rank, int world, size_t align, size_t *begin, size_t *end) {
    if (!begin || !end || world <= 0 || rank < 0 || rank >= world || align == 0) return DWIM_B200_EINVAL;
    // Whole groups of `align` rows, the first (groups % world) ranks one more.
    size_t groups = (rows + align - 1) / align;
    size_t base = groups / world, extra = groups % world;
    size_t g0 = (size_t)rank * base + ((size_t)rank < extra ? rank : extra);
    size_t g1 = g0 + base + ((size_t)rank < extra ? 1 : 0);
    *begin = g0 * align < rows ? g0 * align : rows;
    *end = g1 * align < rows ? g1 * align : rows;
    return 0;
}

__global__ void gather_rows_kernel(float *__restrict__ out, const float *__restrict__ parts, size_t n, size_t rows,
                                   int world, size_t align, size_t part_rows) {
    size_t total = n * rows;
    size_t groups = (rows + align - 1) / align, base = groups / world, extra = groups % world;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t t = i / rows, r = i % rows, g = r / align;
        // rank holding group g
        size_t cut = extra * (base + 1);
        size_t rank = g < cut ? g / (base + 1) : extra + (base ? (g - cut) / base : 0);
        size_t g0 = rank * base + (rank < extra ? rank : extra);
        size_t local = r - g0 * align;
        out[i] = parts[(rank * n + t) * part_rows + local];
    }
}

int dwim_b200_gather_rows(dwim_b200_ctx *ctx, dwim_b200_buffer *out, const dwim_b200_buffer *parts, size_t n, size_t rows,
                          int world, size_t align) {
    DWIM_DEVICE(ctx);
    if (!ctx || !out || !parts || world <= 0 || align == 0) return DWIM_B200_EINVAL;
    size_t b0, e0;
    dwim_b200_shard_rows(rows, 0, world, align, &b0, &e0);
    size_t part_rows = e0 - b0;   // rank 0 holds the most
    REQUIRE(ctx, out->len == n * rows, DWIM_B200_EINVAL, "gather_rows: out of %zu for [%zu, %zu]", out->len, n, rows);
    REQUIRE(ctx, parts->len == (size_t)world * n * part_rows, DWIM_B200_EINVAL,
            "gather_rows: parts of %zu, expected %d x %zu x %zu", parts->len, world, n, part_rows);
    if (out->len == 0) return 0;
    size_t blocks = (out->len + 255) / 256, cap = (size_t)ctx->sm_count * 8;
    gather_rows_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, ctx->stream>>>(out->data, parts->data, n, rows,
                                                                                        world, align, part_rows);
    DWIM_LAUNCHED(ctx);
    out->shadow_kind = SHADOW_NONE;
    out->bf16_exact = false;
    return 0;
}

}  // extern "C"
