// The operators that sit either side of the quantized product in the
// engine's layer (inference/qwen35/mod.rs:547, 603-605, 652-654, 1066-1068):
//   - normalize: RMS norm of the residual stream into the product's input
//     (Cuda::normalize, gpu/cuda/mod.rs:1177-1198; rmsnorm.cu:11-58).  The
//     reference writes the f16 copy its tile kernels read; here the same
//     launch writes the f32 result and the operand form the next product
//     reads, so that no separate activation prologue runs.
//   - the product with bf16 weights (matmul_bf16.cu:19-81): the small gate
//     matrices of the linear-attention layers, 48 calls per token.
//   - argmax over the vocabulary's logits on the device, instead of reading
//     608 KB back per drafted token and scanning them on the host
//     (inference/qwen35/mod.rs:702-710, 1066-1068).
#include <new>

#include "common.cuh"
#include "ptx.cuh"

using namespace dwim;

namespace {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Cpu::rmsnorm (gpu/cpu.rs:157-166) for any row length: one block of 256
// threads per row, v * (scale * w) with scale = 1 / sqrt(sum(v^2) / dim + eps).
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float *x, const float *__restrict__ weight, float eps, float *out,
                                                           size_t dim) {
    griddep_launch();
    griddep_wait();
    __shared__ float part[8];
    const float *src = x + (size_t)blockIdx.x * dim;
    float *dst = out + (size_t)blockIdx.x * dim;
    float ss = 0.0f;
    for (size_t i = threadIdx.x; i < dim; i += 256) ss += src[i] * src[i];
    ss = warp_sum_f(ss);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = part[0];
#pragma unroll
    for (int i = 1; i < 8; i++) total += part[i];
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)dim), eps)));
    for (size_t i = threadIdx.x; i < dim; i += 256) dst[i] = __fmul_rn(src[i], __fmul_rn(scale, weight[i]));
}

// out[t][r] = w[r] . x[t] for bf16 weights: a warp per weight row, up to eight
// tokens per block; lanes walk the row eight weights (16 bytes) at a time.
struct Bf16Args {
    const uint16_t *w;
    size_t rows, cols, n;
    const float *x;
    OutSpec out;
    const float *aux;
    int epi;
};

__device__ __forceinline__ float silu_mul_n(float g, float u) { return g * (1.0f / (1.0f + expf(-g))) * u; }

__global__ void __launch_bounds__(256) matmul_bf16_kernel(const __grid_constant__ Bf16Args a) {
    griddep_launch();
    griddep_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t r = (size_t)blockIdx.x * 8 + warp;
    const size_t t0 = (size_t)blockIdx.y * 8;
    const int nt = (int)min((size_t)8, a.n - t0);
    if (r >= a.rows) return;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const uint16_t *row = a.w + r * a.cols;
    for (size_t k = (size_t)lane * 8; k < a.cols; k += 256) {
        const uint4 wv = *reinterpret_cast<const uint4 *>(row + k);
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        float wf[8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            wf[2 * i] = __uint_as_float(ww[i] << 16);              // gpu/float.rs:5-8
            wf[2 * i + 1] = __uint_as_float(ww[i] & 0xffff0000u);
        }
#pragma unroll
        for (int t = 0; t < 8; t++) {
            if (t < nt) {
                const float *xs = a.x + (t0 + t) * a.cols + k;
#pragma unroll
                for (int i = 0; i < 8; i++) acc[t] = fmaf(wf[i], xs[i], acc[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < 8; t++) {
        const float v = warp_sum_f(acc[t]);
        if (lane == 0 && t < nt) {
            const size_t i = (t0 + t) * a.out.pitch + a.out.row0 + r;
            float y = v;
            if (a.epi == EPI_ADD) y += a.out.dst[0][i];
            else if (a.epi == EPI_SWIGLU) y = silu_mul_n(y, a.aux[(t0 + t) * a.rows + r]);
            a.out.dst[0][i] = y;
            if (a.out.world > 1) {
#pragma unroll
                for (int p = 1; p < DWIM_MAX_WORLD; p++)
                    if (p < a.out.world) a.out.dst[p][i] = y;
            }
        }
    }
}

// argmax: per token (row of `len` logits) the largest value's first index.  A
// value and its index travel as one 64-bit key that orders like the pair
// (value ascending, index descending): the float's bits made monotone in the
// high word, the index's complement in the low word; the maximum over the row
// is taken by warp shuffles, then one atomicMax per block.  A NaN never wins
// (the host's `>` never lets one in either); a row of NaNs gives index 0.
__device__ __forceinline__ unsigned long long argmax_key(float v, uint32_t i) {
    uint32_t b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    if (v != v) b = 0;
    return ((unsigned long long)b << 32) | (0xffffffffu - i);
}

__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ logits, size_t len, unsigned long long *best) {
    griddep_launch();
    griddep_wait();
    const float *row = logits + (size_t)blockIdx.y * len;
    unsigned long long k = 0;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < len; i += (size_t)gridDim.x * 256) {
        const unsigned long long c = argmax_key(row[i], (uint32_t)i);
        k = c > k ? c : k;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long c = __shfl_xor_sync(0xffffffffu, k, o);
        k = c > k ? c : k;
    }
    __shared__ unsigned long long part[8];
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = k;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 1; i < 8; i++) k = part[i] > k ? part[i] : k;
        atomicMax(best + blockIdx.y, k);
    }
}

int reserve_shadow(dwim_b200_ctx *ctx, dwim_b200_buffer *b, size_t need) {
    if (need <= b->shadow_cap) return 0;
    if (b->shadow) {
        DWIM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        cudaFree(b->shadow);
        b->shadow = nullptr;
        b->shadow_cap = 0;
    }
    DWIM_CUDA(ctx, cudaMalloc(&b->shadow, need));
    b->shadow_cap = need;
    return 0;
}

}  // namespace

namespace dwim {

int matmul_bf16(dwim_b200_ctx *ctx, const WeightView &w, const float *x, size_t n, const OutSpec &out, const float *aux, int epi) {
    if (n == 0 || w.rows == 0) return 0;
    Bf16Args a{reinterpret_cast<const uint16_t *>(w.quants), w.rows, w.cols, n, x, out, aux, epi};
    const size_t gy = (n + 7) / 8;
    if (gy > 65535) return fail(ctx, DWIM_B200_EINVAL, "bf16 product: %zu tokens in one call", n);
    DWIM_CUDA(ctx, launch_dependent(!ctx->weights_written, matmul_bf16_kernel, dim3((unsigned)((w.rows + 7) / 8), (unsigned)gy), dim3(256),
                                    0, ctx->stream, a));
    ctx->weights_written = false;
    DWIM_LAUNCHED(ctx);
    return 0;
}

}  // namespace dwim

extern "C" int dwim_b200_normalize(dwim_b200_ctx *ctx, dwim_b200_buffer *out, const dwim_b200_buffer *x,
                                   const dwim_b200_buffer *weight, size_t len, float eps) {
    DWIM_DEVICE(ctx);
    if (!ctx || !out || !x || !weight) return DWIM_B200_EINVAL;
    const size_t dim = weight->len;
    // gpu/cuda/mod.rs:1184-1185
    if (dim == 0 || out->len != len || len > x->len || len % dim != 0)
        return fail(ctx, DWIM_B200_EINVAL, "normalize: out of %zu, %zu of x's %zu, rows of %zu", out->len, len, x->len, dim);
    out->shadow_kind = SHADOW_NONE;
    out->bf16_exact = false;
    if (len == 0) return 0;
    const size_t n = len / dim;
    if (dim % 256 == 0 && n > DWIM_SMALL_M_MAX && n <= 65535) {
        // more tokens than the small-M kernel takes: the next product is the tensor-core GEMM, whose
        // operand (f16 value and remainder columns, sub-block means, the token's scale) this launch writes
        const int split = ctx->act_f16 ? 0 : 1;
        int rc = reserve_shadow(ctx, out, gemm_operand_bytes(dim, n, split));
        if (rc) return rc;
        rc = build_gemm_operand(ctx, x->data, n, dim, split, (__half *)out->shadow, weight->data, eps, out->data);
        if (rc) return rc;
        out->shadow_kind = SHADOW_GEMM;
        out->shadow_cols = dim;
        out->shadow_split = split;
        return 0;
    }
    if (dim % 256 == 0 && n <= (size_t)I8_MAX_TOKENS) {
        // a few tokens: the int8 digit planes of the small-M kernel, from the same launch
        int rc = reserve_shadow(ctx, out, panel_i8_bytes(dim, n));
        if (rc) return rc;
        rc = build_panels_i8(ctx, x->data, n, dim, (uint8_t *)out->shadow, weight->data, eps, out->data);
        if (rc) return rc;
        out->shadow_kind = SHADOW_PANEL_I8;
        out->shadow_cols = dim;
        out->shadow_split = 0;
        return 0;
    }
    DWIM_CUDA(ctx, launch_dependent(!ctx->weights_written, rmsnorm_rows_kernel, dim3((unsigned)n), dim3(256), 0, ctx->stream,
                                    (const float *)x->data, (const float *)weight->data, eps, out->data, dim));
    DWIM_LAUNCHED(ctx);
    return 0;
}

extern "C" int dwim_b200_argmax(dwim_b200_ctx *ctx, const dwim_b200_buffer *logits, size_t len, uint32_t *out, size_t n) {
    DWIM_DEVICE(ctx);
    if (!ctx || !logits || (!out && n)) return DWIM_B200_EINVAL;
    if (len == 0 || n * len != logits->len || len > 0xffffffffull || n > 65535)
        return fail(ctx, DWIM_B200_EINVAL, "argmax: %zu rows of %zu logits in a buffer of %zu", n, len, logits->len);
    if (n == 0) return 0;
    if (n > ctx->argmax_cap) {
        if (ctx->argmax_dev) {
            DWIM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            cudaFree(ctx->argmax_dev);
            cudaFreeHost(ctx->argmax_host);
            ctx->argmax_dev = ctx->argmax_host = nullptr;
            ctx->argmax_cap = 0;
        }
        const size_t cap = n < 16 ? 16 : n;
        DWIM_CUDA(ctx, cudaMalloc((void **)&ctx->argmax_dev, cap * sizeof(unsigned long long)));
        DWIM_CUDA(ctx, cudaMallocHost((void **)&ctx->argmax_host, cap * sizeof(unsigned long long)));
        ctx->argmax_cap = cap;
    }
    DWIM_CUDA(ctx, cudaMemsetAsync(ctx->argmax_dev, 0, n * sizeof(unsigned long long), ctx->stream));
    size_t blocks = (len + 2047) / 2048;
    if (blocks > (size_t)ctx->sm_count * 2) blocks = (size_t)ctx->sm_count * 2;
    argmax_kernel<<<dim3((unsigned)blocks, (unsigned)n), 256, 0, ctx->stream>>>(logits->data, len, ctx->argmax_dev);
    DWIM_LAUNCHED(ctx);
    DWIM_CUDA(ctx, cudaMemcpyAsync(ctx->argmax_host, ctx->argmax_dev, n * sizeof(unsigned long long), cudaMemcpyDeviceToHost, ctx->stream));
    DWIM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (size_t t = 0; t < n; t++) out[t] = 0xffffffffu - (uint32_t)(ctx->argmax_host[t] & 0xffffffffull);
    // a row of NaNs leaves the key at zero: index 0, as the host's scan gives
    for (size_t t = 0; t < n; t++)
        if (ctx->argmax_host[t] == 0) out[t] = 0;
    return 0;
}
