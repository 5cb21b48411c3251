// Layout conversion at upload, bit-exact dequantization, and the quantizers.
// None of this is on the per-token path; the kernels favour plainness.
//
// Every float operation whose rounding matters is written with an _rn
// intrinsic so that the compiler cannot contract a multiply and an add into
// an FMA: results must equal the CPU's, bit for bit.
#include "common.cuh"

namespace dwim {

// ---------------------------------------------------------------------------
// file layout -> device layout
// ---------------------------------------------------------------------------
// Q8_0: a block is 17 halfwords (scale, 16 quant pairs).
__global__ void repack_q8_0(const uint16_t *__restrict__ file, size_t rows, size_t nb, size_t srow, size_t qpitch,
                            uint16_t *__restrict__ quants, uint16_t *__restrict__ scales) {
    size_t total = rows * nb * 17;
    for (size_t u = blockIdx.x * (size_t)blockDim.x + threadIdx.x; u < total; u += (size_t)gridDim.x * blockDim.x) {
        size_t blk = u / 17, part = u % 17, r = blk / nb, b = blk % nb;
        uint16_t v = file[u];
        if (part == 0) scales[r * srow + b] = v;
        else quants[r * (qpitch / 2) + b * 16 + part - 1] = v;
    }
}
// Q6_K: a block is 105 halfwords (104 of ql|qh|scales, then d).
__global__ void repack_q6_k(const uint16_t *__restrict__ file, size_t rows, size_t nb, size_t srow, size_t qpitch,
                            uint16_t *__restrict__ quants, uint16_t *__restrict__ scales) {
    size_t total = rows * nb * 105;
    for (size_t u = blockIdx.x * (size_t)blockDim.x + threadIdx.x; u < total; u += (size_t)gridDim.x * blockDim.x) {
        size_t blk = u / 105, part = u % 105, r = blk / nb, b = blk % nb;
        uint16_t v = file[u];
        if (part == 104) scales[r * srow + b] = v;
        else quants[r * (qpitch / 2) + b * 104 + part] = v;
    }
}

int repack_to_device(dwim_b200_ctx *ctx, int fmt, size_t rows, size_t cols, const uint8_t *file_dev,
                     uint8_t *quants, __half *scales) {
    if (rows == 0) return 0;
    const size_t qpitch = dev_quant_pitch(fmt, cols);
    if (fmt == Q4_K) {
        size_t rb = file_row_bytes(fmt, cols);
        DWIM_CUDA(ctx, cudaMemcpy2DAsync(quants, qpitch, file_dev, rb, rb, rows, cudaMemcpyDeviceToDevice, ctx->stream));
        return 0;
    }
    size_t nb = cols / block_weights(fmt), srow = dev_scale_row_elems(fmt, cols);
    DWIM_CUDA(ctx, cudaMemsetAsync(scales, 0, rows * srow * sizeof(__half), ctx->stream));
    int grid = ctx->sm_count * 8;
    if (fmt == Q8_0)
        repack_q8_0<<<grid, 256, 0, ctx->stream>>>((const uint16_t *)file_dev, rows, nb, srow, qpitch, (uint16_t *)quants,
                                                   (uint16_t *)scales);
    else
        repack_q6_k<<<grid, 256, 0, ctx->stream>>>((const uint16_t *)file_dev, rows, nb, srow, qpitch, (uint16_t *)quants,
                                                   (uint16_t *)scales);
    DWIM_LAUNCHED(ctx);
    return 0;
}

// ---------------------------------------------------------------------------
// Tensor::dequantize (gpu/mod.rs:138-168) on the device layouts
// ---------------------------------------------------------------------------
__global__ void dequantize_kernel(WeightView w, float *__restrict__ out) {
    size_t total = w.rows * w.cols;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t r = i / w.cols, k = i % w.cols;
        const uint8_t *row = w.quants + r * w.qpitch;
        float v;
        if (w.fmt == Q4_K) {
            v = q4k_weight(row + (k >> 8) * Q4_K_FILE, (int)(k & 255));
        } else if (w.fmt == Q6_K) {
            float d = __half2float(w.scales[r * w.srow + (k >> 8)]);
            v = q6k_weight(row + (k >> 8) * Q6_K_DEV, d, (int)(k & 255));
        } else if (w.fmt == BF16) {
            v = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t *>(row)[k] << 16);   // gpu/float.rs:5-8
        } else {
            // gpu/quant.rs:48-62: q as f32 * d
            float d = __half2float(w.scales[r * w.srow + (k >> 5)]);
            v = __fmul_rn((float)(int8_t)row[k], d);
        }
        out[i] = v;
    }
}

int dequantize_device(dwim_b200_ctx *ctx, const WeightView &w, float *out_dev) {
    if (w.rows * w.cols == 0) return 0;
    dequantize_kernel<<<ctx->sm_count * 16, 256, 0, ctx->stream>>>(w, out_dev);
    DWIM_LAUNCHED(ctx);
    return 0;
}

// ---------------------------------------------------------------------------
// quantizers: one thread per block, written as the scalar algorithm
// ---------------------------------------------------------------------------

// The multiple of s nearest a, ties away from zero, decided against the exact
// midpoints (as quant::quantize does, gpu/quant.rs:154-180) so that the
// division's rounding cannot matter; clamped to lo..hi.
__device__ inline int nearest_multiple(float a, float s, int lo, int hi) {
    float mag = fabsf(a);
    float n = fminf(roundf(__fdiv_rn(mag, s)), 1024.0f);
    if (mag >= __fmul_rn(__fadd_rn(n, 0.5f), s)) n = __fadd_rn(n, 1.0f);
    else if (n > 0.0f && mag < __fmul_rn(__fsub_rn(n, 0.5f), s)) n = __fsub_rn(n, 1.0f);
    int v = (int)n;
    if (a < 0.0f) v = -v;
    return v < lo ? lo : (v > hi ? hi : v);
}

// quantize_q8_0_row / quantize (gpu/quant.rs:31-46, 154-180).
__global__ void quantize_q8_0_kernel(const float *__restrict__ w, size_t n_blocks, uint8_t *__restrict__ out) {
    size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const float *x = w + b * 32;
    uint8_t *blk = out + b * Q8_0_FILE;
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[i]));
    const uint32_t bits = to_f16_bits(__fmul_rn(amax, 1.0f / 127.0f));
    float d = from_f16_bits(bits);
    blk[0] = (uint8_t)(bits & 0xff);
    blk[1] = (uint8_t)(bits >> 8);
    for (int i = 0; i < 32; i++) {
        int8_t q = 0;
        if (d > 0.0f) {
            float a = fabsf(x[i]);
            float n = fminf(roundf(__fdiv_rn(a, d)), 128.0f);
            if (a >= __fmul_rn(__fadd_rn(n, 0.5f), d)) n = __fadd_rn(n, 1.0f);
            else if (n > 0.0f && a < __fmul_rn(__fsub_rn(n, 0.5f), d)) n = __fsub_rn(n, 1.0f);
            int v = (int)fminf(n, 127.0f);
            q = (int8_t)(x[i] < 0.0f ? -v : v);
        }
        blk[2 + i] = (uint8_t)q;
    }
}

// Every output byte is computed whole and stored once.
__global__ void quantize_q6_k_kernel(const float *__restrict__ w, size_t n_blocks, uint8_t *__restrict__ out) {
    size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const float *x = w + b * 256;
    uint8_t *blk = out + b * Q6_K_FILE;
    float step[16], top = 0.0f;
    for (int g = 0; g < 16; g++) {
        float amax = 0.0f;
        for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(x[g * 16 + i]));
        step[g] = __fmul_rn(amax, 1.0f / 31.0f);
        top = fmaxf(top, step[g]);
    }
    const uint32_t dbits = to_f16_bits(__fmul_rn(top, 1.0f / 127.0f));
    const float d = from_f16_bits(dbits);
    const bool live = d > 0.0f;
    int sc[16];
    for (int g = 0; g < 16; g++) sc[g] = live ? (int)fminf(ceilf(__fdiv_rn(step[g], d)), 127.0f) : 0;
    for (int half = 0; half < 2; half++)
        for (int l = 0; l < 32; l++) {
            int v[4];
            for (int k = 0; k < 4; k++) {
                int idx = half * 128 + 32 * k + l, s = sc[idx >> 4];
                // all-zero blocks keep every byte zero, as the scalar algorithm does
                v[k] = !live ? 0 : s > 0 ? nearest_multiple(x[idx], __fmul_rn(d, (float)s), -32, 31) + 32 : 32;
            }
            blk[half * 64 + l] = (uint8_t)((v[0] & 0xf) | ((v[2] & 0xf) << 4));
            blk[half * 64 + l + 32] = (uint8_t)((v[1] & 0xf) | ((v[3] & 0xf) << 4));
            blk[128 + half * 32 + l] = (uint8_t)((v[0] >> 4) | ((v[1] >> 4) << 2) | ((v[2] >> 4) << 4) | ((v[3] >> 4) << 6));
        }
    for (int g = 0; g < 16; g++) blk[192 + g] = (uint8_t)(int8_t)sc[g];
    blk[208] = (uint8_t)(dbits & 0xff);
    blk[209] = (uint8_t)(dbits >> 8);
}

__global__ void quantize_q4_k_kernel(const float *__restrict__ w, size_t n_blocks, uint8_t *__restrict__ out) {
    size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const float *x = w + b * 256;
    uint8_t *blk = out + b * Q4_K_FILE;
    float step[8], low[8], top_step = 0.0f, top_low = 0.0f;
    for (int j = 0; j < 8; j++) {
        float mn = 0.0f, mx = 0.0f;
        for (int i = 0; i < 32; i++) { mn = fminf(mn, x[j * 32 + i]); mx = fmaxf(mx, x[j * 32 + i]); }
        low[j] = __fsub_rn(0.0f, mn);   // +0, not -0, when the sub-block has no negative weight
        step[j] = __fmul_rn(__fsub_rn(mx, mn), 1.0f / 15.0f);
        top_step = fmaxf(top_step, step[j]);
        top_low = fmaxf(top_low, low[j]);
    }
    const uint32_t dbits = to_f16_bits(__fmul_rn(top_step, 1.0f / 63.0f));
    const uint32_t mbits = to_f16_bits(__fmul_rn(top_low, 1.0f / 63.0f));
    const float d = from_f16_bits(dbits), dmin = from_f16_bits(mbits);
    int sc8[8], m8[8];
    for (int j = 0; j < 8; j++) {
        sc8[j] = d > 0.0f ? nearest_multiple(step[j], d, 0, 63) : 0;
        m8[j] = dmin > 0.0f ? nearest_multiple(low[j], dmin, 0, 63) : 0;
    }
    blk[0] = (uint8_t)(dbits & 0xff);
    blk[1] = (uint8_t)(dbits >> 8);
    blk[2] = (uint8_t)(mbits & 0xff);
    blk[3] = (uint8_t)(mbits >> 8);
    for (int j = 0; j < 4; j++) {
        blk[4 + j] = (uint8_t)((sc8[j] & 63) | ((sc8[j + 4] >> 4) << 6));
        blk[8 + j] = (uint8_t)((m8[j] & 63) | ((m8[j + 4] >> 4) << 6));
        blk[12 + j] = (uint8_t)((sc8[j + 4] & 0xf) | ((m8[j + 4] & 0xf) << 4));
    }
    for (int g = 0; g < 4; g++) {
        const float ds0 = __fmul_rn(d, (float)sc8[2 * g]), dm0 = __fmul_rn(dmin, (float)m8[2 * g]);
        const float ds1 = __fmul_rn(d, (float)sc8[2 * g + 1]), dm1 = __fmul_rn(dmin, (float)m8[2 * g + 1]);
        for (int i = 0; i < 32; i++) {
            int q0 = ds0 > 0.0f ? nearest_multiple(__fadd_rn(x[(2 * g) * 32 + i], dm0), ds0, 0, 15) : 0;
            int q1 = ds1 > 0.0f ? nearest_multiple(__fadd_rn(x[(2 * g + 1) * 32 + i], dm1), ds1, 0, 15) : 0;
            blk[16 + g * 32 + i] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}

int quantize_device(dwim_b200_ctx *ctx, int fmt, size_t rows, size_t cols, const float *w_dev, uint8_t *file_dev) {
    size_t n_blocks = rows * (cols / block_weights(fmt));
    if (n_blocks == 0) return 0;
    unsigned grid = (unsigned)((n_blocks + 127) / 128);
    if (fmt == Q8_0) quantize_q8_0_kernel<<<grid, 128, 0, ctx->stream>>>(w_dev, n_blocks, file_dev);
    else if (fmt == Q6_K) quantize_q6_k_kernel<<<grid, 128, 0, ctx->stream>>>(w_dev, n_blocks, file_dev);
    else quantize_q4_k_kernel<<<grid, 128, 0, ctx->stream>>>(w_dev, n_blocks, file_dev);
    DWIM_LAUNCHED(ctx);
    return 0;
}

}  // namespace dwim
