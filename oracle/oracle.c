/*
 * CPU oracle for the block-quantized matrix product.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared with; nothing that ships calls it.  It is a plain-C restatement of
 * the reference engine's CPU device for this path, written so that every
 * float operation rounds exactly as the reference's Rust does: build with
 * -O2 -ffp-contract=off (Rust never contracts a multiply and an add into an
 * FMA) and without -ffast-math.
 *
 * Parity status, per format:
 *   f16 / bf16 conversions  pinned by the reference's known-answer tests
 *                           (gpu/cpu.rs:510-533, 560-575)
 *   Q8_0 codec and dot      pinned (gpu/quant.rs:31-83, 154-180; KATs at
 *                           gpu/cpu.rs:535-558, gpu/quant.rs:198-257)
 *   Q4_0 codec and dot      pinned (gpu/quant.rs:85-152; KAT gpu/quant.rs:213-230)
 *   Q6_K decode             pinned (inference/quants.rs:73-104; KAT :236-275)
 *   Q6_K quantizer and dot  PARITY UNPINNED: the reference has neither
 *   Q4_K, everything        PARITY UNPINNED: the reference has no Q4_K code at
 *                           all; the block layout follows the public GGUF
 *                           description and the arithmetic follows the style
 *                           of the reference's Q4_0 functions
 *
 * Layouts.  "File" layouts are GGUF's interleaved blocks.  The reference's
 * devices keep Q4_0/Q8_0 scales and quants apart (gpu/quant.rs:1-12); the
 * functions here that end in _split take that form.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ */
/* bit helpers                                                         */
/* ------------------------------------------------------------------ */
static inline uint32_t f32_bits(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float bits_f32(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }
static inline uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static inline void wr16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }

/* ------------------------------------------------------------------ */
/* gpu/float.rs                                                        */
/* ------------------------------------------------------------------ */

/* gpu/float.rs:5-8 — bf16 is the top half of an f32. */
ORC_API float orc_bf16(uint16_t bits) { return bits_f32((uint32_t)bits << 16); }

/* gpu/float.rs:30-36 — round to nearest even on the dropped half. */
ORC_API uint16_t orc_to_bf16(float x) {
    uint32_t bits = f32_bits(x);
    uint32_t round = 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)((bits + round) >> 16);
}

/* gpu/float.rs:38-48 — exact, subnormals included. */
ORC_API float orc_from_f16(uint16_t h) {
    uint32_t bits = h, sign = bits & 0x8000u;
    uint32_t exp = (bits >> 10) & 0x1fu;
    uint32_t mantissa = (bits & 0x3ffu) | ((uint32_t)(exp != 0) << 10);
    uint32_t e = exp > 1 ? exp : 1;
    float scale = bits_f32((e + 127u - 25u) << 23);
    float magnitude = (float)mantissa * scale;
    return bits_f32(f32_bits(magnitude) | (sign << 16));
}

/* gpu/float.rs:13-28 — nearest, ties to even, clamped to +-65504 (never inf). */
ORC_API uint16_t orc_to_f16(float x) {
    uint16_t sign = (uint16_t)((f32_bits(x) >> 16) & 0x8000u);
    float a = fminf(fabsf(x), 65504.0f);
    if (a < bits_f32((127u - 14u) << 23)) {
        return (uint16_t)(sign | (uint16_t)rintf(a * 16777216.0f));
    }
    int e = (int)((f32_bits(a) >> 23) & 0xffu) - 127;
    uint32_t m = (uint32_t)rintf(a * bits_f32((uint32_t)(127 + 10 - e) << 23));
    if (m == 2048u) { e += 1; m = 1024u; }
    return (uint16_t)(sign | (uint16_t)((e + 15) << 10) | (uint16_t)(m - 1024u));
}

ORC_API void orc_to_f16_array(const float *x, size_t n, uint16_t *out) {
    for (size_t i = 0; i < n; i++) out[i] = orc_to_f16(x[i]);
}
ORC_API void orc_from_f16_array(const uint16_t *h, size_t n, float *out) {
    for (size_t i = 0; i < n; i++) out[i] = orc_from_f16(h[i]);
}
ORC_API void orc_to_bf16_array(const float *x, size_t n, uint16_t *out) {
    for (size_t i = 0; i < n; i++) out[i] = orc_to_bf16(x[i]);
}
ORC_API void orc_bf16_array(const uint16_t *h, size_t n, float *out) {
    for (size_t i = 0; i < n; i++) out[i] = orc_bf16(h[i]);
}

/* gpu/tests.rs:45-54 (and the copies at gpu/quant.rs:186-196,
 * inference/quants.rs:194-204) — the deterministic generator every reference
 * test draws its data from: values in [-1, 1).  The state is updated in
 * place so that consecutive calls continue one stream, as Rng does. */
ORC_API void orc_lcg_floats(uint64_t *state, size_t n, float *out) {
    uint64_t s = *state;
    for (size_t i = 0; i < n; i++) {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        out[i] = ((float)(s >> 40) / 16777216.0f) * 2.0f - 1.0f;
    }
    *state = s;
}

/* ------------------------------------------------------------------ */
/* gpu/quant.rs — 32-weight blocks, split layout                       */
/* ------------------------------------------------------------------ */
#define BLOCK 32

/* gpu/quant.rs:154-180 — scale = f16(amax/127); each value the nearest
 * multiple, ties away from zero, settled against exact midpoints. */
ORC_API uint16_t orc_quantize_block(const float *block, int8_t *q) {
    float amax = 0.0f;
    for (int i = 0; i < BLOCK; i++) amax = fmaxf(amax, fabsf(block[i]));
    uint16_t bits = orc_to_f16(amax * (1.0f / 127.0f));
    float d = orc_from_f16(bits);
    memset(q, 0, BLOCK);
    if (d > 0.0f) {
        for (int i = 0; i < BLOCK; i++) {
            float x = block[i], a = fabsf(x);
            float n = fminf(roundf(a / d), 128.0f);
            if (a >= (n + 0.5f) * d) n += 1.0f;
            else if (n > 0.0f && a < (n - 0.5f) * d) n -= 1.0f;
            int8_t v = (int8_t)fminf(n, 127.0f);
            q[i] = (int8_t)(x < 0.0f ? -v : v);
        }
    }
    return bits;
}

/* gpu/quant.rs:31-46 */
ORC_API void orc_quantize_q8_0_row_split(const float *x, size_t cols, uint16_t *scales, int8_t *quants) {
    for (size_t b = 0; b < cols / BLOCK; b++)
        scales[b] = orc_quantize_block(x + b * BLOCK, quants + b * BLOCK);
}

/* gpu/quant.rs:48-62 — one fp32 multiply of exact operands. */
ORC_API void orc_dequantize_q8_0_row_split(const uint16_t *scales, const int8_t *quants, size_t cols, float *out) {
    for (size_t b = 0; b < cols / BLOCK; b++) {
        float d = orc_from_f16(scales[b]);
        for (int i = 0; i < BLOCK; i++) out[b * BLOCK + i] = (float)quants[b * BLOCK + i] * d;
    }
}

/* Left fold of the eight lane sums, as `sum.iter().sum::<f32>()` does
 * (gpu/quant.rs:80, 149). */
static inline float fold8(const float *s) {
    float t = 0.0f;
    for (int i = 0; i < 8; i++) t += s[i];
    return t;
}

/* gpu/quant.rs:64-83 */
ORC_API float orc_dot_q8_0_split(const uint16_t *scales, const int8_t *quants, const float *x, size_t cols) {
    float acc = 0.0f;
    for (size_t b = 0; b < cols / BLOCK; b++) {
        float sum[8] = {0};
        const int8_t *q = quants + b * BLOCK;
        const float *xb = x + b * BLOCK;
        for (int c = 0; c < 4; c++)
            for (int i = 0; i < 8; i++) sum[i] += (float)q[c * 8 + i] * xb[c * 8 + i];
        acc += orc_from_f16(scales[b]) * fold8(sum);
    }
    return acc;
}

/* gpu/quant.rs:85-113 — llama.cpp's Q4_0: scale = signed max / -8. */
ORC_API void orc_quantize_q4_0_row_split(const float *x, size_t cols, uint16_t *scales, uint8_t *quants) {
    for (size_t b = 0; b < cols / BLOCK; b++) {
        const float *block = x + b * BLOCK;
        float max = 0.0f;
        for (int i = 0; i < BLOCK; i++) if (fabsf(block[i]) > fabsf(max)) max = block[i];
        float d = max / -8.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        scales[b] = orc_to_f16(d);
        for (int j = 0; j < BLOCK / 2; j++) {
            float lo = block[j] * id + 8.5f, hi = block[j + BLOCK / 2] * id + 8.5f;
            lo = lo < 0.0f ? 0.0f : (lo > 15.0f ? 15.0f : lo);
            hi = hi < 0.0f ? 0.0f : (hi > 15.0f ? 15.0f : hi);
            quants[b * 16 + j] = (uint8_t)((uint8_t)lo | ((uint8_t)hi << 4));
        }
    }
}

/* gpu/quant.rs:115-126 */
ORC_API void orc_dequantize_q4_0_row_split(const uint16_t *scales, const uint8_t *quants, size_t cols, float *out) {
    for (size_t b = 0; b < cols / BLOCK; b++) {
        float d = orc_from_f16(scales[b]);
        for (int j = 0; j < 16; j++) {
            uint8_t q = quants[b * 16 + j];
            out[b * BLOCK + j] = ((float)(q & 0xf) - 8.0f) * d;
            out[b * BLOCK + j + 16] = ((float)(q >> 4) - 8.0f) * d;
        }
    }
}

/* gpu/quant.rs:128-152 */
ORC_API float orc_dot_q4_0_split(const uint16_t *scales, const uint8_t *quants, const float *x, size_t cols) {
    float acc = 0.0f;
    for (size_t b = 0; b < cols / BLOCK; b++) {
        const uint8_t *q = quants + b * 16;
        const float *lo = x + b * BLOCK, *hi = lo + 16;
        float sum[8] = {0};
        for (int c = 0; c < 2; c++)
            for (int i = 0; i < 8; i++) {
                float a = ((float)(q[c * 8 + i] & 0xf) - 8.0f) * lo[c * 8 + i];
                float bb = ((float)(q[c * 8 + i] >> 4) - 8.0f) * hi[c * 8 + i];
                sum[i] += a + bb;
            }
        acc += orc_from_f16(scales[b]) * fold8(sum);
    }
    return acc;
}

/* ------------------------------------------------------------------ */
/* inference/quants.rs — GGUF file layouts                             */
/* ------------------------------------------------------------------ */
#define Q8_0_BYTES 34
#define Q4_1_BYTES 20
#define Q6_K_BYTES 210
#define Q4_K_BYTES 144
#define KBLOCK 256

/* inference/quants.rs:59-71 — [d f16][32 x i8]. */
ORC_API void orc_dequantize_q8_0(const uint8_t *row, size_t cols, float *out) {
    for (size_t b = 0; b < cols / BLOCK; b++) {
        const uint8_t *blk = row + b * Q8_0_BYTES;
        float d = orc_from_f16(rd16(blk));
        for (int i = 0; i < BLOCK; i++) out[b * BLOCK + i] = (float)(int8_t)blk[2 + i] * d;
    }
}

/* inference/quants.rs:44-57 — [d f16][m f16][16 bytes of nibbles]. */
ORC_API void orc_dequantize_q4_1(const uint8_t *row, size_t cols, float *out) {
    for (size_t b = 0; b < cols / BLOCK; b++) {
        const uint8_t *blk = row + b * Q4_1_BYTES;
        float d = orc_from_f16(rd16(blk)), m = orc_from_f16(rd16(blk + 2));
        for (int j = 0; j < 16; j++) {
            uint8_t q = blk[4 + j];
            out[b * BLOCK + j] = (float)(q & 0xf) * d + m;
            out[b * BLOCK + j + 16] = (float)(q >> 4) * d + m;
        }
    }
}

/* inference/quants.rs:73-104 — ql[128] qh[64] scales[16] d; the product is
 * evaluated left to right: (d * scale) * q. */
ORC_API void orc_dequantize_q6_k(const uint8_t *row, size_t cols, float *out) {
    for (size_t b = 0; b < cols / KBLOCK; b++) {
        const uint8_t *blk = row + b * Q6_K_BYTES;
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t *scales = (const int8_t *)(blk + 192);
        float d = orc_from_f16(rd16(blk + 208));
        float *o = out + b * KBLOCK;
        for (int half = 0; half < 2; half++)
            for (int l = 0; l < 32; l++)
                for (int k = 0; k < 4; k++) {
                    int low = (ql[half * 64 + l + 32 * (k % 2)] >> (4 * (k / 2))) & 0xf;
                    int high = (qh[half * 32 + l] >> (2 * k)) & 3;
                    int q = (low | (high << 4)) - 32;
                    float ds = d * (float)scales[half * 8 + 2 * k + l / 16];
                    o[half * 128 + l + 32 * k] = ds * (float)q;
                }
    }
}

/* Interleaves / parts the Q8_0 layouts (inference/quants.rs:123-138, 188-199). */
ORC_API void orc_q8_0_split_to_file(const uint16_t *scales, const int8_t *quants, size_t n_blocks, uint8_t *out) {
    for (size_t b = 0; b < n_blocks; b++) {
        wr16(out + b * Q8_0_BYTES, scales[b]);
        memcpy(out + b * Q8_0_BYTES + 2, quants + b * BLOCK, BLOCK);
    }
}
ORC_API void orc_q8_0_file_to_split(const uint8_t *data, size_t n_blocks, uint16_t *scales, int8_t *quants) {
    for (size_t b = 0; b < n_blocks; b++) {
        scales[b] = rd16(data + b * Q8_0_BYTES);
        memcpy(quants + b * BLOCK, data + b * Q8_0_BYTES + 2, BLOCK);
    }
}

/* Quantizes a row straight to GGUF Q8_0 blocks (quantize_q8_0_row, then
 * pack_q8_0: inference/quants.rs:188-199). */
ORC_API void orc_quantize_q8_0(const float *x, size_t cols, uint8_t *row) {
    for (size_t b = 0; b < cols / BLOCK; b++) {
        int8_t q[BLOCK];
        uint16_t s = orc_quantize_block(x + b * BLOCK, q);
        wr16(row + b * Q8_0_BYTES, s);
        memcpy(row + b * Q8_0_BYTES + 2, q, BLOCK);
    }
}

/* Dot of a GGUF Q8_0 row: the same arithmetic as orc_dot_q8_0_split. */
ORC_API float orc_dot_q8_0(const uint8_t *row, const float *x, size_t cols) {
    float acc = 0.0f;
    for (size_t b = 0; b < cols / BLOCK; b++) {
        const uint8_t *blk = row + b * Q8_0_BYTES;
        const float *xb = x + b * BLOCK;
        float sum[8] = {0};
        for (int c = 0; c < 4; c++)
            for (int i = 0; i < 8; i++) sum[i] += (float)(int8_t)blk[2 + c * 8 + i] * xb[c * 8 + i];
        acc += orc_from_f16(rd16(blk)) * fold8(sum);
    }
    return acc;
}

/* ------------------------------------------------------------------ */
/* Q6_K quantizer and dot — no reference counterpart (parity unpinned)  */
/* ------------------------------------------------------------------ */

/* Nearest integer, ties away from zero, of a / s decided against exact
 * midpoints so that a division that is not correctly rounded cannot change
 * the result (the device quantizer must give the same bytes).  lo..hi clamp. */
static inline int nearest_multiple(float a, float s, int lo, int hi) {
    /* a and s are finite, s > 0 */
    float mag = fabsf(a);
    float n = fminf(roundf(mag / s), 1024.0f);
    if (mag >= (n + 0.5f) * s) n += 1.0f;
    else if (n > 0.0f && mag < (n - 0.5f) * s) n -= 1.0f;
    int v = (int)n;
    if (a < 0.0f) v = -v;
    return v < lo ? lo : (v > hi ? hi : v);
}

/* Sixteen groups of 16 weights.  Group step = amax/31; the block's d is the
 * largest step over 127 rounded to f16; each group's 8-bit scale is its step
 * in units of d (rounded up so the largest weight still fits in +-31 steps
 * where it can); each weight is the nearest multiple of d*scale in -32..31. */
ORC_API void orc_quantize_q6_k(const float *x, size_t cols, uint8_t *row) {
    for (size_t b = 0; b < cols / KBLOCK; b++) {
        const float *xb = x + b * KBLOCK;
        uint8_t *blk = row + b * Q6_K_BYTES;
        memset(blk, 0, Q6_K_BYTES);
        float step[16], top = 0.0f;
        for (int g = 0; g < 16; g++) {
            float amax = 0.0f;
            for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(xb[g * 16 + i]));
            step[g] = amax * (1.0f / 31.0f);
            top = fmaxf(top, step[g]);
        }
        uint16_t dbits = orc_to_f16(top * (1.0f / 127.0f));
        float d = orc_from_f16(dbits);
        wr16(blk + 208, dbits);
        if (!(d > 0.0f)) continue;
        int8_t *scales = (int8_t *)(blk + 192);
        int q[KBLOCK];
        for (int g = 0; g < 16; g++) {
            int sc = (int)fminf(ceilf(step[g] / d), 127.0f);
            scales[g] = (int8_t)sc;
            float s = d * (float)sc;
            for (int i = 0; i < 16; i++)
                q[g * 16 + i] = sc > 0 ? nearest_multiple(xb[g * 16 + i], s, -32, 31) + 32 : 32;
        }
        for (int half = 0; half < 2; half++)
            for (int l = 0; l < 32; l++)
                for (int k = 0; k < 4; k++) {
                    int v = q[half * 128 + l + 32 * k];
                    blk[half * 64 + l + 32 * (k % 2)] |= (uint8_t)((v & 0xf) << (4 * (k / 2)));
                    blk[128 + half * 32 + l] |= (uint8_t)((v >> 4) << (2 * k));
                }
    }
}

/* Dot of a Q6_K row in the style of gpu/quant.rs:128-152: per 16-weight
 * group eight lane sums of q*x (two passes of eight), lanes folded left to
 * right, times fl(d*scale), accumulated in group order. */
ORC_API float orc_dot_q6_k(const uint8_t *row, const float *x, size_t cols) {
    float acc = 0.0f;
    for (size_t b = 0; b < cols / KBLOCK; b++) {
        const uint8_t *blk = row + b * Q6_K_BYTES;
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t *scales = (const int8_t *)(blk + 192);
        float d = orc_from_f16(rd16(blk + 208));
        const float *xb = x + b * KBLOCK;
        for (int g = 0; g < 16; g++) {
            float sum[8] = {0};
            for (int i = 0; i < 16; i++) {
                int idx = g * 16 + i;               /* weight index in the block */
                int half = idx / 128, r = idx % 128, k = r / 32, l = r % 32;
                int low = (ql[half * 64 + l + 32 * (k % 2)] >> (4 * (k / 2))) & 0xf;
                int high = (qh[half * 32 + l] >> (2 * k)) & 3;
                int q = (low | (high << 4)) - 32;
                sum[i % 8] += (float)q * xb[idx];
            }
            acc += (d * (float)scales[g]) * fold8(sum);
        }
    }
    return acc;
}

/* ------------------------------------------------------------------ */
/* Q4_K — no reference counterpart (parity unpinned)                    */
/* ------------------------------------------------------------------ */
/* Block, 144 bytes, 256 weights in eight sub-blocks of 32:
 *   [0..2)  d     f16   step of the sub-block scales
 *   [2..4)  dmin  f16   step of the sub-block minimums
 *   [4..16) eight 6-bit scales sc_j and eight 6-bit minimums m_j:
 *           j < 4:  sc_j = b[j] & 63,                    m_j = b[j+4] & 63
 *           j >= 4: sc_j = (b[j+4] & 15) | (b[j-4] >> 6) << 4
 *                   m_j  = (b[j+4] >> 4) | (b[j]   >> 6) << 4
 *   [16..144) four groups of 32 bytes; byte i of group g holds weight i of
 *           sub-block 2g in its low nibble and of sub-block 2g+1 in its high.
 * weight = fl(fl(d*sc_j) * q) - fl(dmin*m_j)      (this evaluation order IS
 * the definition of bit-exact for this format). */
static inline void q4k_scale_min(const uint8_t *b, int j, int *sc, int *m) {
    if (j < 4) { *sc = b[j] & 63; *m = b[j + 4] & 63; }
    else {
        *sc = (b[j + 4] & 0xf) | ((b[j - 4] >> 6) << 4);
        *m = (b[j + 4] >> 4) | ((b[j] >> 6) << 4);
    }
}

ORC_API void orc_q4k_unpack_scales(const uint8_t *b12, uint8_t *sc8, uint8_t *m8) {
    for (int j = 0; j < 8; j++) { int s, m; q4k_scale_min(b12, j, &s, &m); sc8[j] = (uint8_t)s; m8[j] = (uint8_t)m; }
}
ORC_API void orc_q4k_pack_scales(const uint8_t *sc8, const uint8_t *m8, uint8_t *b12) {
    memset(b12, 0, 12);
    for (int j = 0; j < 4; j++) {
        b12[j] = (uint8_t)((sc8[j] & 63) | ((sc8[j + 4] >> 4) << 6));
        b12[j + 4] = (uint8_t)((m8[j] & 63) | ((m8[j + 4] >> 4) << 6));
        b12[j + 8] = (uint8_t)((sc8[j + 4] & 0xf) | ((m8[j + 4] & 0xf) << 4));
    }
}

ORC_API void orc_dequantize_q4_k(const uint8_t *row, size_t cols, float *out) {
    for (size_t b = 0; b < cols / KBLOCK; b++) {
        const uint8_t *blk = row + b * Q4_K_BYTES;
        float d = orc_from_f16(rd16(blk)), dmin = orc_from_f16(rd16(blk + 2));
        const uint8_t *qs = blk + 16;
        float *o = out + b * KBLOCK;
        for (int j = 0; j < 8; j++) {
            int sc, m;
            q4k_scale_min(blk + 4, j, &sc, &m);
            float ds = d * (float)sc, dm = dmin * (float)m;
            for (int i = 0; i < 32; i++) {
                int q = (qs[(j / 2) * 32 + i] >> (4 * (j % 2))) & 0xf;
                o[j * 32 + i] = ds * (float)q - dm;
            }
        }
    }
}

/* This repository's Q4_K quantizer.  Per sub-block: lowest = min(0, min x),
 * step = (max x - lowest)/15.  d = f16(largest step / 63), dmin =
 * f16(largest -lowest / 63).  sc_j, m_j = the 6-bit multiples nearest the
 * sub-block's step and -lowest.  q = nearest multiple of d*sc_j to
 * x + dmin*m_j, clamped to 0..15. */
ORC_API void orc_quantize_q4_k(const float *x, size_t cols, uint8_t *row) {
    for (size_t b = 0; b < cols / KBLOCK; b++) {
        const float *xb = x + b * KBLOCK;
        uint8_t *blk = row + b * Q4_K_BYTES;
        memset(blk, 0, Q4_K_BYTES);
        float step[8], low[8], top_step = 0.0f, top_low = 0.0f;
        for (int j = 0; j < 8; j++) {
            float mn = 0.0f, mx = 0.0f;
            for (int i = 0; i < 32; i++) { mn = fminf(mn, xb[j * 32 + i]); mx = fmaxf(mx, xb[j * 32 + i]); }
            low[j] = 0.0f - mn;                            /* >= 0, and +0 (not -0) when mn is 0 */
            step[j] = (mx - mn) * (1.0f / 15.0f);
            top_step = fmaxf(top_step, step[j]);
            top_low = fmaxf(top_low, low[j]);
        }
        uint16_t dbits = orc_to_f16(top_step * (1.0f / 63.0f));
        uint16_t mbits = orc_to_f16(top_low * (1.0f / 63.0f));
        float d = orc_from_f16(dbits), dmin = orc_from_f16(mbits);
        wr16(blk, dbits);
        wr16(blk + 2, mbits);
        uint8_t sc8[8], m8[8];
        for (int j = 0; j < 8; j++) {
            sc8[j] = d > 0.0f ? (uint8_t)nearest_multiple(step[j], d, 0, 63) : 0;
            m8[j] = dmin > 0.0f ? (uint8_t)nearest_multiple(low[j], dmin, 0, 63) : 0;
        }
        orc_q4k_pack_scales(sc8, m8, blk + 4);
        uint8_t *qs = blk + 16;
        for (int j = 0; j < 8; j++) {
            float ds = d * (float)sc8[j], dm = dmin * (float)m8[j];
            for (int i = 0; i < 32; i++) {
                int q = ds > 0.0f ? nearest_multiple(xb[j * 32 + i] + dm, ds, 0, 15) : 0;
                qs[(j / 2) * 32 + i] |= (uint8_t)(q << (4 * (j % 2)));
            }
        }
    }
}

/* Dot of a Q4_K row in the style of gpu/quant.rs:128-152: per sub-block
 * eight lane sums of q*x and eight of x (four passes of eight), each folded
 * left to right; acc += fl(d*sc)*Sqx - fl(dmin*m)*Sx, sub-blocks in order. */
ORC_API float orc_dot_q4_k(const uint8_t *row, const float *x, size_t cols) {
    float acc = 0.0f;
    for (size_t b = 0; b < cols / KBLOCK; b++) {
        const uint8_t *blk = row + b * Q4_K_BYTES;
        float d = orc_from_f16(rd16(blk)), dmin = orc_from_f16(rd16(blk + 2));
        const uint8_t *qs = blk + 16;
        const float *xb = x + b * KBLOCK;
        for (int j = 0; j < 8; j++) {
            int sc, m;
            q4k_scale_min(blk + 4, j, &sc, &m);
            float sq[8] = {0}, sx[8] = {0};
            for (int c = 0; c < 4; c++)
                for (int i = 0; i < 8; i++) {
                    int q = (qs[(j / 2) * 32 + c * 8 + i] >> (4 * (j % 2))) & 0xf;
                    float xv = xb[j * 32 + c * 8 + i];
                    sq[i] += (float)q * xv;
                    sx[i] += xv;
                }
            float a = (d * (float)sc) * fold8(sq);
            float bterm = (dmin * (float)m) * fold8(sx);
            acc += a - bterm;
        }
    }
    return acc;
}

/* ------------------------------------------------------------------ */
/* row-parallel driver (the reference uses rayon's default pool: one    */
/* thread per logical core, gpu/cpu.rs:4, 125-142)                      */
/* ------------------------------------------------------------------ */
#include <pthread.h>
#include <unistd.h>

typedef void (*row_fn)(size_t r, void *ctx);
typedef struct { row_fn fn; void *ctx; size_t begin, end; } row_job;

static int g_threads = 0;

ORC_API int orc_threads(void) {
    if (g_threads <= 0) {
        const char *e = getenv("ORC_THREADS");
        long n = e ? atol(e) : sysconf(_SC_NPROCESSORS_ONLN);
        g_threads = n < 1 ? 1 : (n > 256 ? 256 : (int)n);
    }
    return g_threads;
}
ORC_API void orc_set_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }

static void *row_worker(void *arg) {
    row_job *j = (row_job *)arg;
    for (size_t r = j->begin; r < j->end; r++) j->fn(r, j->ctx);
    return NULL;
}

/* Contiguous chunks of rows, one per thread; the arithmetic of a row does
 * not depend on the split. */
static void for_rows(size_t rows, row_fn fn, void *ctx) {
    int nt = orc_threads();
    if ((size_t)nt > rows) nt = rows ? (int)rows : 1;
    if (nt <= 1) { for (size_t r = 0; r < rows; r++) fn(r, ctx); return; }
    pthread_t tid[256];
    row_job job[256];
    size_t per = (rows + (size_t)nt - 1) / (size_t)nt;
    int started = 0;
    for (int t = 0; t < nt; t++) {
        size_t b = (size_t)t * per, e = b + per > rows ? rows : b + per;
        if (b >= e) break;
        job[t] = (row_job){fn, ctx, b, e};
        if (pthread_create(&tid[t], NULL, row_worker, &job[t]) != 0) { row_worker(&job[t]); tid[t] = 0; }
        started = t + 1;
    }
    for (int t = 0; t < started; t++) if (tid[t]) pthread_join(tid[t], NULL);
}

/* ------------------------------------------------------------------ */
/* gpu/cpu.rs — the CPU device's operators for this path                */
/* ------------------------------------------------------------------ */
enum { ORC_Q8_0 = 8, ORC_Q4_K = 12, ORC_Q6_K = 14 };   /* GGUF type ids */

ORC_API size_t orc_row_bytes(int fmt, size_t cols) {
    switch (fmt) {
    case ORC_Q8_0: return cols / BLOCK * Q8_0_BYTES;
    case ORC_Q4_K: return cols / KBLOCK * Q4_K_BYTES;
    case ORC_Q6_K: return cols / KBLOCK * Q6_K_BYTES;
    default: return 0;
    }
}

static float row_dot(int fmt, const uint8_t *row, const float *x, size_t cols) {
    switch (fmt) {
    case ORC_Q8_0: return orc_dot_q8_0(row, x, cols);
    case ORC_Q4_K: return orc_dot_q4_k(row, x, cols);
    default: return orc_dot_q6_k(row, x, cols);
    }
}

/* gpu/cpu.rs:110-149 — parallel over weight rows (rayon there, OpenMP here;
 * the schedule does not touch the arithmetic: each out[t*rows+r] is one
 * row's dot with one token, accumulated in block order).  out is
 * token-major: out[t*rows + r]. */
typedef struct { int fmt; const uint8_t *w; size_t rows, cols, rb, n; const float *x; float *out; } mm_ctx;
static void mm_row(size_t r, void *p) {
    mm_ctx *c = (mm_ctx *)p;
    for (size_t t = 0; t < c->n; t++)
        c->out[t * c->rows + r] = row_dot(c->fmt, c->w + r * c->rb, c->x + t * c->cols, c->cols);
}
ORC_API int orc_matmul(int fmt, const uint8_t *w, size_t rows, size_t cols,
                       const float *x, size_t n, float *out) {
    size_t rb = orc_row_bytes(fmt, cols);
    if (rb == 0) return -1;
    mm_ctx c = {fmt, w, rows, cols, rb, n, x, out};
    for_rows(rows, mm_row, &c);
    return 0;
}

/* gpu/mod.rs:256-268 (default body) + gpu/cpu.rs:151-155: x += w . input */
ORC_API int orc_matmul_add(int fmt, const uint8_t *w, size_t rows, size_t cols,
                           const float *input, size_t n, float *x) {
    float *scratch = (float *)malloc(n * rows * sizeof(float));
    if (!scratch) return -2;
    int rc = orc_matmul(fmt, w, rows, cols, input, n, scratch);
    if (rc == 0) for (size_t i = 0; i < n * rows; i++) x[i] += scratch[i];
    free(scratch);
    return rc;
}

/* gpu/cpu.rs:425-427 sigmoid = 1/(1+exp(-x)); gpu/cpu.rs:238-242 silu_mul:
 * g = g * sigmoid(g) * u, left to right. */
static inline float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

/* gpu/mod.rs:270-285 (default body): out = silu(gate.x) * (up.x) */
ORC_API int orc_swiglu(int fmt, const uint8_t *gate, const uint8_t *up, size_t rows, size_t cols,
                       const float *x, size_t n, float *out) {
    float *scratch = (float *)malloc(n * rows * sizeof(float));
    if (!scratch) return -2;
    int rc = orc_matmul(fmt, gate, rows, cols, x, n, out);
    if (rc == 0) rc = orc_matmul(fmt, up, rows, cols, x, n, scratch);
    if (rc == 0) for (size_t i = 0; i < n * rows; i++) out[i] = out[i] * sigmoidf_(out[i]) * scratch[i];
    free(scratch);
    return rc;
}

/* Tensor::dequantize (gpu/mod.rs:138-168) for the GGUF layouts. */
typedef struct { int fmt; const uint8_t *w; size_t cols, rb; float *f; uint8_t *q; const float *src; } codec_ctx;
static void deq_row(size_t r, void *p) {
    codec_ctx *c = (codec_ctx *)p;
    const uint8_t *row = c->w + r * c->rb;
    float *o = c->f + r * c->cols;
    if (c->fmt == ORC_Q8_0) orc_dequantize_q8_0(row, c->cols, o);
    else if (c->fmt == ORC_Q4_K) orc_dequantize_q4_k(row, c->cols, o);
    else orc_dequantize_q6_k(row, c->cols, o);
}
ORC_API int orc_dequantize(int fmt, const uint8_t *w, size_t rows, size_t cols, float *out) {
    size_t rb = orc_row_bytes(fmt, cols);
    if (rb == 0) return -1;
    codec_ctx c = {fmt, w, cols, rb, out, NULL, NULL};
    for_rows(rows, deq_row, &c);
    return 0;
}

static void q_row(size_t r, void *p) {
    codec_ctx *c = (codec_ctx *)p;
    const float *row = c->src + r * c->cols;
    uint8_t *o = c->q + r * c->rb;
    if (c->fmt == ORC_Q8_0) orc_quantize_q8_0(row, c->cols, o);
    else if (c->fmt == ORC_Q4_K) orc_quantize_q4_k(row, c->cols, o);
    else orc_quantize_q6_k(row, c->cols, o);
}
ORC_API int orc_quantize(int fmt, const float *w, size_t rows, size_t cols, uint8_t *out) {
    size_t rb = orc_row_bytes(fmt, cols);
    if (rb == 0) return -1;
    codec_ctx c = {fmt, NULL, cols, rb, NULL, out, w};
    for_rows(rows, q_row, &c);
    return 0;
}

/* ---- the operators either side of the product ---------------------------------- */

/* Cpu::rmsnorm, gpu/cpu.rs:157-166: per row of `dim`, mean_square = (left fold of
 * v*v from 0.0) / dim; scale = 1.0 / sqrt(mean_square + eps); v *= scale * w.
 * Device::normalize (gpu/mod.rs:295-305) is a copy followed by this. */
ORC_API void orc_rmsnorm(float *x, size_t n, const float *weight, size_t dim, float eps) {
    for (size_t t = 0; t < n; t++) {
        float *row = x + t * dim;
        float sum = 0.0f;
        for (size_t i = 0; i < dim; i++) sum += row[i] * row[i];
        float mean_square = sum / (float)dim;
        float scale = 1.0f / sqrtf(mean_square + eps);
        for (size_t i = 0; i < dim; i++) row[i] *= scale * weight[i];
    }
}

/* gpu/cpu.rs:370-384: eight running sums over chunks of eight, the rest summed
 * on its own, then (left fold of the eight from 0.0) + rest. */
ORC_API float orc_dot_bf16(const uint16_t *w, const float *x, size_t cols) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t done = cols / 8 * 8;
    for (size_t k = 0; k < done; k += 8)
        for (int i = 0; i < 8; i++) acc[i] += orc_bf16(w[k + i]) * x[k + i];
    float rest = 0.0f;
    for (size_t k = done; k < cols; k++) rest += orc_bf16(w[k]) * x[k];
    return fold8(acc) + rest;
}

/* Cpu::matmul's Bf16 arm, gpu/cpu.rs:124-128, 144-148: token-major output. */
typedef struct { const uint16_t *w; size_t rows, cols; const float *x; size_t n; float *out; } bf16_ctx;
static void bf16_row(size_t r, void *p) {
    bf16_ctx *c = (bf16_ctx *)p;
    for (size_t t = 0; t < c->n; t++) c->out[t * c->rows + r] = orc_dot_bf16(c->w + r * c->cols, c->x + t * c->cols, c->cols);
}
ORC_API int orc_matmul_bf16(const uint16_t *w, size_t rows, size_t cols, const float *x, size_t n, float *out) {
    bf16_ctx c = {w, rows, cols, x, n, out};
    for_rows(rows, bf16_row, &c);
    return 0;
}

/* inference/qwen35/mod.rs:702-710: the first index of the largest value
 * (a later equal value does not replace it; index 0 if nothing compares greater). */
ORC_API uint32_t orc_argmax(const float *logits, size_t n) {
    size_t best = 0;
    for (size_t i = 0; i < n; i++)
        if (logits[i] > logits[best]) best = i;
    return (uint32_t)best;
}
