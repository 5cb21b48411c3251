// Block formats as they sit in device memory, and the bit-exact decoders.
//
// GGUF ("file") layouts, as the host hands them over:
//   Q8_0  34 B / 32 w : [d f16][32 x i8]                    (inference/quants.rs:59-71)
//   Q4_K 144 B / 256 w: [d f16][dmin f16][12 B scales][128 B nibbles]
//   Q6_K 210 B / 256 w: [ql 128][qh 64][scales 16 x i8][d f16] (inference/quants.rs:73-104)
//
// Device layouts.  Q4_K blocks are already 16-byte aligned and stay as they
// are.  Q8_0 and Q6_K blocks are 2-byte aligned in the file, so upload parts
// them — as the reference parts Q4_0/Q8_0 scales from quants
// (gpu/quant.rs:1-12) — into a 16-byte aligned quant array and an f16 scale
// array, both row-major with rows padded to 16 bytes:
//   Q8_0: quants [rows][cols] i8                scales [rows][pad8(cols/32)] f16
//   Q6_K: quants [rows][cols/256][208]          scales [rows][pad8(cols/256)] f16
//         (208 = ql 128 | qh 64 | sub-scales 16)
// Rows of every quant array sit `qpitch` bytes apart: the row's bytes rounded
// up to an odd number of 16-byte steps.  A tile of consecutive rows is then
// one contiguous run of HBM (one bulk copy into shared memory) and, once
// there, the eight rows a warp reads together fall in different banks.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace dwim {

enum Format : int { Q8_0 = 8, Q4_K = 12, Q6_K = 14, BF16 = 30 };   // GGUF's type ids (inference/gguf.rs:28-33)

constexpr int Q8_0_FILE = 34, Q4_K_FILE = 144, Q6_K_FILE = 210;
constexpr int Q6_K_DEV = 208;

__host__ __device__ inline size_t pad8(size_t n) { return (n + 7) & ~size_t(7); }

// Weights per scale unit along K.
__host__ __device__ inline int block_weights(int fmt) { return fmt == BF16 ? 1 : fmt == Q8_0 ? 32 : 256; }
__host__ __device__ inline size_t file_row_bytes(int fmt, size_t cols) {
    switch (fmt) {
    case Q8_0: return cols % 32 ? 0 : cols / 32 * Q8_0_FILE;
    case Q4_K: return cols % 256 ? 0 : cols / 256 * Q4_K_FILE;
    case Q6_K: return cols % 256 ? 0 : cols / 256 * Q6_K_FILE;
    case BF16: return cols * 2;
    default: return 0;
    }
}
// Bytes of one row of the device quant array, and f16 entries of one row of
// the device scale array (0 for Q4_K, whose scales stay in the block).
__host__ __device__ inline size_t dev_quant_row_bytes(int fmt, size_t cols) {
    switch (fmt) {
    case Q8_0: return cols;
    case Q4_K: return cols / 256 * Q4_K_FILE;
    case BF16: return cols * 2;
    default: return cols / 256 * Q6_K_DEV;
    }
}
__host__ __device__ inline size_t dev_quant_pitch(int fmt, size_t cols) {
    size_t b = dev_quant_row_bytes(fmt, cols);
    if (fmt == BF16) return b;   // plain rows (cols is a multiple of 8: 16-byte aligned)
    return (b / 16) % 2 == 0 ? b + 16 : b;
}
__host__ __device__ inline size_t dev_scale_row_elems(int fmt, size_t cols) {
    switch (fmt) {
    case Q8_0: return pad8(cols / 32);
    case Q6_K: return pad8(cols / 256);
    default: return 0;
    }
}

// A weight matrix in device memory.
struct WeightView {
    int fmt;
    size_t rows, cols;
    const uint8_t *quants;   // [rows][qpitch]
    const __half *scales;    // [rows][srow] (null for Q4_K)
    size_t qrow;             // bytes of quants in a row
    size_t qpitch;           // bytes from one row to the next
    size_t srow;             // f16 per row of scales
};

// ---- f16 ------------------------------------------------------------------
// gpu/float.rs:38-48: exact.
__device__ __forceinline__ float from_f16_bits(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }
// gpu/float.rs:13-28: nearest even, clamped to +-65504 instead of overflowing.
// The conversion goes through PTX and comes back as a 32-bit integer: with
// the 16-bit intrinsic types the compiler was seen to drop the low byte of
// the result when it was stored a byte at a time.
__device__ __forceinline__ uint32_t to_f16_bits(float x) {
    float a = fminf(fabsf(x), 65504.0f);
    uint32_t h;
    asm("{\n\t.reg .b16 t;\n\tcvt.rn.f16.f32 t, %1;\n\tmov.b32 %0, {t, t};\n\t}" : "=r"(h) : "f"(a));
    return (h & 0x7fffu) | ((__float_as_uint(x) >> 16) & 0x8000u);
}
__device__ __forceinline__ __half to_f16_clamped(float x) { return __ushort_as_half((unsigned short)to_f16_bits(x)); }

// ---- Q4_K -----------------------------------------------------------------
// The 6-bit scale and minimum of sub-block j from the block's 12 bytes.
__device__ __forceinline__ void q4k_scale_min(const uint8_t *b, int j, int &sc, int &m) {
    if (j < 4) { sc = b[j] & 63; m = b[j + 4] & 63; }
    else {
        sc = (b[j + 4] & 0xf) | ((b[j - 4] >> 6) << 4);
        m = (b[j + 4] >> 4) | ((b[j] >> 6) << 4);
    }
}
// weight i (0..255) of a Q4_K block: fl(fl(d*sc)*q) - fl(dmin*m); the
// intrinsics keep the compiler from contracting the products into an FMA.
__device__ __forceinline__ float q4k_weight(const uint8_t *blk, int i) {
    float d = from_f16_bits(*(const uint16_t *)blk), dmin = from_f16_bits(*(const uint16_t *)(blk + 2));
    int j = i >> 5, sc, m;
    q4k_scale_min(blk + 4, j, sc, m);
    int q = (blk[16 + (j >> 1) * 32 + (i & 31)] >> (4 * (j & 1))) & 0xf;
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
}

// ---- Q6_K (device block: ql[128] qh[64] sc[16]) ------------------------------
__device__ __forceinline__ int q6k_quant(const uint8_t *blk, int i) {
    int half = i >> 7, r = i & 127, k = r >> 5, l = r & 31;
    int low = (blk[half * 64 + l + 32 * (k & 1)] >> (4 * (k >> 1))) & 0xf;
    int high = (blk[128 + half * 32 + l] >> (2 * k)) & 3;
    return (low | (high << 4)) - 32;
}
// inference/quants.rs:99: (d * scale) * q, left to right.
__device__ __forceinline__ float q6k_weight(const uint8_t *blk, float d, int i) {
    int sc = (int8_t)blk[192 + (i >> 4)];
    return __fmul_rn(__fmul_rn(d, (float)sc), (float)q6k_quant(blk, i));
}

}  // namespace dwim
