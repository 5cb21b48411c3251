// The small-M product (decode and speculative verify): out[t][r] = w[r] . x[t]
// for up to eight tokens, bound by how fast the packed weights stream from HBM.
//
// Replaces the reference's matmul_tile16_* / matmul_rows* kernels for few
// tokens (matmul_tile.cu:94-258, matmul_rows.cu:29-184; dispatch at
// gpu/cuda/mod.rs:1084-1131).
//
// Shape of the kernel
//   - Persistent grid, one CTA per SM.  A CTA walks tiles of R = 16*RT weight
//     rows; for each tile it streams the rows' packed blocks, K in chunks of
//     `kc` units of 256 weights, through a ring of shared-memory stages.
//   - One producer warp fills the ring with cp.async.bulk (the TMA engine's
//     untiled copy): a stage of whole rows is one contiguous run of HBM and one
//     copy (plus one for the rows' scales where the format keeps them apart);
//     longer rows are cut in chunks, one copy per row and chunk.  Stages are
//     handed over with mbarriers (full: transaction bytes; empty: one arrival
//     per consumer warp).  Every wait is bounded.
//   - RT*KS consumer warps.  Warp (rt, ks) owns row tile rt and every KS-th
//     unit of a chunk.  The quants stay integers: nibbles (Q4_K) are masked
//     four at a time, Q6_K's six bits assembled into signed bytes, Q8_0's bytes
//     used as they are, and multiplied on the tensor cores (mma.sync int8,
//     weight rows on the M side) with the activations' signed base-256 digit
//     planes as columns (prologue.cu).  The integer sums of a sub-block are
//     weighted by its scale (integer multiply-add for the 6-bit and 8-bit
//     sub-scales, fp32 for Q8_0's f16 ones), and the unit's d and the plane's
//     worth scale once per unit in fp32: the result differs from the CPU's by
//     fp32 summation order and the planes' rounding (2^-31 or 2^-23 of a unit's
//     largest activation).
//   - The K-split warps of a row tile are summed through shared memory in a
//     fixed order (deterministic), then the epilogue stores, adds to, or
//     SwiGLU-combines the output (modes after prelude.cu:29-35).
#include <cuda_fp16.h>
#include <stdlib.h>

#include "common.cuh"
#include "ptx.cuh"

namespace dwim {

constexpr int MAX_STAGES = 8;

struct GemvArgs {
    WeightView w;
    const uint8_t *panels;   // [units][i8_unit_bytes(ncols)]: the activations' digit planes (prologue.cu)
    int xunit;               // bytes of one unit's panels for this launch
    int xsrc_stride;         // bytes between units in the panel array
    // SwiGLU in one launch (int8 routine): `w` is the gate matrix, these the quants and scales of
    // the up matrix of the same shape; a CTA takes a row tile of the one, then of the other, and
    // writes silu(gate . x) * (up . x).  Null: an ordinary product.
    const uint8_t *up_quants;
    const __half *up_scales;
    int ncols;               // digit-plane columns: planes * tokens
    int n_tokens;            // tokens of this launch
    size_t t0;               // first token's index in out
    OutSpec out;
    const float *aux;        // EPI_SWIGLU: the `up` product, token-major [n][rows]
    int epi;
    int units;               // ceil(cols / 256)
    int kc;                  // units per stage
    int n_tiles;
    int stages;
    int q_stride;            // bytes between rows of a stage's quant region
    int s_off, s_stride;     // scale region
    int x_off;               // panel region (when the panels travel with the stages)
    int stage_bytes;
    int whole_rows;          // 1: a stage holds whole rows (kc == units): one copy for the tile's quants, one for its scales
    int x_resident;          // 1: the launch's panels sit in shared memory for the CTA's whole life
    int xres_bytes;
    uint32_t *status;
};


// Q4_K through the int8 tensor-core path (one or two tokens): the same blocks,
// another activation operand and unit routine.
constexpr int Q4K_I8 = 1012;
constexpr int Q8_I8 = 1008;     // Q8_0 and Q6_K through the same int8 path (up to eight tokens)
constexpr int Q6K_I8 = 1014;
constexpr bool is_i8(int fmt) { return fmt == Q4K_I8 || fmt == Q8_I8 || fmt == Q6K_I8; }
constexpr int base_of(int fmt) { return fmt == Q4K_I8 ? (int)Q4_K : fmt == Q8_I8 ? (int)Q8_0 : fmt == Q6K_I8 ? (int)Q6_K : fmt; }

template <int FMT> struct Traits;
template <> struct Traits<Q4K_I8> { static constexpr int UNIT_Q = 144; };
template <> struct Traits<Q8_I8> { static constexpr int UNIT_Q = 256; };
template <> struct Traits<Q6K_I8> { static constexpr int UNIT_Q = 208; };

// What a consumer lane needs to know about the stage it reads.
struct Lane {
    int g, c;                // row within the 8-row group; k-quarter
    uint32_t row_a, row_b;   // shared addresses of rows g and g+8 (quant region)
    uint32_t srow_a, srow_b; // shared addresses of the rows' scales
    uint32_t xbase;          // shared address of the launch's panels (unit 0 of the stage, or of the row when resident)
};

// ---------------------------------------------------------------------------
// Q4_K, one or two tokens, int8 tensor-core path
// ---------------------------------------------------------------------------
// The nibbles stay integers: four of them per AND, multiplied on the tensor
// cores (mma.sync m16n8k32 u8 x s8 -> s32) with the activations' signed
// base-256 digit planes as columns (prologue.cu: column = 4*token + plane).
// One MMA covers one 32-weight sub-block of 16 rows; its sums are weighted by
// the sub-block's 6-bit scale with integer multiply-adds, so a whole unit is an
// exact integer per (row, column), which d and the plane's worth then scale.
// High nibbles are masked in place (16*q: no shift) and their sums divided by
// 16 once per unit.  The minimums use the digits' per-sub-block sums (dp4a).
// About half the instructions of the f16 routine above for the same weights.
// c = a * b (the accumulator operand is zero, not a register that has to be cleared first)
__device__ __forceinline__ void imma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {   // a unsigned bytes, b signed bytes
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ float2 lds64f2(uint32_t a) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
    return v;
}

__device__ __forceinline__ void imma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// 16 rows x 16 k: one 16-weight scale group of Q6_K
__device__ __forceinline__ void imma16_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
__device__ __forceinline__ float lds32f(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}

// The digit planes' columns as the int8 routines see them: NTILE column tiles
// of the MMA (8 columns each).  Tile p's column g is blob column
// p*tile_stride + g, present when g < tile_cols.
//   one and two tokens:  one tile, column = 4*token + plane, tile_cols = 4n
//   three to eight:      a tile per plane, column g = token g, tile_stride = tile_cols = n
// In both a lane's accumulators are (row a | row b) x (tile column 2c, 2c+1).
struct I8Cols {
    int nc;           // columns in a unit's blob
    int tile_stride;
    int tile_cols;
};

// Q4_K.  Lane (g, c) owns bytes [8c, 8c+8) of each 32-byte group of its two rows: MMA
// k-slots 4c..4c+3 and 16+4c..16+4c+3, matched by the same eight digits of the
// lane's column.  acc: (row a, col 2c), (row a, col 2c+1), (row b, ..), (row b, ..),
// summed over the tiles (the planes of a token, in the layout of three to eight tokens).
template <int NTILE>
__device__ __forceinline__ void unit_q4k_i8(const Lane &L, const I8Cols X, int ul, int xu, float (&acc)[4]) {
    const uint32_t ba = L.row_a + ul * 144, bb = L.row_b + ul * 144;
    const uint4 ha = lds128(ba), hb = lds128(bb);
    const uint32_t blob = L.xbase + xu * i8_unit_bytes(X.nc);
    const bool bcol = L.g < X.tile_cols;   // this lane's B column exists
    // the 6-bit scales and minimums as bytes: entries 0..3 and 4..7
    const uint32_t sa[2] = {ha.y & 0x3f3f3f3fu, (ha.w & 0x0f0f0f0fu) | ((ha.y >> 2) & 0x30303030u)};
    const uint32_t sb[2] = {hb.y & 0x3f3f3f3fu, (hb.w & 0x0f0f0f0fu) | ((hb.y >> 2) & 0x30303030u)};
    int ilo[NTILE][4], ihi[NTILE][4];
#pragma unroll
    for (int p = 0; p < NTILE; p++)
#pragma unroll
        for (int i = 0; i < 4; i++) ilo[p][i] = ihi[p][i] = 0;
    const uint32_t qa = ba + 16 + 8 * L.c, qb = bb + 16 + 8 * L.c;
    uint32_t xcol = blob + L.g * 32 + 8 * L.c;      // this lane's column of tile 0, sub-block 0
    const uint32_t xstep = 32 * X.nc;                // a sub-block further on
    const uint32_t tstep = 32 * X.tile_stride;       // a tile further on
#pragma unroll
    for (int G = 0; G < 4; G++) {   // group G: low nibbles = sub-block 2G, high nibbles = 2G+1
        const uint2 wa = lds64(qa + 32 * G), wb = lds64(qb + 32 * G);
        // the two sub-blocks' scales: bytes 2(G&1) and 2(G&1)+1 of the word, each by one byte permute
        const int s0a = (int)prmt(sa[G >> 1], 0u, 0x4440u + 2 * (G & 1)), s1a = (int)prmt(sa[G >> 1], 0u, 0x4441u + 2 * (G & 1));
        const int s0b = (int)prmt(sb[G >> 1], 0u, 0x4440u + 2 * (G & 1)), s1b = (int)prmt(sb[G >> 1], 0u, 0x4441u + 2 * (G & 1));
#pragma unroll
        for (int p = 0; p < NTILE; p++) {
            uint2 x0 = make_uint2(0, 0), x1 = make_uint2(0, 0);
            if (bcol) {
                x0 = lds64(xcol + p * tstep);
                x1 = lds64(xcol + p * tstep + xstep);
            }
            int c0[4], c1[4];
            imma_u8s8(c0, wa.x & 0x0f0f0f0fu, wb.x & 0x0f0f0f0fu, wa.y & 0x0f0f0f0fu, wb.y & 0x0f0f0f0fu, x0.x, x0.y);
            imma_u8s8(c1, wa.x & 0xf0f0f0f0u, wb.x & 0xf0f0f0f0u, wa.y & 0xf0f0f0f0u, wb.y & 0xf0f0f0f0u, x1.x, x1.y);
            ilo[p][0] += s0a * c0[0]; ilo[p][1] += s0a * c0[1]; ilo[p][2] += s0b * c0[2]; ilo[p][3] += s0b * c0[3];
            ihi[p][0] += s1a * c1[0]; ihi[p][1] += s1a * c1[1]; ihi[p][2] += s1b * c1[2]; ihi[p][3] += s1b * c1[3];
        }
        xcol += 2 * xstep;
    }
    // minimums: sum_j m_j * (128*a_j + b_j) per column
    const uint32_t ma[2] = {ha.z & 0x3f3f3f3fu, ((ha.w >> 4) & 0x0f0f0f0fu) | ((ha.z >> 2) & 0x30303030u)};
    const uint32_t mb[2] = {hb.z & 0x3f3f3f3fu, ((hb.w >> 4) & 0x0f0f0f0fu) | ((hb.z >> 2) & 0x30303030u)};
    const float da = h2f_lo(ha.x), dma = h2f_hi(ha.x), db = h2f_lo(hb.x), dmb = h2f_hi(hb.x);
    if constexpr (NTILE == 1) {
        // one tile of 4n columns: the lane's two columns exist together, their sums and worths sit side by side
        uint4 t0 = make_uint4(0, 0, 0, 0), t1 = t0;
        float2 worth = make_float2(0.0f, 0.0f);
        if (2 * L.c < X.tile_cols) {
            t0 = lds128(blob + 256 * X.nc + (2 * L.c) * 16);
            t1 = lds128(blob + 256 * X.nc + (2 * L.c + 1) * 16);
            worth = lds64f2(blob + 272 * X.nc + 8 * L.c);
        }
        const int m0 = (dp4a_us(ma[1], t0.y, dp4a_us(ma[0], t0.x, 0)) << 7) + dp4a_us(ma[1], t0.w, dp4a_us(ma[0], t0.z, 0));
        const int m1 = (dp4a_us(ma[1], t1.y, dp4a_us(ma[0], t1.x, 0)) << 7) + dp4a_us(ma[1], t1.w, dp4a_us(ma[0], t1.z, 0));
        const int m2 = (dp4a_us(mb[1], t0.y, dp4a_us(mb[0], t0.x, 0)) << 7) + dp4a_us(mb[1], t0.w, dp4a_us(mb[0], t0.z, 0));
        const int m3 = (dp4a_us(mb[1], t1.y, dp4a_us(mb[0], t1.x, 0)) << 7) + dp4a_us(mb[1], t1.w, dp4a_us(mb[0], t1.z, 0));
        acc[0] += worth.x * (da * (float)(ilo[0][0] + (ihi[0][0] >> 4)) - dma * (float)m0);
        acc[1] += worth.y * (da * (float)(ilo[0][1] + (ihi[0][1] >> 4)) - dma * (float)m1);
        acc[2] += worth.x * (db * (float)(ilo[0][2] + (ihi[0][2] >> 4)) - dmb * (float)m2);
        acc[3] += worth.y * (db * (float)(ilo[0][3] + (ihi[0][3] >> 4)) - dmb * (float)m3);
    } else {
#pragma unroll
        for (int p = 0; p < NTILE; p++)
#pragma unroll
            for (int i = 0; i < 2; i++) {
                uint4 t = make_uint4(0, 0, 0, 0);
                float worth = 0.0f;
                if (2 * L.c + i < X.tile_cols) {
                    const int col = p * X.tile_stride + 2 * L.c + i;
                    t = lds128(blob + 256 * X.nc + col * 16);
                    worth = lds32f(blob + 272 * X.nc + 4 * col);
                }
                const int m_a = (dp4a_us(ma[1], t.y, dp4a_us(ma[0], t.x, 0)) << 7) + dp4a_us(ma[1], t.w, dp4a_us(ma[0], t.z, 0));
                const int m_b = (dp4a_us(mb[1], t.y, dp4a_us(mb[0], t.x, 0)) << 7) + dp4a_us(mb[1], t.w, dp4a_us(mb[0], t.z, 0));
                acc[i] += worth * (da * (float)(ilo[p][i] + (ihi[p][i] >> 4)) - dma * (float)m_a);
                acc[2 + i] += worth * (db * (float)(ilo[p][2 + i] + (ihi[p][2 + i] >> 4)) - dmb * (float)m_b);
            }
    }
}

// Q8_0.  A 32-weight block is one MMA (s8 x s8); its f16 scale weighs the block's
// integer sums in fp32.  Lane c owns bytes [8c, 8c+8) of each block.
template <int NTILE>
__device__ __forceinline__ void unit_q8_i8(const Lane &L, const I8Cols X, int ul, int xu, float (&acc)[4]) {
    const uint32_t qa = L.row_a + ul * 256 + 8 * L.c, qb = L.row_b + ul * 256 + 8 * L.c;
    const uint4 sa = lds128(L.srow_a + ul * 16), sb = lds128(L.srow_b + ul * 16);
    const uint32_t sca[4] = {sa.x, sa.y, sa.z, sa.w}, scb[4] = {sb.x, sb.y, sb.z, sb.w};
    const uint32_t blob = L.xbase + xu * i8_unit_bytes(X.nc);
    const bool bcol = L.g < X.tile_cols;
    float fs[NTILE][4];
#pragma unroll
    for (int p = 0; p < NTILE; p++)
#pragma unroll
        for (int i = 0; i < 4; i++) fs[p][i] = 0.0f;
    uint32_t xcol = blob + L.g * 32 + 8 * L.c;
    const uint32_t xstep = 32 * X.nc, tstep = 32 * X.tile_stride;
#pragma unroll
    for (int blk = 0; blk < 8; blk++) {
        const uint2 wa = lds64(qa + 32 * blk), wb = lds64(qb + 32 * blk);
        const float da = (blk & 1) ? h2f_hi(sca[blk >> 1]) : h2f_lo(sca[blk >> 1]);
        const float db = (blk & 1) ? h2f_hi(scb[blk >> 1]) : h2f_lo(scb[blk >> 1]);
#pragma unroll
        for (int p = 0; p < NTILE; p++) {
            uint2 x = make_uint2(0, 0);
            if (bcol) x = lds64(xcol + p * tstep);
            int c[4];
            imma_s8s8(c, wa.x, wb.x, wa.y, wb.y, x.x, x.y);
            fs[p][0] += da * (float)c[0];
            fs[p][1] += da * (float)c[1];
            fs[p][2] += db * (float)c[2];
            fs[p][3] += db * (float)c[3];
        }
        xcol += xstep;
    }
#pragma unroll
    for (int p = 0; p < NTILE; p++)
#pragma unroll
        for (int i = 0; i < 2; i++) {
            float worth = 0.0f;
            if (2 * L.c + i < X.tile_cols) worth = lds32f(blob + 272 * X.nc + 4 * (p * X.tile_stride + 2 * L.c + i));
            acc[i] += worth * fs[p][i];
            acc[2 + i] += worth * fs[p][2 + i];
        }
}

// Q6_K.  One MMA of k = 16 per 16-weight scale group: lane c holds weights
// 4c..4c+3 of the group as signed bytes; the group's i8 sub-scale weighs its
// integer sums, d the unit's.  For (half, lh) the lane reads two ql words and
// one qh word per row and makes the four groups k = 0..3 from them.
__device__ __forceinline__ uint32_t q6_signed(uint32_t low, uint32_t high2) {
    // bytes low | high2 hold q + 32 in [0, 63]; flipping bit 5 gives q's 6-bit two's
    // complement, whose sign bit is then copied into bits 6 and 7
    const uint32_t t = (low | high2) ^ 0x20202020u, sgn = t & 0x20202020u;
    return t | (sgn << 1) | (sgn << 2);
}
template <int NTILE>
__device__ __forceinline__ void unit_q6k_i8(const Lane &L, const I8Cols X, int ul, int xu, int d_index, float (&acc)[4]) {
    const uint32_t ba = L.row_a + ul * 208, bb = L.row_b + ul * 208;
    const uint4 ta = lds128(ba + 192), tb = lds128(bb + 192);
    const uint32_t sca[4] = {ta.x, ta.y, ta.z, ta.w}, scb[4] = {tb.x, tb.y, tb.z, tb.w};
    const float da = __half2float(__ushort_as_half((uint16_t)lds16(L.srow_a + 2 * d_index)));
    const float db = __half2float(__ushort_as_half((uint16_t)lds16(L.srow_b + 2 * d_index)));
    const uint32_t blob = L.xbase + xu * i8_unit_bytes(X.nc);
    const bool bcol = L.g < X.tile_cols;
    int is[NTILE][4];
#pragma unroll
    for (int p = 0; p < NTILE; p++)
#pragma unroll
        for (int i = 0; i < 4; i++) is[p][i] = 0;
    const uint32_t xlane = blob + L.g * 32 + 4 * L.c;
    const uint32_t xstep = 32 * X.nc, tstep = 32 * X.tile_stride;
#pragma unroll
    for (int hf = 0; hf < 2; hf++)
#pragma unroll
        for (int lh = 0; lh < 2; lh++) {
            const uint32_t o = 64 * hf + 16 * lh + 4 * L.c, oh = 128 + 32 * hf + 16 * lh + 4 * L.c;
            const uint32_t la0 = lds32(ba + o), la1 = lds32(ba + o + 32), hha = lds32(ba + oh);
            const uint32_t lb0 = lds32(bb + o), lb1 = lds32(bb + o + 32), hhb = lds32(bb + oh);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const uint32_t la = (k & 1) ? la1 : la0, lb = (k & 1) ? lb1 : lb0;
                const uint32_t lowa = ((k >> 1) ? (la >> 4) : la) & 0x0f0f0f0fu;
                const uint32_t lowb = ((k >> 1) ? (lb >> 4) : lb) & 0x0f0f0f0fu;
                const uint32_t ha = (k == 0 ? hha << 4 : k == 1 ? hha << 2 : k == 2 ? hha : hha >> 2) & 0x30303030u;
                const uint32_t hb = (k == 0 ? hhb << 4 : k == 1 ? hhb << 2 : k == 2 ? hhb : hhb >> 2) & 0x30303030u;
                const uint32_t qa = q6_signed(lowa, ha), qb = q6_signed(lowb, hb);
                const int sidx = 8 * hf + 2 * k + lh;
                // byte sidx & 3 of the word, sign-extended (a selector nibble of 8 + b replicates byte b's sign)
                constexpr uint32_t SEXT = 0x8880u;
                const int fa = (int)prmt(sca[sidx >> 2], 0u, SEXT + (sidx & 3) * 0x1111u);
                const int fb = (int)prmt(scb[sidx >> 2], 0u, SEXT + (sidx & 3) * 0x1111u);
                // sub-block 4*hf + k of the unit, digits 16*lh + 4c .. +3
                const uint32_t xo = (4 * hf + k) * xstep + 16 * lh;
#pragma unroll
                for (int p = 0; p < NTILE; p++) {
                    uint32_t x = 0;
                    if (bcol) x = lds32(xlane + xo + p * tstep);
                    int c[4];
                    imma16_s8s8(c, qa, qb, x);
                    is[p][0] += fa * c[0];
                    is[p][1] += fa * c[1];
                    is[p][2] += fb * c[2];
                    is[p][3] += fb * c[3];
                }
            }
        }
#pragma unroll
    for (int p = 0; p < NTILE; p++)
#pragma unroll
        for (int i = 0; i < 2; i++) {
            float worth = 0.0f;
            if (2 * L.c + i < X.tile_cols) worth = lds32f(blob + 272 * X.nc + 4 * (p * X.tile_stride + 2 * L.c + i));
            acc[i] += worth * (da * (float)is[p][i]);
            acc[2 + i] += worth * (db * (float)is[p][2 + i]);
        }
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
__device__ __forceinline__ float silu_mul(float g, float u) {
    // gpu/cpu.rs:238-242, 425-427: g * (1 / (1 + exp(-g))) * u
    return g * (1.0f / (1.0f + expf(-g))) * u;
}

__device__ __forceinline__ void emit(const GemvArgs &a, size_t t, size_t r, float v) {
    if (r >= a.w.rows) return;
    if (a.out.scatter_per) {
        // a K-sharded product's partial sum: to the row's owner alone, into its slot for this rank
        const size_t owner = r / a.out.scatter_per, local = r - owner * a.out.scatter_per;
        float *d = a.out.dst[0];
#pragma unroll
        for (int p = 1; p < DWIM_MAX_WORLD; p++)
            if ((size_t)p == owner) d = a.out.dst[p];
        d[(a.t0 + t) * a.out.pitch + a.out.row0 + local] = v;
        return;
    }
    const size_t i = (a.t0 + t) * a.out.pitch + a.out.row0 + r;
    if (a.epi == EPI_ADD) v += a.out.dst[0][i];
    else if (a.epi == EPI_SWIGLU) v = silu_mul(v, a.aux[(a.t0 + t) * a.w.rows + r]);
    a.out.dst[0][i] = v;
    // a shared result: the same element of every peer's copy (plain stores over NVLink).  The
    // parameter array is indexed by constants only: a variable index would make the compiler keep
    // a copy of the kernel's parameters in local memory.
    if (a.out.world > 1) {
#pragma unroll
        for (int p = 1; p < DWIM_MAX_WORLD; p++)
            if (p < a.out.world) a.out.dst[p][i] = v;
    }
}

template <int FMT, int NT, int RT, int KS>
__global__ void __launch_bounds__((RT * KS + 1) * 32, 1) dwim_smallm_kernel(const __grid_constant__ GemvArgs a) {
    constexpr int NW = RT * KS;
    constexpr int R = RT * 16;
    constexpr int UNIT_Q = Traits<FMT>::UNIT_Q;
    constexpr int BASE = base_of(FMT);
    constexpr bool HAS_SCALES = BASE == Q6_K || BASE == Q8_0;   // scales kept apart from the quants
    // a lane's four accumulators (two rows by two columns); the unit routines sum a token's planes as they go
    constexpr int RED_FLOATS = KS > 1 ? 2 * KS * RT * 4 * 32 : 0;

    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);   // full[MAX_STAGES], empty[MAX_STAGES], panels
    float *red = reinterpret_cast<float *>(smem + 256);
    uint8_t *xres = smem + 256 + ((RED_FLOATS * 4 + 127) & ~127);
    uint8_t *stages = xres + a.xres_bytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = a.stages;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + MAX_STAGES), xbar = smem_u32(bars + 2 * MAX_STAGES);
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, NW);
        }
        mbar_init(xbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // The next launch in the stream may start as soon as SMs free up: what it
    // does before its own griddep_wait() (streaming its weights) depends on
    // nothing this kernel writes.
    griddep_launch();

    const int n_chunks = (a.units + a.kc - 1) / a.kc;
    const uint32_t stage0 = smem_u32(stages);

    if (warp == NW) {
        // ------------------------------ producer ------------------------------
        // Weights are written by uploads only, which are ordinary launches long
        // complete: their copies may start before the kernel ahead has finished.
        // The panels come from the prologue that may be that very kernel.
        // So: the first ring-full of weight stages is requested at once, then the
        // warp waits for the kernel ahead and requests the panels.
        uint32_t it = 0;
        const int my_tiles = (int)blockIdx.x < a.n_tiles ? (a.n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        const int n_mats = a.up_quants ? 2 : 1;
        const uint32_t ahead = (uint32_t)min(S, my_tiles * n_mats * n_chunks);   // stages that need no free slot
        bool waited = false;
        for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x)
        for (int mat = 0; mat < n_mats; mat++) {
            const uint8_t *wq = mat ? a.up_quants : a.w.quants;
            const __half *wsc = mat ? a.up_scales : a.w.scales;
            const size_t row0 = (size_t)tile * R;
            const int nrows = (int)min((size_t)R, a.w.rows - row0);
            for (int ch = 0; ch < n_chunks; ch++, it++) {
                const int s = it % S;
                const uint32_t ph = (it / S) & 1;
                mbar_wait(empty0 + 8 * s, ph ^ 1, a.status, 0x1u);
                const int u0 = ch * a.kc, kcc = min(a.kc, a.units - u0);
                const uint32_t qbytes = UNIT_Q * kcc;
                uint32_t sbytes = 0;
                size_t s_first = 0;   // first f16 of the row's scales to copy
                if (BASE == Q8_0) { sbytes = 16 * kcc; s_first = (size_t)8 * u0; }
                if (BASE == Q6_K) {
                    s_first = (size_t)(u0 & ~7);
                    size_t s_end = min((size_t)pad8(u0 + kcc), a.w.srow);
                    sbytes = (uint32_t)(s_end - s_first) * 2;
                }
                const uint32_t xbytes = a.x_resident ? 0u : (uint32_t)a.xunit;
                const uint32_t bar = full0 + 8 * s;
                if (a.whole_rows) {
                    if (lane == 0)
                        mbar_expect_tx(bar, nrows * (uint32_t)(a.w.qpitch + (HAS_SCALES ? a.w.srow * 2 : 0)) + kcc * xbytes);
                } else if (lane == 0) {
                    mbar_expect_tx(bar, nrows * (qbytes + sbytes) + kcc * xbytes);
                }
                __syncwarp();
                const uint32_t st = stage0 + s * a.stage_bytes;
                if (a.whole_rows) {
                    // consecutive rows are one contiguous run (rows sit qpitch apart, and so do the stage's)
                    if (lane == 0) bulk_g2s(st, wq + row0 * a.w.qpitch, nrows * (uint32_t)a.w.qpitch, bar);
                    if (HAS_SCALES && lane == 1)
                        bulk_g2s(st + a.s_off, wsc + row0 * a.w.srow, nrows * (uint32_t)a.w.srow * 2, bar);
                } else {
                    for (int r = lane; r < nrows; r += 32) {
                        bulk_g2s(st + r * a.q_stride, wq + (row0 + r) * a.w.qpitch + (size_t)u0 * UNIT_Q, qbytes, bar);
                        if (HAS_SCALES)
                            bulk_g2s(st + a.s_off + r * a.s_stride, wsc + (row0 + r) * a.w.srow + s_first, sbytes, bar);
                    }
                }
                if (!waited && (!a.x_resident || it + 1 == ahead)) {
                    griddep_wait();
                    waited = true;
                    if (a.x_resident && lane == 0) {
                        // the launch's panels are one contiguous run
                        mbar_expect_tx(xbar, a.xres_bytes);
                        bulk_g2s(smem_u32(xres), a.panels, a.xres_bytes, xbar);
                    }
                }
                for (int u = lane; u < kcc && !a.x_resident; u += 32)
                    bulk_g2s(st + a.x_off + u * xbytes, a.panels + (size_t)(u0 + u) * a.xsrc_stride, xbytes, bar);
            }
        }
        // Drain: the copies this warp issued must have landed before the CTA's
        // shared memory is given up.  Normally the consumers have already
        // waited on every stage and this returns at once.
        if (*(volatile uint32_t *)a.status != 0) {
            uint64_t start = globaltimer();
            uint32_t first = it > (uint32_t)S ? it - S : 0;
            for (uint32_t i = first; i < it; i++) {
                while (!mbar_try(full0 + 8 * (i % S), (i / S) & 1))
                    if (globaltimer() - start > WAIT_LIMIT_NS) break;
            }
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    const int rt = warp % RT, ks = warp / RT;
    Lane L;
    L.g = lane >> 2;
    L.c = lane & 3;
    // The int8 routine reads 8 bytes per lane and row: with rows an odd number
    // of 16-byte steps apart, the four rows of a half-warp must be two steps
    // apart to cover all banks, so lanes g = 0..3 take rows 0, 2, 4, 6 of the
    // eight and g = 4..7 rows 1, 3, 5, 7.
    const int grow = (FMT == Q4K_I8 || FMT == Q8_I8) ? ((L.g & 3) * 2 + (L.g >> 2)) : L.g;
    // the digit planes' columns: one tile of 4n columns (one and two tokens), or a tile of n columns per plane
    const I8Cols X = {a.ncols, NT == 1 ? 0 : a.n_tokens, NT == 1 ? a.ncols : a.n_tokens};

    uint32_t it = 0;
    int tile_parity = 0;
    bool out_ready = false;
    if (a.x_resident && (int)blockIdx.x < a.n_tiles) mbar_wait(xbar, 0, a.status, 0x4u);
    const int n_mats = a.up_quants ? 2 : 1;
    float gate[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // SwiGLU in one launch: the gate's sums of this lane, kept until up's arrive
    for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x)
    for (int mat = 0; mat < n_mats; mat++, tile_parity ^= 1) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};

        for (int ch = 0; ch < n_chunks; ch++, it++) {
            const int s = it % S;
            const uint32_t ph = (it / S) & 1;
            mbar_wait(full0 + 8 * s, ph, a.status, 0x2u);
            const int u0 = ch * a.kc, kcc = min(a.kc, a.units - u0);
            const uint32_t st = stage0 + s * a.stage_bytes;
            L.row_a = st + (rt * 16 + grow) * a.q_stride;
            L.row_b = L.row_a + 8 * a.q_stride;
            L.srow_a = st + a.s_off + (rt * 16 + grow) * a.s_stride;
            L.srow_b = L.srow_a + 8 * a.s_stride;
            L.xbase = a.x_resident ? smem_u32(xres) : st + a.x_off;
            const int xu0 = a.x_resident ? u0 : 0;
            // units are dealt to the K-split warps round-robin over the whole row,
            // so every warp gets the same number whatever the chunking
            for (int ul = (ks + KS - u0 % KS) % KS; ul < kcc; ul += KS) {
                if constexpr (FMT == Q4K_I8) unit_q4k_i8<NT>(L, X, ul, xu0 + ul, acc);
                else if constexpr (FMT == Q8_I8) unit_q8_i8<NT>(L, X, ul, xu0 + ul, acc);
                else unit_q6k_i8<NT>(L, X, ul, xu0 + ul, (a.whole_rows ? u0 : (u0 & 7)) + ul, acc);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);
        }

        // ---- sum the K-split warps of this row tile, in warp order ----
        if (KS > 1) {
            float *buf = red + tile_parity * (KS * RT * 128);
#pragma unroll
            for (int i = 0; i < 4; i++) buf[((ks * RT + rt) * 4 + i) * 32 + lane] = acc[i];
            asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
            if (ks != 0) continue;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float v = 0.0f;
#pragma unroll
                for (int k2 = 0; k2 < KS; k2++) v += buf[((k2 * RT + rt) * 4 + i) * 32 + lane];
                acc[i] = v;
            }
        }

        if (!out_ready) {   // the kernel ahead may still be writing `out` or `aux`
            griddep_wait();
            out_ready = true;
        }
        // ---- epilogue: lane (g, c) holds rows g, g+8 and columns 2c, 2c+1 of each group ----
        const size_t r0 = (size_t)tile * R + rt * 16 + grow, r1 = r0 + 8;
        if constexpr (NT == 1) {
            // a token's four planes are columns 4t..4t+3: lanes c = 2t, 2t+1
            float va = acc[0] + acc[1], vb = acc[2] + acc[3];
            va += __shfl_xor_sync(0xffffffffu, va, 1);
            vb += __shfl_xor_sync(0xffffffffu, vb, 1);
            const int t = L.c >> 1;
            if (n_mats == 2 && mat == 0) {
                gate[0] = va;
                gate[2] = vb;
            } else if (!(L.c & 1) && t < a.n_tokens) {
                emit(a, t, r0, n_mats == 2 ? silu_mul(gate[0], va) : va);
                emit(a, t, r1, n_mats == 2 ? silu_mul(gate[2], vb) : vb);
            }
        } else {
            // a tile per plane, summed by the unit routine: this lane holds tokens 2c and 2c+1 of its two rows
            if (n_mats == 2 && mat == 0) {
#pragma unroll
                for (int i = 0; i < 4; i++) gate[i] = acc[i];
            } else {
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const int t = 2 * L.c + i;
                    if (t < a.n_tokens) {
                        emit(a, t, r0, n_mats == 2 ? silu_mul(gate[i], acc[i]) : acc[i]);
                        emit(a, t, r1, n_mats == 2 ? silu_mul(gate[2 + i], acc[2 + i]) : acc[2 + i]);
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
template <int FMT, int NT, int RT, int KS>
static int launch(dwim_b200_ctx *ctx, GemvArgs &a) {
    constexpr int R = RT * 16;
    constexpr int UNIT_Q = Traits<FMT>::UNIT_Q;
    constexpr int BASE = base_of(FMT);
    constexpr int RED_BYTES = KS > 1 ? ((2 * KS * RT * 4 * 32 * 4 + 127) & ~127) : 0;
    constexpr int SMEM_LIMIT = 227 * 1024;
    const int SMEM_MAX = SMEM_LIMIT;   // one CTA per SM
    const int fixed = 256 + RED_BYTES;
    // The digit planes stay resident in shared memory when they are small next to the ring, or
    // when two stages of whole rows still fit beside them (the planes of five tokens of a
    // 5120-wide row are 83 KB).
    const int xall = a.units * a.xunit;
    const int two_whole = 2 * (int)((R * (a.w.qpitch + a.w.srow * 2) + 127) & ~127);
    a.x_resident = xall <= 80 * 1024 || fixed + xall + two_whole <= SMEM_MAX;
    a.xres_bytes = a.x_resident ? xall : 0;
    // K per stage.  Whole rows when two stages of them fit: the tile is then one
    // contiguous run of HBM and moves with a single bulk copy (issuing a bulk
    // copy costs the producer on the order of a hundred cycles, so a stage
    // made of one copy per row starves the consumers).  Longer rows are cut in
    // even chunks, one copy per row and chunk.
    const int budget = SMEM_MAX - fixed - a.xres_bytes;
    const int srow_bytes = (int)a.w.srow * 2;
    auto whole_stage = [&]() {
        return (int)((R * (a.w.qpitch + srow_bytes) + (a.x_resident ? 0 : a.units * a.xunit) + 127) & ~127);
    };
    a.whole_rows = 2 * whole_stage() <= budget;
    if (a.whole_rows) {
        a.kc = a.units;
        a.q_stride = (int)a.w.qpitch;
        a.s_off = R * a.q_stride;
        a.s_stride = srow_bytes;
        a.x_off = a.s_off + R * a.s_stride;
        a.stage_bytes = whole_stage();
        a.stages = budget / a.stage_bytes;
    } else {
        int chunks = 2;
        for (;; chunks++) {
            a.kc = (a.units + chunks - 1) / chunks;
            int qs = UNIT_Q * a.kc;
            if ((qs / 16) % 2 == 0) qs += 16;   // an odd number of 16-byte steps between rows: no bank conflicts
            a.q_stride = qs;
            a.s_off = R * qs;
            a.s_stride = BASE == Q8_0 ? 16 * a.kc + 16 : BASE == Q6_K ? ((2 * (a.kc + 14) + 15) & ~15) + 16 : 0;
            a.x_off = a.s_off + R * a.s_stride;
            a.stage_bytes = (a.x_off + (a.x_resident ? 0 : a.kc * a.xunit) + 127) & ~127;
            a.stages = budget / a.stage_bytes;
            if (a.stages >= 2 || a.kc == 1) break;
        }
    }
    if (a.stages > MAX_STAGES) a.stages = MAX_STAGES;
    if (a.stages < 2) return fail(ctx, DWIM_B200_EINVAL, "small-M kernel: a stage of %d bytes does not fit", a.stage_bytes);
    a.n_tiles = (int)((a.w.rows + R - 1) / R);
    const int smem = fixed + a.xres_bytes + a.stages * a.stage_bytes;
    auto kern = dwim_smallm_kernel<FMT, NT, RT, KS>;
    static bool configured[64] = {false};   // per instantiation, per device
    if (!configured[ctx->device & 63]) {
        DWIM_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
        configured[ctx->device & 63] = true;
    }
    int grid = a.n_tiles < ctx->sm_count ? a.n_tiles : ctx->sm_count;
    const int nwarps = RT * KS + 1;
    const bool dependent = !ctx->weights_written;   // see dwim_b200_ctx::weights_written
    ctx->weights_written = false;
    DWIM_CUDA(ctx, launch_dependent(dependent, kern, dim3((unsigned)grid), dim3((unsigned)(nwarps * 32)), (size_t)smem, ctx->stream, a));
    DWIM_LAUNCHED(ctx);
    return 0;
}

template <int FMT, int NT>
static int launch_shape(dwim_b200_ctx *ctx, GemvArgs &a) {
    // Row tiles per CTA (RT) x K-split warps per row tile (KS).  KS should
    // divide the row's units so that every warp gets the same share.
    // Measured on B200 at the model's shapes: one and two tokens of Q4_K run
    // best with 32-row tiles when there are rows enough for two tiles per SM,
    // the wider formats with 16-row tiles (their stages are larger); eight
    // K-split warps throughout.  Three to eight tokens (NT = 3) keep 16-row
    // tiles: their planes then stay resident beside two stages of whole rows.
    if constexpr (FMT == Q4K_I8 && NT == 1) {
        if ((a.w.rows + 31) / 32 >= (size_t)2 * ctx->sm_count) return launch<FMT, NT, 2, 8>(ctx, a);
    }
    return launch<FMT, NT, 1, 8>(ctx, a);
}

// Whether the small-M kernel takes a product of n tokens: up to eight tokens of
// any format (Q8_0 rows need not be whole 256-weight units: their scale rows are
// padded with zeros).
bool gemv_takes_i8(const WeightView &w, size_t n) {
    if (n < 1 || n > I8_MAX_TOKENS) return false;
    return w.fmt == Q8_0 || ((w.fmt == Q4_K || w.fmt == Q6_K) && w.cols % 256 == 0);
}

// Up to eight tokens through the int8 routines; `panels` from build_panels_i8.
// `up`, when given, makes it the SwiGLU of the pair (w = gate) in one launch.
int gemv_small_i8(dwim_b200_ctx *ctx, const WeightView &w, const uint8_t *panels, int n_tokens, size_t t0, const OutSpec &out,
                  const float *aux, int epilogue, const WeightView *up) {
    if (w.rows == 0 || n_tokens == 0) return 0;
    if (!gemv_takes_i8(w, (size_t)n_tokens))
        return fail(ctx, DWIM_B200_EINVAL, "int8 small-M kernel: format %d, %d tokens", w.fmt, n_tokens);
    GemvArgs a{};
    a.w = w;
    a.panels = panels;
    a.ncols = i8_planes(n_tokens) * n_tokens;
    a.n_tokens = n_tokens;
    a.t0 = t0;
    a.out = out;
    a.aux = aux;
    a.epi = epilogue;
    a.units = (int)((w.cols + 255) / 256);
    a.xunit = a.xsrc_stride = i8_unit_bytes(a.ncols);
    if (up) {
        if (up->fmt != w.fmt || up->rows != w.rows || up->cols != w.cols || up->qpitch != w.qpitch || epilogue != EPI_STORE)
            return fail(ctx, DWIM_B200_EINVAL, "int8 small-M kernel: gate and up differ");
        a.up_quants = up->quants;
        a.up_scales = up->scales;
    }
    a.status = ctx->status;
    const bool packed = n_tokens <= 2;   // one column tile (4 planes x 1-2 tokens), or a tile per plane (3 planes)
    switch (w.fmt) {
    case Q4_K: return packed ? launch_shape<Q4K_I8, 1>(ctx, a) : launch_shape<Q4K_I8, 3>(ctx, a);
    case Q8_0: return packed ? launch_shape<Q8_I8, 1>(ctx, a) : launch_shape<Q8_I8, 3>(ctx, a);
    case Q6_K: return packed ? launch_shape<Q6K_I8, 1>(ctx, a) : launch_shape<Q6K_I8, 3>(ctx, a);
    default: return fail(ctx, DWIM_B200_EFORMAT, "unknown weight format %d", w.fmt);
    }
}

}  // namespace dwim
