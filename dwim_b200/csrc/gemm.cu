// The large-M product (prefill, long verify batches) for Q4_K: a dense
// contraction on the 5th-generation tensor cores whose weight products are
// exact.  Replaces the reference's matmul_tile64_* kernels
// (matmul_tile.cu:94-258; host side gpu/cuda/mod.rs:402-442).
//
// out[t][r] = sum_k W[r][k] x[t][k], with W[r][k] = d*(sc_j*q) - dmin*m_j
// (d, dmin per 256-weight unit and row; sc_j, m_j per 32-weight sub-block).
// The integer sc_j*q <= 945 is exact in f16, so for every unit u of K
//     S_u[r][t] = sum_k (sc*q)[r][k] * x[t][k]                    16 MMAs of K=16
//               - sum_j (32*dmin/d * m_j)[r] * mean_j(x[t])         2 MMAs of K=16
// is accumulated in the tensor cores' fp32 accumulators and
//     out[r][t] = sum_u d_u[r] * S_u[r][t]
// is applied by CUDA cores in fp32.  The first sum's products are exact; the
// second's factors travel as f16 value + rounding remainder on both sides (22
// bits each), and a power of two moves between d and the operands when dmin/d
// is large (q4k_fold below).  The reference's tile kernel rounds every
// dequantized weight to f16 instead (matmul_tile.cu:66-74): 2e-4 of rms error
// against 5e-7 here.  An f32 activation travels as two f16 columns, value and
// rounding remainder, which the epilogue adds up again; a bf16 one is exact in
// one column.
//
// A CTA owns 128 weight rows (one TMEM lane each) by BN columns (32..256):
//   warp 0        activations' producer (one thread): per K block of 64 the f16
//                 tile [BN][64] (TMA, 128-byte swizzle) into the B ring; per
//                 unit the sub-block means' hi and lo parts.
//   warp 1        MMA issuer: tcgen05.mma M=128 N=BN K=16 into the unit's
//                 accumulator buffer (two buffers, so unit u+1 multiplies
//                 while unit u drains).  The whole warp runs the loop and one
//                 lane issues: that thread has about one instruction slot per
//                 five cycles, and an N=128 MMA leaves it 64 cycles.
//   warps 2-17    workers.  Warp w owns TMEM lane quadrant w % 4 (weight rows
//                 32*(w % 4) + lane) and K block (w - 2) / 4 of every unit:
//                 thread = row turns the block's 64 nibbles into sc*q halves
//                 (lop3 magic number + one HFMA2 per two weights) and stores
//                 them into the stage's A tile in the K-major 128-byte-
//                 swizzled layout of the MMA's descriptor; then it drains a
//                 quarter of the previous unit's columns: tcgen05.ld, acc +=
//                 d*S in registers.  K blocks 2 and 3's warps also write the
//                 unit's minimums operand and the row scales.  After the last
//                 unit: the operator's epilogue (store / add / SwiGLU),
//                 coalesced over rows.
//   warp 18       packed weights' producer (one thread): per unit the tile's
//                 blocks [128 rows][144 B] from HBM into the raw ring.
// Every mbarrier wait is bounded (ptx.cuh); a kernel that gave up says so in
// the context's status word.
#include <cuda.h>
#include <stdlib.h>


#include "common.cuh"
#include "ptx.cuh"

namespace dwim {

namespace {

constexpr int TILE_M = 128;   // weight rows per CTA
constexpr int BK = 64;        // K per stage: one 128-byte swizzled row of f16
constexpr int KBLOCKS = 4;    // K blocks per unit = stages of the A ring: A stage index == K block within the unit
constexpr int SCALE_SLOTS = 4;
constexpr int N_WORKERS = 16;                                      // warps 2..17: four per TMEM lane quadrant
constexpr int RAW_WARP = 2 + N_WORKERS;                            // the packed weights' producer
constexpr int GEMM_THREADS = (3 + N_WORKERS) * 32;
constexpr int RAW_BYTES = ((TILE_M * 144 + 1023) / 1024) * 1024;   // 18 KB
constexpr int A_BYTES = TILE_M * BK * 2;                           // 16 KB
constexpr int AMIN_BYTES = TILE_M * 16 * 4;                        // 8 KB: [K group of 8][row][16 B], four groups
constexpr int MAX_SMEM = 227 * 1024;
constexpr int BAR_BYTES = 1024;

struct GemmArgs {
    size_t rows, n, ncols, units;   // weight rows, tokens, operand columns, 256-weight units of K
    int split;                      // 1: columns 2t, 2t+1 are token t's hi and lo halves
    OutSpec out;
    const float *tok_scale;         // per token: the power of two its activations were divided by (prologue.cu)
    const float *aux;               // EPI_SWIGLU: the `up` product, token-major [n][rows]
    int epi;
    uint32_t *status;
};

// Per tile width.  Up to 128 columns everything is double-buffered by units:
// the B ring has one stage per K block like the A ring, and K blocks change
// hands in pairs (one barrier round trip per 128 of K, which the MMA warp's
// 64-cycle issue budget needs).  At 256 columns a decoded weight is used twice
// as often, an MMA takes 128 cycles, and shared memory is the limit: three B
// stages, two raw stages, one stage of the minimums' operands, and a hand-over
// per K block (a B stage is reloaded as soon as its own K block is done).
template <int BN> struct Cfg {
    static constexpr int B_STAGES = BN > 128 ? 3 : 4;
    static constexpr int RAW_STAGES = BN > 128 ? 2 : 3;
    static constexpr int MIN_STAGES = BN > 128 ? 1 : 2;
    static constexpr int HAND = BN > 128 ? 1 : 2;                  // K blocks per hand-over
    static constexpr int NHAND = KBLOCKS / HAND;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int BMIN_BYTES = BN * 16 * 2;                 // [K group of 8][column][16 B]: the means' hi and lo parts
    static constexpr int MIN_BYTES = AMIN_BYTES + ((BMIN_BYTES + 1023) / 1024) * 1024;
    static constexpr int SCALE_BYTES = SCALE_SLOTS * TILE_M * 4;   // the unit's scale per row
    static constexpr int TOK_BYTES = BN * 4;                       // the columns' token scales, for the epilogue
    static constexpr int SMEM = BAR_BYTES + KBLOCKS * A_BYTES + B_STAGES * B_BYTES + MIN_STAGES * MIN_BYTES +
                                RAW_STAGES * RAW_BYTES + SCALE_BYTES + TOK_BYTES + 1024;   // + alignment slack
    static_assert(SMEM <= MAX_SMEM, "the tile does not fit shared memory");
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;    // two accumulator buffers
    static constexpr int DRAIN_COLS = BN / 4 < 16 ? 16 : BN / 4;   // accumulator columns per draining warp
    static constexpr int DRAINERS = BN / DRAIN_COLS;               // draining warps per lane quadrant (4, or 2 at BN=32)
};

// ---- tcgen05 wrappers -----------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; f16 inputs, f32 accumulate.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// The same with the descriptors given as (low word, shared high word) and the
// accumulate flag fixed at compile time: the issuing thread has about one
// instruction slot per five cycles, so every instruction between two MMAs counts.
template <int ACC>
__device__ __forceinline__ void umma_f16_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, {%6, %6, %6, %6}, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "n"(ACC), "r"(0u)
        : "memory");
}
// Arrive on an mbarrier once every MMA this thread issued so far has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// d = a * b + d on two packed floats.
__device__ __forceinline__ void ffma2(uint64_t &d, uint64_t a, uint64_t b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
    uint32_t a, b;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
    lo = __uint_as_float(a);
    hi = __uint_as_float(b);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors (K-major operands).
//   [0,14) address >> 4   [16,30) leading byte offset >> 4   [32,46) stride
//   byte offset >> 4   [46,48) version 1   [61,64) layout
// 128-byte swizzle: rows are 128 bytes (64 f16), eight-row groups 1024 bytes
// apart (stride offset); the leading offset is not used: (addr & 0x3ffff) >> 4 | 1 << 16 |
// 64 << 32 | 1 << 46 | 2 << 61.  The kernels keep it as a low word per stage and the high word
// all stages share (`desc_hi`), so that the MMA warp adds to 32-bit values only.
// No swizzle: 8 rows x 16 bytes are contiguous (128 bytes); eight-row groups
// 128 bytes apart (stride offset); the second 8 of K `lbo` bytes further on.
__device__ __forceinline__ uint64_t smem_desc_plain(uint32_t addr, uint32_t lbo) {
    return (uint64_t)((addr & 0x3ffffu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | (8ull << 32) | (1ull << 46);
}
// Instruction descriptor: f32 accumulate (bits 4-5 = 1), f16 A and B (0),
// both K-major (0), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void sts64(uint32_t a, uint32_t x, uint32_t y) {
    asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(a), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void sts32f(uint32_t a, float x) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(x) : "memory"); }
__device__ __forceinline__ float lds32f(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
// Two floats rounded to f16, `lo` in the low half.
__device__ __forceinline__ uint32_t f16x2_rn(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float silu_mul_f(float g, float u) { return g * (1.0f / (1.0f + expf(-g))) * u; }

// Where a thread's results go: its row of one destination; or (SHARED kernels) of every rank's
// copy of a shared result; or (a K-sharded product's partial sums) of its owner's slot alone.
// The pointers are read from the kernel's parameters by constant index, once, ahead of the
// stores' loop: indexing the parameter array by a variable, or reading a parameter after every
// store, cost the 256-column kernel half its speed.  The many-destination stores live in kernel
// instantiations of their own, so that the usual kernel's code stays small (an epilogue with
// eight predicated stores per value stalled the main loop on instruction fetch).
struct EmitTo {
    float *own;              // the first (or only) destination's element (token 0, this thread's row)
    size_t offset;           // the same element's offset in every other destination
    size_t pitch;
    const float *aux_row;
    const OutSpec *out;
    int world, epi;
};
__device__ __forceinline__ EmitTo emit_to(const OutSpec &out, const float *aux, int epi, size_t row) {
    EmitTo e;
    float *d = out.dst[0];
    e.offset = out.row0 + row;
    if (out.scatter_per) {
        // the row's owner alone, its slot for this rank; the owner is picked by constant indices
        const size_t owner = row / out.scatter_per;
        e.offset = out.row0 + row - owner * out.scatter_per;
#pragma unroll
        for (int p = 1; p < DWIM_MAX_WORLD; p++)
            if ((size_t)p == owner) d = out.dst[p];
    }
    e.own = d + e.offset;
    e.pitch = out.pitch;
    e.aux_row = aux ? aux + row : nullptr;
    e.out = &out;
    e.world = out.scatter_per ? 1 : out.world;
    e.epi = epi;
    return e;
}
// One finished element: the operator's epilogue, then the store.
template <bool SHARED>
__device__ __forceinline__ void gemm_emit(const EmitTo &e, size_t rows, size_t t, float x) {
    float *o = e.own + t * e.pitch;
    if (!SHARED) {
        if (e.epi == EPI_ADD) x += *o;
        else if (e.epi == EPI_SWIGLU) x = silu_mul_f(x, e.aux_row[t * rows]);
    }
    *o = x;
    if (SHARED) {
#pragma unroll
        for (int p = 1; p < DWIM_MAX_WORLD; p++)
            if (p < e.world) e.out->dst[p][e.offset + t * e.pitch] = x;
    }
}

constexpr uint32_t H2_1024 = 0x64006400u, H2_M1024 = 0xE400E400u, H2_64 = 0x54005400u, H2_M64 = 0xD400D400u;

// ---- dequantizer: the 64 weights of one row and K block as exact sc*q halves ----------
// K block g (0..3 inside the unit) is group g of the block's quants: 32 bytes
// whose low nibbles are sub-block 2g (k = 0..31 of the K block) and high
// nibbles sub-block 2g+1 (k = 32..63).  A word's bytes come out in the order
// (0, 2, 1, 3); the activations are stored in the same order.
// A row's unit is drained as s * S, with S the one accumulator both operands
// add into, and s = d * 2^e.  The main operand is sc*q*2^-e (still exact in
// f16, subnormals included, for e <= 24) and the minimums enter as
// -(32*dmin/s)*m_j.  e = 0 unless dmin is more than ~32 times d: it is chosen
// from the two exponents so that 63 * 32*dmin/s stays below f16's maximum.
// When d is zero, or e would pass 24 (the sc*q term is then below 2^-19 of the
// other), s = 32*dmin, the main operand is zero and the minimums enter as -m_j.
struct Q4kFold {
    int e;        // the main operand is scaled by 2^-e
    bool zero;    // the main operand is dropped
};
__device__ __forceinline__ Q4kFold q4k_fold(uint32_t d_dmin) {
    const float d = h2f_lo(d_dmin), dmin = h2f_hi(d_dmin);
    const int ed = (int)((__float_as_uint(d) >> 23) & 0xffu), em = (int)((__float_as_uint(dmin) >> 23) & 0xffu);
    Q4kFold f;
    f.e = max(0, em - ed - 4);
    f.zero = d == 0.0f || f.e > 24;
    if (f.zero) f.e = 0;
    return f;
}

struct Q4kBlock {
    uint32_t words[8];                 // the 32 bytes of group g
    uint32_t mul[2], add[2];           // per nibble half: x*mul + add turns the magic-number halves into sc*q
};
__device__ __forceinline__ void load_q4k_block(const uint4 &hdr, uint32_t raw_row, int g, Q4kBlock &b) {
    const uint4 q0 = lds128(raw_row + 16 + 32 * g), q1 = lds128(raw_row + 32 + 32 * g);
    b.words[0] = q0.x; b.words[1] = q0.y; b.words[2] = q0.z; b.words[3] = q0.w;
    b.words[4] = q1.x; b.words[5] = q1.y; b.words[6] = q1.z; b.words[7] = q1.w;
    const int sh = (g & 1) * 16;
    const uint32_t y = (hdr.y >> sh) & 0xffffu, w = (hdr.w >> sh) & 0xffffu;
    const uint32_t sc2 = g < 2 ? (y & 0x3f3fu) : ((w & 0x0f0fu) | ((y >> 2) & 0x3030u));
    const uint32_t sa = sc2 & 0xffu, sb = sc2 >> 8;
    const Q4kFold f = q4k_fold(hdr.x);
    // 2^-e as a half: normal down to 2^-14, subnormal below; zero drops the operand
    const uint32_t p1 = f.zero ? 0u : (f.e <= 14 ? (uint32_t)(15 - f.e) << 10 : 1u << (24 - f.e));
    const uint32_t p2 = p1 | (p1 << 16);
    const uint32_t spa = hmul2(hsub2(0x64006400u | sa | (sa << 16), H2_1024), p2);   // half2 of sc_2g * 2^-e
    const uint32_t spb = hmul2(hsub2(0x64006400u | sb | (sb << 16), H2_1024), p2);   // half2 of sc_2g+1 * 2^-e
    // low nibbles: (1024 + q)*sc - 1024*sc; high nibbles: (64 + q)*sc - 64*sc
    b.mul[0] = spa; b.add[0] = hmul2(spa, H2_M1024);
    b.mul[1] = spb; b.add[1] = hmul2(spb, H2_M64);
}
// Writes the row's 128 bytes of the stage's A tile (K-major, 128-byte swizzle:
// 16-byte chunk c of row r sits at chunk c ^ (r & 7)).  `a_row_sw` is the row's
// address with (r & 7) << 4 or-ed in (rows are 128-byte aligned), so chunk c
// is at a_row_sw ^ (c << 4).
__device__ __forceinline__ void store_q4k_block(const Q4kBlock &b, uint32_t a_row_sw) {
#pragma unroll
    for (int c = 0; c < 4; c++) {   // words 2c, 2c+1: weights 8c .. 8c+7 of either sub-block
        const uint32_t w0 = b.words[2 * c], w1 = b.words[2 * c + 1], s0 = w0 >> 8, s1 = w1 >> 8;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            // 0x6400 | q = 1024 + q; 0x5400 | q << 4 = 64 + q (the ulp of 64.0 is 1/16)
            const uint32_t mask = h ? 0x00f000f0u : 0x000f000fu, magic = h ? H2_64 : H2_1024;
            const uint32_t o0 = hfma2(lop3_and_or(w0, mask, magic), b.mul[h], b.add[h]);   // bytes 0, 2
            const uint32_t o1 = hfma2(lop3_and_or(s0, mask, magic), b.mul[h], b.add[h]);   // bytes 1, 3
            const uint32_t o2 = hfma2(lop3_and_or(w1, mask, magic), b.mul[h], b.add[h]);
            const uint32_t o3 = hfma2(lop3_and_or(s1, mask, magic), b.mul[h], b.add[h]);
            sts128(a_row_sw ^ ((4 * h + c) << 4), o0, o1, o2, o3);
        }
    }
}

// Four of the row's eight 6-bit minimums (m_0..m_3 for part 0, m_4..m_7 for
// part 1), each times f, as two f16 terms (value and rounding remainder):
// b[t] holds term t of the four values, two per word.
__device__ __forceinline__ void mins_q4k_terms(const uint4 &hdr, int part, float f, uint32_t (&b)[2][2]) {
    const uint32_t m4 = part ? (((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u)) : (hdr.z & 0x3f3f3f3fu);
#pragma unroll
    for (int i = 0; i < 2; i++) {
        // byte -> float through the 2^23 magic number
        const float p0 = (__uint_as_float(prmt(m4, 0x4B000000u, 0x7650 + 2 * i)) - 8388608.0f) * f;
        const float p1 = (__uint_as_float(prmt(m4, 0x4B000000u, 0x7651 + 2 * i)) - 8388608.0f) * f;
        const uint32_t hi = f16x2_rn(p0, p1);
        b[0][i] = hi;
        b[1][i] = f16x2_rn(p0 - h2f_lo(hi), p1 - h2f_hi(hi));
    }
}

// One map per destination of a shared result, for the form of the kernel that writes it with TMA:
// this rank's rows of destination p as [tokens][rows], box [a draining warp group's tokens][128 rows].
struct OutMaps {
    CUtensorMap m[DWIM_MAX_WORLD];
};

// OUT: 0 = one destination (or a scattered one); 1 = a result shared by several ranks, every value
// stored to each copy from registers; 2 = the same through shared memory and one TMA store per
// destination and group of columns (whole 512-byte runs over NVLink instead of 4-byte stores).
template <int BN, int OUT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_q4k_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                const __grid_constant__ CUtensorMap tmap_m, const __grid_constant__ GemmArgs a,
                const __grid_constant__ OutMaps maps) {
    constexpr bool SHARED = OUT == 1;
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // the swizzled tiles want 1024-byte alignment
    // barriers, 8 bytes each
    const uint32_t full0 = base, empty0 = base + 32, minfull0 = base + 64;
    const uint32_t rawfull0 = base + 96, rawempty0 = base + 128, accfull0 = base + 160, accempty0 = base + 176;
    const uint32_t tmem_slot = base + 192;
    const uint32_t astage0 = base + BAR_BYTES;
    const uint32_t bstage0 = astage0 + KBLOCKS * A_BYTES;
    const uint32_t min0 = bstage0 + C::B_STAGES * C::B_BYTES;
    const uint32_t raw0 = min0 + C::MIN_STAGES * C::MIN_BYTES;
    const uint32_t scale0 = raw0 + C::RAW_STAGES * RAW_BYTES;
    const uint32_t tok0 = scale0 + C::SCALE_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * TILE_M, col0 = blockIdx.y * BN;
    const int units = (int)a.units;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::NHAND; s++) {
            mbar_init(full0 + 8 * s, 1 + 4 * C::HAND);   // the producer's expect_tx arrival + the hand-over's worker warps
            mbar_init(empty0 + 8 * s, 1);                // the MMA warp's commit
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(minfull0 + 8 * s, 1 + 8);          // the producer + the eight warps that write the minimums
            mbar_init(accfull0 + 8 * s, 1);              // also says that the unit's minimums and means have been read
            mbar_init(accempty0 + 8 * s, 4 * C::DRAINERS);
        }
        for (int s = 0; s < C::RAW_STAGES; s++) {
            mbar_init(rawfull0 + 8 * s, 1);
            mbar_init(rawempty0 + 8 * s, N_WORKERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = lds32(tmem_slot);
    // Launched as a programmatic dependent: the next launch on the stream may begin as SMs
    // free up; here only the packed weights (written by uploads alone) are touched before
    // griddep_wait(): the activations' producer waits before its first load, the workers
    // before their first store.
    griddep_launch();

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        griddep_wait();   // the operand comes from the prologue kernel just ahead
        if (lane == 0) {
            for (int u = 0; u < units; u++) {
                const int ms = u % C::MIN_STAGES;
                for (int h = 0; h < C::NHAND; h++) {
                    // B stage kb % B_STAGES was last read by K block kb - B_STAGES
                    for (int g = h * C::HAND; g < (h + 1) * C::HAND; g++) {
                        const int prev = KBLOCKS * u + g - C::B_STAGES;
                        if (prev >= 0)
                            mbar_wait_parked(empty0 + 8 * ((prev % KBLOCKS) / C::HAND), (prev / KBLOCKS) & 1, a.status, 0x20u);
                    }
                    mbar_expect_tx(full0 + 8 * h, C::HAND * C::B_BYTES);
                    for (int g = h * C::HAND; g < (h + 1) * C::HAND; g++) {
                        const int kb = KBLOCKS * u + g;
                        tma_load_2d(bstage0 + (kb % C::B_STAGES) * C::B_BYTES, &tmap_x, kb * BK, col0, full0 + 8 * h);
                    }
                }
                // the minimums' stage was last read by unit u - MIN_STAGES
                if (u >= C::MIN_STAGES) {
                    const int uu = u - C::MIN_STAGES;
                    mbar_wait_parked(accfull0 + 8 * (uu & 1), (uu >> 1) & 1, a.status, 0x40u);
                }
                mbar_expect_tx(minfull0 + 8 * ms, C::BMIN_BYTES);
                const uint32_t bm = min0 + ms * C::MIN_BYTES + AMIN_BYTES;
                tma_load_2d(bm, &tmap_m, u * 16, col0, minfull0 + 8 * ms);                 // the means' hi parts
                tma_load_2d(bm + BN * 16, &tmap_m, u * 16 + 8, col0, minfull0 + 8 * ms);   // and lo parts
            }
        }
    } else if (warp == RAW_WARP) {
        // ------------------------------ packed weights' producer ------------------------------
        // Its own warp: the blocks come from HBM and must run as far ahead as the
        // ring allows, whatever the activations' producer is waiting for.
        if (lane == 0) {
            for (int u = 0; u < units; u++) {
                const int rs = u % C::RAW_STAGES;
                mbar_wait_parked(rawempty0 + 8 * rs, ((u / C::RAW_STAGES) & 1) ^ 1, a.status, 0x10u);
                mbar_expect_tx(rawfull0 + 8 * rs, TILE_M * 144);
                tma_load_2d(raw0 + rs * RAW_BYTES, &tmap_w, u * 144, row0, rawfull0 + 8 * rs);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        // The whole warp runs the loop (uniform control flow keeps addresses
        // and descriptors on the uniform data path) and one lane issues.  Units
        // are taken two at a time so that the accumulator buffer is static.
        constexpr uint32_t idesc = idesc_f16(TILE_M, BN);
        constexpr uint32_t desc_hi = 64u | (1u << 14) | (2u << 29);   // stride offset 1024 B, version 1, 128-byte swizzle
        const uint32_t a_lo = ((astage0 & 0x3ffffu) >> 4) | (1u << 16), b_lo = ((bstage0 & 0x3ffffu) >> 4) | (1u << 16);
        const uint32_t tm = __shfl_sync(0xffffffffu, tmem_base, 0);
        int bs = 0;                                                   // the B stage of the next K block
        for (int u0 = 0; u0 < units; u0 += 2) {
#pragma unroll
            for (int ab = 0; ab < 2; ab++) {
                const int u = u0 + ab;
                if (u >= units) break;
                const uint32_t s1 = tm + ab * BN;
                const uint32_t upar = (u0 >> 1) & 1;
                mbar_wait_parked(accempty0 + 8 * ab, upar ^ 1, a.status, 0x80u);   // the drain of unit u-2 is done
#pragma unroll
                for (int h = 0; h < C::NHAND; h++) {
                    mbar_wait_parked(full0 + 8 * h, ab, a.status, 0x100u);
                    tc_fence_after();
#pragma unroll
                    for (int gg = 0; gg < C::HAND; gg++) {
                        const int g = h * C::HAND + gg;
                        const uint32_t ad = a_lo + g * (A_BYTES >> 4);
                        const uint32_t bd = b_lo + (C::B_STAGES == KBLOCKS ? g : bs) * (C::B_BYTES >> 4);
                        if (lane == 0) {
#pragma unroll
                            for (int k = 0; k < BK / 16; k++) {   // 32 bytes further along the swizzled row per K=16
                                if (g == 0 && k == 0) umma_f16_lo<0>(s1, ad, bd, desc_hi, idesc);
                                else umma_f16_lo<1>(s1, ad + 2 * k, bd + 2 * k, desc_hi, idesc);
                            }
                        }
                        bs = bs + 1 == C::B_STAGES ? 0 : bs + 1;
                    }
                    if (lane == 0) umma_commit(empty0 + 8 * h);   // the stages may be refilled once these finish
                    __syncwarp();
                }
                const int ms = u % C::MIN_STAGES;
                mbar_wait_parked(minfull0 + 8 * ms, (u / C::MIN_STAGES) & 1, a.status, 0x200u);
                tc_fence_after();
                if (lane == 0) {
                    // the minimums: terms (hi, hi | lo, lo) against the means' (hi, lo) twice
                    const uint32_t am = min0 + ms * C::MIN_BYTES;
                    const uint64_t bdm = smem_desc_plain(am + AMIN_BYTES, BN * 16);
                    umma_f16(s1, smem_desc_plain(am, TILE_M * 16), bdm, idesc, 1);
                    umma_f16(s1, smem_desc_plain(am + 2 * TILE_M * 16, TILE_M * 16), bdm, idesc, 1);
                    umma_commit(accfull0 + 8 * ab);     // the unit's sum is complete
                }
                __syncwarp();
            }
        }
    } else {
        // ------------------------------ workers (warps 2-17) ------------------------------
        // Warp w owns TMEM lane quadrant w % 4 (weight rows 32*(w % 4) + lane)
        // and K block g = (w - 2) / 4 of every unit: it decodes that block of
        // its rows into the stage's A tile, then drains column quarter g of the
        // previous unit's sums while the tensor cores work on this one.
        const int quad = warp & 3;
        const int g = (warp - 2) >> 2;
        const int rl = quad * 32 + lane;                // row within the tile = TMEM lane
        const bool drains = g < C::DRAINERS;
        const uint32_t drain_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + g * C::DRAIN_COLS;
        const uint32_t a_row_sw = (astage0 + g * A_BYTES + rl * 128) | ((rl & 7) << 4);
        uint64_t acc2[C::DRAIN_COLS / 2];   // the row's sums, two columns per packed pair
#pragma unroll
        for (int j = 0; j < C::DRAIN_COLS / 2; j++) acc2[j] = 0ull;

        auto drain = [&](int u) {
            const int ab = u & 1;
            // the unit's sum is complete; its last MMAs waited for the minimums'
            // stage, which the row scales were written before
            mbar_wait_parked(accfull0 + 8 * ab, (u >> 1) & 1, a.status, 0x4000u);
            tc_fence_after();
            const uint32_t sc = __float_as_uint(lds32f(scale0 + ((u % SCALE_SLOTS) * TILE_M + rl) * 4));
            const uint64_t sc2 = pack2(sc, sc);
#pragma unroll
            for (int c = 0; c < C::DRAIN_COLS / 16; c++) {
                uint32_t v[16];
                tmem_ld16(drain_addr + ab * BN + c * 16, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; j++) ffma2(acc2[c * 8 + j], sc2, pack2(v[2 * j], v[2 * j + 1]));
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(accempty0 + 8 * ab);
        };

        for (int u = 0; u < units; u++) {
            const int rs = u % C::RAW_STAGES, ms = u % C::MIN_STAGES;
            mbar_wait_parked(rawfull0 + 8 * rs, (u / C::RAW_STAGES) & 1, a.status, 0x400u);
            const uint32_t raw_row = raw0 + rs * RAW_BYTES + rl * 144;
            const uint4 hdr = lds128(raw_row);
            Q4kBlock blk;
            load_q4k_block(hdr, raw_row, g, blk);
            mbar_wait_parked(empty0 + 8 * (g / C::HAND), (u & 1) ^ 1, a.status, 0x800u);   // the MMAs that read this stage are done
            store_q4k_block(blk, a_row_sw);
            fence_async_smem();          // the tensor core reads shared memory through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(full0 + 8 * (g / C::HAND));
            if (g >= 2) {
                // the minimums' A operand [K group][row][16 B]: groups (hi, hi, lo, lo) of the
                // two f16 terms of -(32*dmin/s)*m_j; K block 2's warp writes m_0..m_3, K block 3's m_4..m_7
                if (u >= C::MIN_STAGES) {   // the unit that used this stage last has read its minimums
                    const int uu = u - C::MIN_STAGES;
                    mbar_wait_parked(accfull0 + 8 * (uu & 1), (uu >> 1) & 1, a.status, 0x1000u);
                }
                const Q4kFold f = q4k_fold(hdr.x);
                const float dmin32 = 32.0f * h2f_hi(hdr.x);
                const float sc = f.zero ? dmin32 : h2f_lo(hdr.x) * __uint_as_float((uint32_t)(127 + f.e) << 23);
                uint32_t b[2][2];
                mins_q4k_terms(hdr, g - 2, f.zero ? -1.0f : -(dmin32 / sc), b);
                const uint32_t am = min0 + ms * C::MIN_BYTES + rl * 16 + (g - 2) * 8;
                sts64(am, b[0][0], b[0][1]);
                sts64(am + TILE_M * 16, b[0][0], b[0][1]);
                sts64(am + 2 * TILE_M * 16, b[1][0], b[1][1]);
                sts64(am + 3 * TILE_M * 16, b[1][0], b[1][1]);
                if (g == 2) sts32f(scale0 + ((u % SCALE_SLOTS) * TILE_M + rl) * 4, sc);
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(minfull0 + 8 * ms);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(rawempty0 + 8 * rs);
            if (drains && u > 0) drain(u - 1);
        }
        if (drains) {
            griddep_wait();   // the kernel ahead may still read or write `out` and `aux`
            // this warp's columns' token scales through shared memory (the four quadrants' warps of a
            // column group write the same values): a load from global memory ahead of every store
            // would wait for the store before it
            for (int j = lane; j < C::DRAIN_COLS; j += 32) {
                const size_t t = ((size_t)col0 + g * C::DRAIN_COLS + j) >> (a.split ? 1 : 0);
                sts32f(tok0 + (g * C::DRAIN_COLS + j) * 4, t < a.n ? a.tok_scale[t] : 1.0f);
            }
            __syncwarp();
            // nothing to multiply by for activations of the usual range: every scale is one
            const uint32_t tk = tok0 + g * C::DRAIN_COLS * 4;
            bool ones = true;
            for (int j = lane; j < C::DRAIN_COLS; j += 32) ones = ones && lds32f(tk + j * 4) == 1.0f;
            const bool scaled = !__all_sync(0xffffffffu, ones);
            drain(units - 1);
            float acc[C::DRAIN_COLS];
#pragma unroll
            for (int j = 0; j < C::DRAIN_COLS / 2; j++) unpack2(acc2[j], acc[2 * j], acc[2 * j + 1]);
            const size_t row = (size_t)row0 + rl;
            if (OUT == 2) {
                // The group's tile [token][row] into the rings' shared memory, which nothing reads any
                // more (the last unit's MMAs are done, its accumulator drained), then one store per
                // destination.  Rows and tokens past the end are cut off by the maps' bounds.
                const uint32_t stage = astage0 + g * (C::DRAIN_COLS * TILE_M * 4);
                if (scaled) {
#pragma unroll
                    for (int j = 0; j < C::DRAIN_COLS; j++) acc[j] *= lds32f(tk + j * 4);
                }
                int nvals = C::DRAIN_COLS;
                if (a.split) {
#pragma unroll
                    for (int j = 0; j < C::DRAIN_COLS / 2; j++) acc[j] = acc[2 * j] + acc[2 * j + 1];
                    nvals = C::DRAIN_COLS / 2;
                }
#pragma unroll
                for (int j = 0; j < C::DRAIN_COLS; j++)
                    if (j < nvals) sts32f(stage + (j * TILE_M + rl) * 4, acc[j]);
                fence_async_smem();
                asm volatile("bar.sync %0, 128;" ::"r"(1 + g) : "memory");   // the group's four warps: all 128 rows are in
                const size_t t0 = ((size_t)col0 + g * C::DRAIN_COLS) >> (a.split ? 1 : 0);
                if (quad == 0 && lane == 0 && t0 < a.n) {
#pragma unroll
                    for (int p = 0; p < DWIM_MAX_WORLD; p++)
                        if (p < a.out.world) tma_store_2d(&maps.m[p], row0, (int)t0, stage);
                    tma_store_commit_wait();
                }
            } else if (row < a.rows) {
                const size_t cbase = (size_t)col0 + g * C::DRAIN_COLS;
                const EmitTo to = emit_to(a.out, a.aux, a.epi, row);
                const size_t n = a.n, rows = a.rows;
                if (scaled) {   // the tokens' powers of two
#pragma unroll
                    for (int j = 0; j < C::DRAIN_COLS; j++) acc[j] *= lds32f(tk + j * 4);
                }
                if (a.split) {
#pragma unroll
                    for (int j = 0; j < C::DRAIN_COLS; j += 2) {
                        const size_t t = (cbase + j) >> 1;
                        if (t < n) gemm_emit<SHARED>(to, rows, t, acc[j] + acc[j + 1]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < C::DRAIN_COLS; j++) {
                        const size_t t = cbase + j;
                        if (t < n) gemm_emit<SHARED>(to, rows, t, acc[j]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ---- the dense pair kernel: Q8_0 and Q6_K above the small-M kernel's range --------------------
// Those formats scale every 32 (Q8_0) or 16 (Q6_K) weights by a factor of their own,
// so their integer quants cannot share an accumulator the way Q4_K's sc*q do, and a
// weight times its scales does not fit f16's 11 bits.  Their large-M product therefore
// runs on dequantized weights carried exactly as two f16 terms: a row panel of W is
// decoded (bit-exact decoders of formats.cuh), scaled by a power of two per row so
// that its largest weight lands in [8, 16), and written as hi = f16(w) and
// lo = f16(w - hi) (22 bits between them); the kernel below multiplies
// (hi + lo) . x with two MMAs per 16 of K into one TMEM accumulator over the whole of
// K, and the epilogue multiplies by the row's and the token's powers of two again.
// Plain tcgen05 pipeline: warp 0 feeds hi, lo and activation tiles by TMA, warp 1
// issues the MMAs, warps 2-5 (one per TMEM lane quadrant) drain and store.
struct PairArgs {
    size_t rows;            // weight rows of the whole matrix (the pitch of aux)
    size_t panel_row0;      // first row of this panel
    size_t panel_rows;      // rows in this panel
    size_t n, ncols, kblocks;
    int split;
    OutSpec out;
    const float *row_scale;   // [panel_rows]
    const float *tok_scale;   // [n]
    const float *aux;
    int epi;
    uint32_t *status;
};
template <int BN> struct PairCfg {
    static constexpr int STAGE = 2 * A_BYTES + BN * BK * 2;
    static constexpr int STAGES = (MAX_SMEM - 4096 - BN * 4) / STAGE > 6 ? 6 : (MAX_SMEM - 4096 - BN * 4) / STAGE;
    static constexpr int SMEM = 2048 + STAGES * STAGE + BN * 4 + 1024;
    static_assert(STAGES >= 3 && SMEM <= MAX_SMEM, "the pair kernel's stages do not fit");
};
constexpr int PAIR_THREADS = 6 * 32;

template <int BN, bool SHARED>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_hi, const __grid_constant__ CUtensorMap tmap_lo,
                 const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ PairArgs a) {
    using C = PairCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t full0 = base, empty0 = base + 64, accfull = base + 128, tmem_slot = base + 136;
    const uint32_t stage0 = base + 1024, tok0 = stage0 + C::STAGES * C::STAGE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * TILE_M, col0 = blockIdx.y * BN;
    const int kblocks = (int)a.kblocks;
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(accfull, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, BN < 32 ? 32 : BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = lds32(tmem_slot);
    griddep_launch();
    if (warp == 0) {
        griddep_wait();   // the weight panel and the activations' operand come from the kernels just ahead
        if (lane == 0) {
            for (int kb = 0; kb < kblocks; kb++) {
                const int s = kb % C::STAGES;
                mbar_wait_parked(empty0 + 8 * s, ((kb / C::STAGES) & 1) ^ 1, a.status, 0x100000u);
                mbar_expect_tx(full0 + 8 * s, C::STAGE);
                const uint32_t st = stage0 + s * C::STAGE;
                tma_load_2d(st, &tmap_hi, kb * BK, row0, full0 + 8 * s);
                tma_load_2d(st + A_BYTES, &tmap_lo, kb * BK, row0, full0 + 8 * s);
                tma_load_2d(st + 2 * A_BYTES, &tmap_x, kb * BK, col0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        constexpr uint32_t idesc = idesc_f16(TILE_M, BN);
        constexpr uint32_t desc_hi = 64u | (1u << 14) | (2u << 29);   // stride offset 1024 B, version 1, 128-byte swizzle
        const uint32_t tm = __shfl_sync(0xffffffffu, tmem_base, 0);
        for (int kb = 0; kb < kblocks; kb++) {
            const int s = kb % C::STAGES;
            mbar_wait_parked(full0 + 8 * s, (kb / C::STAGES) & 1, a.status, 0x200000u);
            tc_fence_after();
            const uint32_t st = stage0 + s * C::STAGE;
            const uint32_t hi_lo = ((st & 0x3ffffu) >> 4) | (1u << 16), lo_lo = (((st + A_BYTES) & 0x3ffffu) >> 4) | (1u << 16);
            const uint32_t b_lo = (((st + 2 * A_BYTES) & 0x3ffffu) >> 4) | (1u << 16);
            if (lane == 0) {
#pragma unroll
                for (int k = 0; k < BK / 16; k++) {
                    if (kb == 0 && k == 0) umma_f16_lo<0>(tm, hi_lo, b_lo, desc_hi, idesc);
                    else umma_f16_lo<1>(tm, hi_lo + 2 * k, b_lo + 2 * k, desc_hi, idesc);
                    umma_f16_lo<1>(tm, lo_lo + 2 * k, b_lo + 2 * k, desc_hi, idesc);
                }
                umma_commit(empty0 + 8 * s);
                if (kb == kblocks - 1) umma_commit(accfull);
            }
            __syncwarp();
        }
    } else {
        const int quad = warp & 3;
        const int rl = quad * 32 + lane;
        griddep_wait();   // the kernel ahead may still read or write `out` and `aux`
        for (int j = lane; j < BN; j += 32) {
            const size_t t = ((size_t)col0 + j) >> (a.split ? 1 : 0);
            sts32f(tok0 + j * 4, t < a.n ? a.tok_scale[t] : 0.0f);
        }
        __syncwarp();
        const size_t prow = (size_t)row0 + rl;                 // row within the panel
        const bool live = prow < a.panel_rows;
        const float rs = live ? a.row_scale[prow] : 0.0f;
        mbar_wait_parked(accfull, 0, a.status, 0x400000u);
        tc_fence_after();
        // destinations of this thread's row, by constant index (see EmitTo)
        const EmitTo to = emit_to(a.out, a.aux, a.epi, a.panel_row0 + prow);
        const size_t n = a.n, rows = a.rows;
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
        for (int c = 0; c < BN / 16; c++) {
            uint32_t v[16];
            tmem_ld16(taddr + c * 16, v);
            tmem_ld_wait();
            if (!live) continue;
            const size_t cbase = (size_t)col0 + c * 16;
            if (a.split) {
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    const size_t t = (cbase + j) >> 1;
                    if (t < n) gemm_emit<SHARED>(to, rows, t, (__uint_as_float(v[j]) + __uint_as_float(v[j + 1])) * rs * lds32f(tok0 + (c * 16 + j) * 4));
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const size_t t = cbase + j;
                    if (t < n) gemm_emit<SHARED>(to, rows, t, __uint_as_float(v[j]) * rs * lds32f(tok0 + (c * 16 + j) * 4));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, BN < 32 ? 32 : BN);
}

// A row of W decoded, scaled by its own power of two and written as two f16 terms, each run of
// four k in the order (0, 2, 1, 3) the activations' operand is stored in.  One block per row; the
// decoded row waits in shared memory (cols floats) while its largest magnitude is found.
__global__ void __launch_bounds__(256) dequant_pair_kernel(const WeightView w, size_t row0, size_t cols, __half *__restrict__ hi,
                                                           __half *__restrict__ lo, float *__restrict__ row_scale) {
    griddep_launch();
    griddep_wait();   // the kernel ahead may still read the panel
    extern __shared__ __align__(16) float wrow[];
    __shared__ float part[8];
    const size_t r = row0 + blockIdx.x;
    const uint8_t *row = w.quants + r * w.qpitch;
    float amax = 0.0f;
    for (size_t k = (size_t)threadIdx.x * 4; k < cols; k += 1024) {   // four consecutive weights: one sub-block, one scale
        float v[4];
        if (w.fmt == Q6_K) {
            const uint8_t *blk = row + (k >> 8) * Q6_K_DEV;
            const float d = __half2float(w.scales[r * w.srow + (k >> 8)]);
#pragma unroll
            for (int i = 0; i < 4; i++) v[i] = q6k_weight(blk, d, (int)(k & 255) + i);
        } else {
            // gpu/quant.rs:48-62: q as f32 * d
            const float d = __half2float(w.scales[r * w.srow + (k >> 5)]);
            const uint32_t q4 = *reinterpret_cast<const uint32_t *>(row + k);
#pragma unroll
            for (int i = 0; i < 4; i++) v[i] = __fmul_rn((float)(int8_t)(q4 >> (8 * i)), d);
        }
        *reinterpret_cast<float4 *>(wrow + k) = make_float4(v[0], v[1], v[2], v[3]);
        amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fmaxf(fabsf(v[2]), fabsf(v[3])), amax));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = part[0];
#pragma unroll
    for (int i = 1; i < 8; i++) amax = fmaxf(amax, part[i]);
    int e = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 130;     // the largest weight to [8, 16)
    e = amax > 0.0f ? max(-100, min(100, e)) : 0;
    const float down = __uint_as_float((uint32_t)(127 - e) << 23);
    if (threadIdx.x == 0) row_scale[blockIdx.x] = __uint_as_float((uint32_t)(127 + e) << 23);
    __half *h = hi + (size_t)blockIdx.x * cols, *l = lo + (size_t)blockIdx.x * cols;
    for (size_t k = (size_t)threadIdx.x * 4; k < cols; k += 1024) {
        const float4 v4 = *reinterpret_cast<const float4 *>(wrow + k);
        const float v[4] = {v4.x * down, v4.y * down, v4.z * down, v4.w * down};
        uint32_t a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            a[i] = to_f16_bits(v[i]);
            b[i] = to_f16_bits(v[i] - from_f16_bits(a[i]));
        }
        *reinterpret_cast<uint2 *>(h + k) = make_uint2(a[0] | (a[2] << 16), a[1] | (a[3] << 16));
        *reinterpret_cast<uint2 *>(l + k) = make_uint2(b[0] | (b[2] << 16), b[1] | (b[3] << 16));
    }
}

// ---- host side ---------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiled)p;
    }();
    return fn;
}

int encode_2d(dwim_b200_ctx *ctx, CUtensorMap *map, CUtensorMapDataType type, const void *ptr, uint64_t inner, uint64_t outer,
              uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle, const char *what) {
    EncodeTiled enc = encode_fn();
    if (!enc) return fail(ctx, DWIM_B200_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {inner, outer}, strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_outer}, es[2] = {1, 1};
    CUresult r = enc(map, type, 2, const_cast<void *>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, DWIM_B200_ECUDA, "encoding the %s tensor map failed (%d)", what, (int)r);
    return 0;
}

template <int BN>
int launch_gemm(dwim_b200_ctx *ctx, const WeightView &w, const __half *operand, size_t n, int split, const OutSpec &out,
                const float *aux, int epi) {
    using C = Cfg<BN>;
    const size_t ncols = n * (split ? 2 : 1), units = w.cols / 256;
    CUtensorMap tw, tx, tm;
    int rc;
    // packed weights as bytes: [rows][qpitch], box [128 rows][144 bytes]; rows past the end read as zero blocks
    if ((rc = encode_2d(ctx, &tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, w.quants, w.qpitch, w.rows, w.qpitch, 144, TILE_M,
                        CU_TENSOR_MAP_SWIZZLE_NONE, "weight")))
        return rc;
    // activations: [ncols][K] f16, box [BN][64], 128-byte swizzle; columns past the end read as zero
    if ((rc = encode_2d(ctx, &tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, operand, w.cols, ncols, w.cols * 2, BK, BN,
                        CU_TENSOR_MAP_SWIZZLE_128B, "activation")))
        return rc;
    // sub-block means: [ncols][units*16] f16, box [BN][8]
    if ((rc = encode_2d(ctx, &tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, operand + ncols * w.cols, units * 16, ncols, units * 32, 8,
                        BN, CU_TENSOR_MAP_SWIZZLE_NONE, "means")))
        return rc;
    const float *tok_scale = reinterpret_cast<const float *>(operand + ncols * w.cols + ncols * units * 16);
    GemmArgs a{w.rows, n, ncols, units, split, out, tok_scale, aux, epi, ctx->status};
    // A result shared by several ranks' copies takes an instantiation that stores to all of them: with
    // TMA from shared memory when every copy's slice starts on a 16-byte boundary, else from registers.
    int shared = out.world > 1 && !out.scatter_per ? 1 : 0;
    OutMaps maps;          // only the TMA form reads it
    if (shared && epi == EPI_STORE && out.pitch % 4 == 0) {
        shared = 2;
        for (int p = 0; p < out.world; p++)
            if (reinterpret_cast<uintptr_t>(out.dst[p] + out.row0) % 16) shared = 1;
        for (int p = 0; p < out.world && shared == 2; p++)
            if ((rc = encode_2d(ctx, &maps.m[p], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, out.dst[p] + out.row0, w.rows, n,
                                out.pitch * sizeof(float), TILE_M, (uint32_t)(C::DRAIN_COLS >> (split ? 1 : 0)),
                                CU_TENSOR_MAP_SWIZZLE_NONE, "output")))
                return rc;
    }
    auto kern = shared == 2 ? gemm_q4k_kernel<BN, 2> : shared == 1 ? gemm_q4k_kernel<BN, 1> : gemm_q4k_kernel<BN, 0>;
    static bool configured[64][3] = {};
    if (!configured[ctx->device & 63][shared]) {
        DWIM_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        configured[ctx->device & 63][shared] = true;
    }
    dim3 grid((unsigned)((w.rows + TILE_M - 1) / TILE_M), (unsigned)((ncols + BN - 1) / BN));
    const bool dependent = !ctx->weights_written;   // see dwim_b200_ctx::weights_written
    DWIM_CUDA(ctx, launch_dependent(dependent, kern, grid, dim3(GEMM_THREADS), (size_t)C::SMEM, ctx->stream, tw, tx, tm, a, maps));
    ctx->weights_written = false;
    DWIM_LAUNCHED(ctx);
    return 0;
}

constexpr size_t PAIR_PANEL_ROWS = 16384;   // rows decoded at a time: 335 MB of f16 pairs at 5120 columns

template <int BN>
int launch_pair(dwim_b200_ctx *ctx, const WeightView &w, size_t r0, size_t nr, const __half *operand, size_t n, int split,
                const OutSpec &out, const float *aux, int epi) {
    using C = PairCfg<BN>;
    const size_t ncols = n * (split ? 2 : 1), units = w.cols / 256;
    const __half *hi = ctx->pair_hi, *lo = ctx->pair_lo;
    CUtensorMap th, tl, tx;
    int rc;
    if ((rc = encode_2d(ctx, &th, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, hi, w.cols, nr, w.cols * 2, BK, TILE_M, CU_TENSOR_MAP_SWIZZLE_128B,
                        "weight panel (hi)")))
        return rc;
    if ((rc = encode_2d(ctx, &tl, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, lo, w.cols, nr, w.cols * 2, BK, TILE_M, CU_TENSOR_MAP_SWIZZLE_128B,
                        "weight panel (lo)")))
        return rc;
    if ((rc = encode_2d(ctx, &tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, operand, w.cols, ncols, w.cols * 2, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B,
                        "activation")))
        return rc;
    const float *tok_scale = reinterpret_cast<const float *>(operand + ncols * w.cols + ncols * units * 16);
    PairArgs a{w.rows, r0, nr, n, ncols, w.cols / BK, split, out, ctx->pair_scale, tok_scale, aux, epi, ctx->status};
    const bool shared = out.world > 1 && !out.scatter_per;
    auto kern = shared ? gemm_pair_kernel<BN, true> : gemm_pair_kernel<BN, false>;
    static bool configured[64][2] = {};
    if (!configured[ctx->device & 63][shared]) {
        DWIM_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        configured[ctx->device & 63][shared] = true;
    }
    dim3 grid((unsigned)((nr + TILE_M - 1) / TILE_M), (unsigned)((ncols + BN - 1) / BN));
    DWIM_CUDA(ctx, launch_dependent(true, kern, grid, dim3(PAIR_THREADS), (size_t)C::SMEM, ctx->stream, th, tl, tx, a));
    DWIM_LAUNCHED(ctx);
    return 0;
}

}  // namespace

// Formats the tensor-core kernels take: Q4_K by the kernel that multiplies its integers
// directly, the others as dequantized f16 pairs, a panel of rows at a time.
bool gemm_supports(const WeightView &w) {
    if (w.cols % 256) return false;
    return w.fmt == Q4_K || ((w.fmt == Q6_K || w.fmt == Q8_0) && w.cols <= 12288);
}

int gemm_large(dwim_b200_ctx *ctx, const WeightView &w, const __half *operand, size_t n, int split, const OutSpec &out,
               const float *aux, int epilogue) {
    if (!gemm_supports(w)) return fail(ctx, DWIM_B200_EFORMAT, "the tensor-core GEMM does not take format %d", w.fmt);
    const size_t ncols = n * (split ? 2 : 1);
    if (w.fmt == Q4_K) {
        if (ncols <= 32) return launch_gemm<32>(ctx, w, operand, n, split, out, aux, epilogue);
        if (ncols <= 64) return launch_gemm<64>(ctx, w, operand, n, split, out, aux, epilogue);
        if (ncols <= 128) return launch_gemm<128>(ctx, w, operand, n, split, out, aux, epilogue);
        return launch_gemm<256>(ctx, w, operand, n, split, out, aux, epilogue);
    }
    if (w.cols * sizeof(float) > 48 * 1024)
        return fail(ctx, DWIM_B200_EINVAL, "dense kernel: rows of %zu weights are too long for the decoder's shared memory", w.cols);
    // the panel's buffers: created on first use, grown when a wider matrix comes
    const size_t panel = w.rows < PAIR_PANEL_ROWS ? (w.rows + TILE_M - 1) / TILE_M * TILE_M : PAIR_PANEL_ROWS;
    const size_t need = panel * w.cols;
    if (need > ctx->pair_cap) {
        if (ctx->pair_hi) {
            DWIM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            cudaFree(ctx->pair_hi);
            cudaFree(ctx->pair_lo);
            ctx->pair_hi = ctx->pair_lo = nullptr;
            ctx->pair_cap = 0;
        }
        DWIM_CUDA(ctx, cudaMalloc((void **)&ctx->pair_hi, need * sizeof(__half)));
        DWIM_CUDA(ctx, cudaMalloc((void **)&ctx->pair_lo, need * sizeof(__half)));
        if (!ctx->pair_scale) DWIM_CUDA(ctx, cudaMalloc((void **)&ctx->pair_scale, PAIR_PANEL_ROWS * sizeof(float)));
        ctx->pair_cap = need;
    }
    for (size_t r0 = 0; r0 < w.rows; r0 += panel) {
        const size_t nr = w.rows - r0 < panel ? w.rows - r0 : panel;
        DWIM_CUDA(ctx, launch_dependent(!ctx->weights_written, dequant_pair_kernel, dim3((unsigned)nr), dim3(256), w.cols * sizeof(float),
                                        ctx->stream, w, r0, w.cols, ctx->pair_hi, ctx->pair_lo, ctx->pair_scale));
        ctx->weights_written = false;
        DWIM_LAUNCHED(ctx);
        int rc;
        if (ncols <= 64) rc = launch_pair<64>(ctx, w, r0, nr, operand, n, split, out, aux, epilogue);
        else if (ncols <= 128) rc = launch_pair<128>(ctx, w, r0, nr, operand, n, split, out, aux, epilogue);
        else rc = launch_pair<256>(ctx, w, r0, nr, operand, n, split, out, aux, epilogue);
        if (rc) return rc;
    }
    return 0;
}

void gemm_release(dwim_b200_ctx *ctx) {
    if (ctx->pair_hi) cudaFree(ctx->pair_hi);
    if (ctx->pair_lo) cudaFree(ctx->pair_lo);
    if (ctx->pair_scale) cudaFree(ctx->pair_scale);
    ctx->pair_hi = ctx->pair_lo = nullptr;
    ctx->pair_scale = nullptr;
    ctx->pair_cap = 0;
}

}  // namespace dwim
