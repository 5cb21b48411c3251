// The large-M product (prefill, long verify batches): a dense contraction on
// the 5th-generation tensor cores.  Replaces the reference's matmul_tile64_*
// kernels (matmul_tile.cu:94-258; host side gpu/cuda/mod.rs:402-442).
//
// out[t][r] = sum_k W[r][k] * X[t][k].  A CTA owns a tile of 128 weight rows
// (the MMA's M side, one TMEM lane per row) by BN tokens (the N side, one TMEM
// column per token) and walks K in blocks of 64:
//
//   warp 0       TMA producer.  Per 256 weights of K one tiled tensor copy
//                brings the tile's packed blocks ([128 rows][144 B] for Q4_K)
//                into a raw ring; per K block one tensor copy brings the
//                activations' f16 tile ([BN][64], 128-byte swizzle).
//   warps 6-13   dequantizers.  Thread (row, half) decodes 32 weights of its
//                row from the raw ring in fp32 — fma(d*sc, q, -dmin*m), the
//                reference's order — rounds once to f16 (as the reference's
//                tile kernel does, matmul_tile.cu:66-74) and stores them into
//                the stage's A tile in the canonical K-major 128-byte-swizzled
//                layout the MMA's shared-memory descriptor expects.
//   warp 1       MMA issuer: one thread issues four tcgen05.mma (M=128, N=BN,
//                K=16, f16 x f16 -> f32 in TMEM) per K block and commits the
//                stage back to the producers.
//   warps 2-5    epilogue: tcgen05.ld the accumulators (32 lanes x 32 columns
//                per warp and instruction), apply the operator's mode
//                (store / add / SwiGLU) and write out[t][r], coalesced over r.
//
// Every mbarrier wait is bounded (ptx.cuh); a kernel that gave up says so in
// the context's status word.
#include <cuda.h>

#include "common.cuh"
#include "ptx.cuh"

namespace dwim {

namespace {

constexpr int TILE_M = 128;   // weight rows per CTA
constexpr int BK = 64;        // K per stage: one 128-byte swizzled row of f16
constexpr int RAW_STAGES = 3;
constexpr int N_DEQ_WARPS = 8;
constexpr int GEMM_THREADS = (6 + N_DEQ_WARPS) * 32;

struct GemmArgs {
    size_t rows, n, units;   // weight rows, tokens, 256-weight units of K
    float *out;
    const float *aux;
    int epi;
    uint32_t *status;
};

template <int BN> struct Cfg {
    static constexpr int STAGES = BN >= 256 ? 3 : 4;
    static constexpr int A_BYTES = TILE_M * BK * 2;            // 16 KB
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int RAW_BYTES = ((TILE_M * 144 + 1023) / 1024) * 1024;   // Q4_K: 18 KB
    static constexpr int BAR_BYTES = 1024;
    static constexpr int SMEM = BAR_BYTES + STAGES * STAGE_BYTES + RAW_STAGES * RAW_BYTES + 1024;   // + alignment slack
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
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
// Arrive on an mbarrier once every MMA this thread issued so far has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes
// (64 f16), 128-byte swizzled, eight-row groups 1024 bytes apart:
//   [0,14) address >> 4   [16,30) leading offset >> 4 (unused for swizzled
//   K-major: 1)   [32,46) stride between eight-row groups >> 4 (64)
//   [46,48) descriptor version 1   [61,64) layout 2 = 128-byte swizzle
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr & 0x3ffffu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: f32 accumulate (bits 4-5 = 1), f16 A and B (0),
// both K-major (0), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    uint32_t r;   // cvt packs its first source into the upper half
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ float silu_mul_f(float g, float u) { return g * (1.0f / (1.0f + expf(-g))) * u; }

// ---- Q4_K dequantizer: 32 weights of one row ---------------------------------------
// Thread (row, h) of K block `g` (0..3 inside the 256-weight unit) decodes
// sub-block 2g + h: nibble h of the 32 bytes of group g.
__device__ __forceinline__ void dequant_q4k_32(uint32_t raw_row, int g, int h, uint32_t a_row, int row7) {
    const uint4 hdr = lds128(raw_row);
    const uint4 q0 = lds128(raw_row + 16 + 32 * g), q1 = lds128(raw_row + 32 + 32 * g);
    // the 6-bit scale and minimum of sub-blocks 2g, 2g+1 as two bytes each (see gemv.cu: q4k_scales)
    const int sh = (g & 1) * 16;
    const uint32_t y = (hdr.y >> sh) & 0xffffu, z = (hdr.z >> sh) & 0xffffu, w = (hdr.w >> sh) & 0xffffu;
    const uint32_t sc2 = g < 2 ? (y & 0x3f3fu) : ((w & 0x0f0fu) | ((y >> 2) & 0x3030u));
    const uint32_t m2 = g < 2 ? (z & 0x3f3fu) : (((w >> 4) & 0x0f0fu) | ((z >> 2) & 0x3030u));
    const float sc = (float)((sc2 >> (8 * h)) & 0xffu), m = (float)((m2 >> (8 * h)) & 0xffu);
    const float ds = __fmul_rn(h2f_lo(hdr.x), sc), ndm = -__fmul_rn(h2f_hi(hdr.x), m);
    const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int c = 0; c < 4; c++) {   // 16-byte chunk c of this half: weights 8c .. 8c+7
        uint32_t o[4];
#pragma unroll
        for (int p = 0; p < 2; p++) {
            const uint32_t nib = (words[2 * c + p] >> (4 * h)) & 0x0f0f0f0fu;
            // byte b of nib -> 8388608 + q as a float, then q, then ds*q - dm in one rounding
            const float f0 = __uint_as_float(prmt(nib, 0x4B000000u, 0x7540u)) - 8388608.0f;
            const float f1 = __uint_as_float(prmt(nib, 0x4B000000u, 0x7541u)) - 8388608.0f;
            const float f2 = __uint_as_float(prmt(nib, 0x4B000000u, 0x7542u)) - 8388608.0f;
            const float f3 = __uint_as_float(prmt(nib, 0x4B000000u, 0x7543u)) - 8388608.0f;
            o[2 * p] = pack_f16x2(fmaf(ds, f0, ndm), fmaf(ds, f1, ndm));
            o[2 * p + 1] = pack_f16x2(fmaf(ds, f2, ndm), fmaf(ds, f3, ndm));
        }
        sts128(a_row + (((4 * h + c) ^ row7) << 4), o[0], o[1], o[2], o[3]);
    }
}

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_q4k_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const GemmArgs a) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled tiles
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base;                       // 8-byte barriers
    const uint32_t full0 = bars, empty0 = bars + 64, rawfull0 = bars + 128, rawempty0 = bars + 192, accbar = bars + 256;
    const uint32_t tmem_slot = bars + 320;
    const uint32_t stage0 = base + C::BAR_BYTES;
    const uint32_t raw0 = stage0 + C::STAGES * C::STAGE_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * TILE_M, tok0 = blockIdx.y * BN;
    const int n_kb = (int)a.units * 4;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(full0 + 8 * s, 1 + N_DEQ_WARPS);   // the producer's expect_tx arrival + one per dequant warp
            mbar_init(empty0 + 8 * s, 1);                // the MMA warp's commit
        }
        for (int s = 0; s < RAW_STAGES; s++) {
            mbar_init(rawfull0 + 8 * s, 1);
            mbar_init(rawempty0 + 8 * s, N_DEQ_WARPS);
        }
        mbar_init(accbar, 1);
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

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            for (int kb = 0; kb < n_kb; kb++) {
                if ((kb & 3) == 0) {
                    const int u = kb >> 2, rs = u % RAW_STAGES;
                    mbar_wait(rawempty0 + 8 * rs, ((u / RAW_STAGES) & 1) ^ 1, a.status, 0x10u);
                    mbar_expect_tx(rawfull0 + 8 * rs, TILE_M * 144);
                    tma_load_2d(raw0 + rs * C::RAW_BYTES, &tmap_w, u * 144, row0, rawfull0 + 8 * rs);
                }
                const int s = kb % C::STAGES;
                mbar_wait(empty0 + 8 * s, ((kb / C::STAGES) & 1) ^ 1, a.status, 0x20u);
                mbar_expect_tx(full0 + 8 * s, C::B_BYTES);
                tma_load_2d(stage0 + s * C::STAGE_BYTES + C::A_BYTES, &tmap_x, kb * BK, tok0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        constexpr uint32_t idesc = idesc_f16(TILE_M, BN);
        for (int kb = 0; kb < n_kb; kb++) {
            const int s = kb % C::STAGES;
            mbar_wait(full0 + 8 * s, (kb / C::STAGES) & 1, a.status, 0x40u);
            tc_fence_after();
            if (lane == 0) {
                const uint32_t a_addr = stage0 + s * C::STAGE_BYTES, b_addr = a_addr + C::A_BYTES;
                const uint64_t ad = smem_desc_sw128(a_addr), bd = smem_desc_sw128(b_addr);
#pragma unroll
                for (int k = 0; k < BK / 16; k++)   // 32 bytes further along the swizzled row per K=16
                    umma_f16(tmem_base, ad + 2 * k, bd + 2 * k, idesc, (kb | k) != 0);
                umma_commit(empty0 + 8 * s);                  // the stage may be refilled once these finish
                if (kb == n_kb - 1) umma_commit(accbar);      // and the accumulators are complete
            }
            __syncwarp();
        }
    } else if (warp >= 6) {
        // ------------------------------ dequantizers ------------------------------
        const int dt = threadIdx.x - 6 * 32;      // 0..255
        const int r = dt >> 1, h = dt & 1;
        for (int kb = 0; kb < n_kb; kb++) {
            const int u = kb >> 2, g = kb & 3, rs = u % RAW_STAGES, s = kb % C::STAGES;
            if (g == 0) mbar_wait(rawfull0 + 8 * rs, (u / RAW_STAGES) & 1, a.status, 0x80u);
            mbar_wait(empty0 + 8 * s, ((kb / C::STAGES) & 1) ^ 1, a.status, 0x100u);
            dequant_q4k_32(raw0 + rs * C::RAW_BYTES + r * 144, g, h, stage0 + s * C::STAGE_BYTES + r * 128, r & 7);
            fence_async_smem();      // the tensor core reads shared memory through the async proxy
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(full0 + 8 * s);
                if (g == 3) mbar_arrive(rawempty0 + 8 * rs);
            }
        }
    } else {
        // ------------------------------ epilogue (warps 2-5) ------------------------------
        const int quad = warp & 3;                 // the TMEM lanes this warp may read: 32*quad ..
        const size_t row = (size_t)row0 + quad * 32 + lane;
        mbar_wait(accbar, 0, a.status, 0x200u);
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < BN / 32; c++) {
            uint32_t v[32];
            tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + c * 32, v);
            tmem_ld_wait();
            if (row < a.rows) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const size_t t = (size_t)tok0 + c * 32 + j;
                    if (t < a.n) {
                        const size_t i = t * a.rows + row;
                        float x = __uint_as_float(v[j]);
                        if (a.epi == EPI_ADD) x += a.out[i];
                        else if (a.epi == EPI_SWIGLU) x = silu_mul_f(x, a.aux[i]);
                        a.out[i] = x;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
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

template <int BN>
int launch_gemm(dwim_b200_ctx *ctx, const WeightView &w, const __half *x16, size_t n, float *out, const float *aux, int epi) {
    using C = Cfg<BN>;
    EncodeTiled enc = encode_fn();
    if (!enc) return fail(ctx, DWIM_B200_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMap tw, tx;
    {   // packed weights as bytes: [rows][qpitch], box [128 rows][144 bytes]
        cuuint64_t dims[2] = {w.qpitch, w.rows}, strides[1] = {w.qpitch};
        cuuint32_t box[2] = {144, TILE_M}, es[2] = {1, 1};
        CUresult r = enc(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)w.quants, dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(ctx, DWIM_B200_ECUDA, "encoding the weight tensor map failed (%d)", (int)r);
    }
    {   // activations as f16: [n][cols], box [BN tokens][64], 128-byte swizzle; rows past n read as zero
        cuuint64_t dims[2] = {w.cols, n}, strides[1] = {w.cols * 2};
        cuuint32_t box[2] = {BK, BN}, es[2] = {1, 1};
        CUresult r = enc(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)x16, dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(ctx, DWIM_B200_ECUDA, "encoding the activation tensor map failed (%d)", (int)r);
    }
    GemmArgs a{w.rows, n, w.cols / 256, out, aux, epi, ctx->status};
    auto kern = gemm_q4k_kernel<BN>;
    static bool configured[64] = {false};
    if (!configured[ctx->device & 63]) {
        DWIM_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        configured[ctx->device & 63] = true;
    }
    dim3 grid((unsigned)((w.rows + TILE_M - 1) / TILE_M), (unsigned)((n + BN - 1) / BN));
    kern<<<grid, GEMM_THREADS, C::SMEM, ctx->stream>>>(tw, tx, a);
    DWIM_LAUNCHED(ctx);
    return 0;
}

}  // namespace

bool gemm_available() { return true; }

// Formats and shapes the tensor-core kernel takes; the rest goes through the
// small-M kernel in groups of tokens.
bool gemm_supports(const WeightView &w) { return w.fmt == Q4_K && w.cols % 256 == 0; }

int gemm_large(dwim_b200_ctx *ctx, const WeightView &w, const __half *x16, size_t n, float *out, const float *aux,
               int epilogue) {
    if (!gemm_supports(w)) return fail(ctx, DWIM_B200_EFORMAT, "the tensor-core GEMM does not take format %d", w.fmt);
    if (n <= 32) return launch_gemm<32>(ctx, w, x16, n, out, aux, epilogue);
    if (n <= 64) return launch_gemm<64>(ctx, w, x16, n, out, aux, epilogue);
    if (n <= 128) return launch_gemm<128>(ctx, w, x16, n, out, aux, epilogue);
    return launch_gemm<256>(ctx, w, x16, n, out, aux, epilogue);
}

void gemm_release(dwim_b200_ctx *) {}

}  // namespace dwim
