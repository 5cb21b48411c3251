// Activation prologue: f32 activations -> the 16-bit operand forms the matmul
// kernels read.  The reference does the same with its f16 shadow buffers
// (`halves`, gpu/cuda/mod.rs:313-384; to_f16.cu:6-18): convert once, reuse for
// every matmul that takes the same input.
//
// Panels (small-M kernel).  K is cut in units of 256 weights.  For unit u and
// column c the panel is PANEL_STRIDE = 272 halves:
//     [0, 256)   the column's activations for k in [256u, 256u+256)
//     [256, 272) per-32-weight means of those activations (Q4_K only),
//                each as a hi and a lo half: entry 4p+{0,1} = hi of sub-blocks
//                2p, 2p+1; entry 4p+{2,3} = their lo parts
// laid out [unit][column][272].  A "column" is one token (single mode) or one
// half of a token: with split = 1 token t owns columns 2t (x rounded to f16)
// and 2t+1 (the rounding's remainder, again as f16), so that hi + lo carries
// 22 bits of the f32 activation and the tensor-core products stay exact.
//
// Order of k inside [0, 256):
//   natural (Q8_0, Q6_K): position = k.
//   Q4_K: the kernel's lane c (0..3) owns the 64 weights [64c, 64c+64) and
//   unpacks bytes (0, 2) and (1, 3) of each 32-bit word together, so each run
//   of four k is stored in the order (0, 2, 1, 3); and the 8-byte runs are
//   XOR-swizzled by c so that the four lanes of a row hit different banks:
//     run  = 16c + 8*nib + (j ^ c)      k = 64c + 32*nib + 4j + e
//     position = 4*run + {0,2,1,3}[e]
#include "common.cuh"
#include "ptx.cuh"

namespace dwim {

size_t panel_bytes(size_t cols, int ncols) {
    size_t units = (cols + 255) / 256;
    return units * (size_t)ncols * PANEL_STRIDE * sizeof(__half);
}

__device__ __forceinline__ int panel_pos_q4k(int k) {
    int c = k >> 6, nib = (k >> 5) & 1, j = (k >> 2) & 7, e = k & 3;
    int run = 16 * c + 8 * nib + (j ^ c);
    int pe = ((e & 1) << 1) | (e >> 1);   // 0,1,2,3 -> 0,2,1,3
    return 4 * run + pe;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// grid (units, tokens), 256 threads: thread k converts x[t][256u + k].
template <bool Q4K>
__global__ void __launch_bounds__(256) panel_kernel(const float *__restrict__ x, size_t cols, int ncols, int split,
                                                    __half *__restrict__ panels) {
    // as panel_i8_kernel: let the next small-M launch begin, wait for the kernel ahead
    griddep_launch();
    griddep_wait();
    int u = blockIdx.x, t = blockIdx.y, k = threadIdx.x;
    size_t kk = (size_t)u * 256 + k;
    float v = kk < cols ? x[(size_t)t * cols + kk] : 0.0f;
    __half hi = to_f16_clamped(v);
    float rem = v - __half2float(hi);
    __half lo = to_f16_clamped(rem);
    int pos = Q4K ? panel_pos_q4k(k) : k;
    int col = split ? 2 * t : t;
    __half *p = panels + ((size_t)u * ncols + col) * PANEL_STRIDE;
    p[pos] = hi;
    if (split) p[PANEL_STRIDE + pos] = lo;
    // means of the 32 activations of each sub-block (a warp = a sub-block)
    float mh = 0.0f, ml = 0.0f;
    if (Q4K) {
        mh = warp_sum(__half2float(hi)) * (1.0f / 32.0f);
        ml = warp_sum(__half2float(lo)) * (1.0f / 32.0f);
    }
    if ((k & 31) == 0) {
        int j = k >> 5;
        int e = 256 + 4 * (j >> 1) + (j & 1);
        __half a = to_f16_clamped(mh);
        p[e] = a;
        p[e + 2] = to_f16_clamped(mh - __half2float(a));
        if (split) {
            __half b = to_f16_clamped(ml);
            p[PANEL_STRIDE + e] = b;
            p[PANEL_STRIDE + e + 2] = to_f16_clamped(ml - __half2float(b));
        }
    }
}

int build_panels(dwim_b200_ctx *ctx, const float *x, size_t n, size_t cols, int kind, int split, __half *panels) {
    if (n == 0 || cols == 0) return 0;
    size_t units = (cols + 255) / 256;
    if (n > 65535) return fail(ctx, DWIM_B200_EINVAL, "too many tokens for one panel build: %zu", n);
    dim3 grid((unsigned)units, (unsigned)n);
    int ncols = (int)n * (split ? 2 : 1);
    if (kind == SHADOW_PANEL_Q4K)
        DWIM_CUDA(ctx, launch_dependent(!ctx->weights_written, panel_kernel<true>, grid, dim3(256), 0, ctx->stream, x, cols, ncols, split, panels));
    else
        DWIM_CUDA(ctx, launch_dependent(!ctx->weights_written, panel_kernel<false>, grid, dim3(256), 0, ctx->stream, x, cols, ncols, split, panels));
    DWIM_LAUNCHED(ctx);
    return 0;
}

// Operands of the tensor-core GEMM (Q4_K).  Two arrays, one row per column
// (a column is a token, or with split = 1 a token's hi or lo half, columns 2t
// and 2t+1):
//   x16   [ncols][K] f16      the activations; each run of four k is stored in
//                             the order (0, 2, 1, 3), the order the dequantizer
//                             produces weights in (it unpacks bytes 0,2 and 1,3
//                             of a word together)
//   means [ncols][K/256][16]  per 32-weight sub-block the mean of the column's
//                             f16 values, as a hi half (entries 0-7) and the
//                             remainder (entries 8-15): the operand the
//                             sub-block minimums are multiplied with
// ---- int8 digit planes (one- and two-token Q4_K kernel) --------------------------------
// A unit's 256 activations of a token share one exponent e (|x| < 2^e for all of
// them) and become 31-bit fixed point, Y = rint(x * 2^(30-e)), written as four
// signed base-256 digits: Y = d0*2^24 + d1*2^16 + d2*2^8 + d3, each in
// [-128, 127].  An activation within 2^-6 of the unit's largest is exact; a
// smaller one is rounded at 2^-31 of the largest.  Plane p of token t is column
// 4t + p of the int8 MMA; a unit of its digit is worth 2^(e-6-8p).
// One block per (unit, token slot); warp j owns sub-block j.
size_t panel_i8_bytes(size_t cols, size_t n) { return ((cols + 255) / 256) * (size_t)i8_unit_bytes(4 * (int)n); }

__global__ void __launch_bounds__(256) panel_i8_kernel(const float *__restrict__ x, size_t cols, int n, uint8_t *__restrict__ panels) {
    // the small-M kernel launched next may start streaming its weights now; the
    // panels may still be read, and x written, by the kernel ahead
    griddep_launch();
    griddep_wait();
    const int u = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, j = tid >> 5, lane = tid & 31;
    const int nc = 4 * n;
    uint8_t *blob = panels + (size_t)u * i8_unit_bytes(nc);
    const size_t k = (size_t)u * 256 + tid;
    const float v = k < cols ? x[(size_t)t * cols + k] : 0.0f;
    // the unit's largest magnitude
    __shared__ float wmax[8];
    float m = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) wmax[j] = m;
    __syncthreads();
    m = wmax[0];
#pragma unroll
    for (int i = 1; i < 8; i++) m = fmaxf(m, wmax[i]);
    // |x| < 2^e; floored so that the planes' worths stay normal floats
    int e = m > 0.0f ? (int)((__float_as_uint(m) >> 23) & 0xffu) - 126 : -90;
    if (e < -90) e = -90;
    const float up = __uint_as_float((uint32_t)(127 + 15 - (e >> 1)) << 23) * __uint_as_float((uint32_t)(127 + 15 - (e - (e >> 1))) << 23);
    int y = __float2int_rn(v * up);   // v * 2^(30-e), |y| <= 2^30
    int d[4];
#pragma unroll
    for (int p = 3; p > 0; p--) {
        d[p] = ((y + 128) & 255) - 128;
        y = (y - d[p]) >> 8;
    }
    d[0] = y;
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const int col = 4 * t + p;
        blob[(j * nc + col) * 32 + lane] = (uint8_t)(int8_t)d[p];
        int s = d[p];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) {
            const int b = ((s + 64) & 127) - 64, a = (s - b) >> 7;   // s = 128*a + b
            blob[256 * nc + col * 16 + j] = (uint8_t)(int8_t)a;
            blob[256 * nc + col * 16 + 8 + j] = (uint8_t)(int8_t)b;
        }
        if (tid == 0)
            reinterpret_cast<float *>(blob + 272 * nc)[col] = __uint_as_float((uint32_t)(127 + e - 6 - 8 * p) << 23);
    }
}

int build_panels_i8(dwim_b200_ctx *ctx, const float *x, size_t n, size_t cols, uint8_t *panels) {
    if (n == 0 || cols == 0) return 0;
    if (n > I8_MAX_TOKENS) return fail(ctx, DWIM_B200_EINVAL, "int8 panels take at most %d tokens, not %zu", I8_MAX_TOKENS, n);
    dim3 grid((unsigned)((cols + 255) / 256), (unsigned)n);
    DWIM_CUDA(ctx, launch_dependent(!ctx->weights_written, panel_i8_kernel, grid, dim3(256), 0, ctx->stream, x, cols, (int)n, panels));
    DWIM_LAUNCHED(ctx);
    return 0;
}

size_t gemm_operand_bytes(size_t cols, size_t ncols) {
    return ncols * cols * sizeof(__half) + ncols * (cols / 256) * 16 * sizeof(__half);
}

// grid (ceil(units / 4), tokens), 256 threads: a thread takes four consecutive
// activations (one 16-byte load, one 8-byte store per column), eight threads a
// 32-wide sub-block, 64 a unit.
template <bool ALIGNED>   // whether x is 16-byte aligned (a wrapped caller's pointer need not be)
__global__ void __launch_bounds__(256) gemm_operand_kernel(const float *__restrict__ x, size_t cols, size_t units, int split,
                                                           __half *__restrict__ x16, __half *__restrict__ means) {
    // as the small-M prologues: let the product's kernel begin (it streams weights first),
    // wait for the kernel ahead, which may still read the operand or write x
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.y, k = threadIdx.x;
    const size_t u = (size_t)blockIdx.x * 4 + (k >> 6);
    if (u >= units) return;                           // whole 64-thread groups leave together
    const size_t at = u * 256 + (size_t)(k & 63) * 4;
    const float *src = x + (size_t)t * cols + at;
    float f[4];
    if (ALIGNED) {
        const float4 v = *reinterpret_cast<const float4 *>(src);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    } else {
#pragma unroll
        for (int e = 0; e < 4; e++) f[e] = src[e];
    }
    __half hi[4], lo[4];
    float sh = 0.0f, sl = 0.0f;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        hi[e] = to_f16_clamped(f[e]);
        lo[e] = to_f16_clamped(f[e] - __half2float(hi[e]));
        sh += __half2float(hi[e]);
        sl += __half2float(lo[e]);
    }
    // a group of four goes out in the order (0, 2, 1, 3): the order the weights' bytes decode in
    const size_t col = split ? 2 * (size_t)t : (size_t)t;
    auto pack = [](const __half (&h)[4]) {
        uint2 r;
        r.x = (uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[2]) << 16);
        r.y = (uint32_t)__half_as_ushort(h[1]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
        return r;
    };
    *reinterpret_cast<uint2 *>(x16 + col * cols + at) = pack(hi);
    if (split) *reinterpret_cast<uint2 *>(x16 + (col + 1) * cols + at) = pack(lo);
    // sub-block sums over the eight threads that share it
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        sh += __shfl_xor_sync(0xffffffffu, sh, o);
        sl += __shfl_xor_sync(0xffffffffu, sl, o);
    }
    if ((k & 7) == 0) {
        const int j = (k & 63) >> 3;
        const float mh = sh * (1.0f / 32.0f), ml = sl * (1.0f / 32.0f);
        __half *m = means + (col * units + u) * 16;
        const __half a = to_f16_clamped(mh);
        m[j] = a;
        m[8 + j] = to_f16_clamped(mh - __half2float(a));
        if (split) {
            __half *m2 = m + units * 16;
            const __half b = to_f16_clamped(ml);
            m2[j] = b;
            m2[8 + j] = to_f16_clamped(ml - __half2float(b));
        }
    }
}

int build_gemm_operand(dwim_b200_ctx *ctx, const float *x, size_t n, size_t cols, int split, __half *out) {
    if (n == 0 || cols == 0) return 0;
    if (cols % 256) return fail(ctx, DWIM_B200_EINVAL, "GEMM operand: %zu columns are not whole 256-weight units", cols);
    if (n > 65535) return fail(ctx, DWIM_B200_EINVAL, "too many tokens for one operand build: %zu", n);
    const size_t units = cols / 256, ncols = n * (split ? 2 : 1);
    dim3 grid((unsigned)((units + 3) / 4), (unsigned)n);
    const bool dependent = !ctx->weights_written;
    if (reinterpret_cast<uintptr_t>(x) % 16 == 0)
        DWIM_CUDA(ctx, launch_dependent(dependent, gemm_operand_kernel<true>, grid, dim3(256), 0, ctx->stream, x, cols, units, split,
                                        out, out + ncols * cols));
    else
        DWIM_CUDA(ctx, launch_dependent(dependent, gemm_operand_kernel<false>, grid, dim3(256), 0, ctx->stream, x, cols, units, split,
                                        out, out + ncols * cols));
    DWIM_LAUNCHED(ctx);
    return 0;
}

}  // namespace dwim
