// Activation prologue: f32 activations -> the operand forms the matmul
// kernels read.  The reference does the same with its f16 shadow buffers
// (`halves`, gpu/cuda/mod.rs:313-384; to_f16.cu:6-18): convert once, reuse for
// every matmul that takes the same input.  Two forms: int8 digit planes per
// 256-wide unit for the small-M kernel (up to eight tokens), and f16 rows with
// sub-block means and a scale per token for the tensor-core kernels; either
// can be written by the same launch that applies the RMS norm in front of the
// product (rmsnorm.cu:11-58).
#include "common.cuh"
#include "ptx.cuh"

namespace dwim {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- int8 digit planes (the small-M kernel's int8 routines) --------------------------------
// A unit's 256 activations of a token share one exponent e (|x| < 2^e for all of
// them) and become fixed point with P signed base-256 digits, Y = rint(x * 2^(8P-2-e))
// = sum_p d_p * 256^(P-1-p), each digit in [-128, 127] (the leading one in [-64, 64]).
// P = 4 for one and two tokens (31 bits: an activation within 2^-6 of the unit's
// largest is exact, a smaller one is rounded at 2^-31 of the largest), P = 3 for
// three to eight (23 bits: rounded at 2^-23 of the unit's largest).  A unit of
// plane p's digit is worth 2^(e-6-8p).  Columns of the int8 MMA:
//   P = 4: column = 4*token + plane   (both tokens' planes share one 8-column tile)
//   P = 3: column = plane*n + token   (tile p of the MMA holds plane p of every token)
size_t panel_i8_bytes(size_t cols, size_t n) { return ((cols + 255) / 256) * (size_t)i8_unit_bytes(i8_planes((int)n) * (int)n); }

// What one thread does with its activation once the unit's largest magnitude is
// known: the digits, their per-sub-block sums, the planes' worths.  `lane` and
// `j` are the thread's place in its sub-block and the sub-block's in the unit.
template <int P>
__device__ __forceinline__ void i8_digits(float v, float m, int t, int n, int j, int lane, bool first, uint8_t *blob) {
    const int nc = P * n;
    // |x| < 2^e; floored so that the planes' worths stay normal floats
    int e = m > 0.0f ? (int)((__float_as_uint(m) >> 23) & 0xffu) - 126 : -90;
    if (e < -90) e = -90;
    if (e > 100) e = 100;
    // v * 2^(8P-2-e) in two steps: either factor is a normal float
    const int s = 8 * P - 2 - e, s1 = s >> 1;
    const float up1 = __uint_as_float((uint32_t)(127 + s1) << 23), up2 = __uint_as_float((uint32_t)(127 + s - s1) << 23);
    const float lim = (float)(1 << (8 * P - 2));
    int y = __float2int_rn(fminf(fmaxf(v * up1 * up2, -lim), lim));   // |y| <= 2^(8P-2); the clamp only matters for inf
    int d[P];
#pragma unroll
    for (int p = P - 1; p > 0; p--) {
        d[p] = ((y + 128) & 255) - 128;
        y = (y - d[p]) >> 8;
    }
    d[0] = y;
#pragma unroll
    for (int p = 0; p < P; p++) {
        const int col = P == 4 ? 4 * t + p : p * n + t;
        blob[(j * nc + col) * 32 + lane] = (uint8_t)(int8_t)d[p];
        int sum = d[p];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) {
            const int b = ((sum + 64) & 127) - 64, a = (sum - b) >> 7;   // sum = 128*a + b
            blob[256 * nc + col * 16 + j] = (uint8_t)(int8_t)a;
            blob[256 * nc + col * 16 + 8 + j] = (uint8_t)(int8_t)b;
        }
        if (first) reinterpret_cast<float *>(blob + 272 * nc)[col] = __uint_as_float((uint32_t)(127 + e - 6 - 8 * p) << 23);
    }
}

// One block per (unit, token); warp j owns sub-block j.
template <int P>
__global__ void __launch_bounds__(256) panel_i8_kernel(const float *__restrict__ x, size_t cols, int n, uint8_t *__restrict__ panels) {
    // the small-M kernel launched next may start streaming its weights now; the
    // panels may still be read, and x written, by the kernel ahead
    griddep_launch();
    griddep_wait();
    const int u = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, j = tid >> 5, lane = tid & 31;
    uint8_t *blob = panels + (size_t)u * i8_unit_bytes(P * n);
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
    i8_digits<P>(v, m, t, n, j, lane, tid == 0, blob);
}

// The same with the RMS norm in front (Cpu::rmsnorm, gpu/cpu.rs:157-166): one
// block of 1024 threads per token row, four units per round; the f32 result
// goes to xout.
template <int P>
__global__ void __launch_bounds__(1024) normalize_i8_kernel(const float *x, const float *__restrict__ weight, float eps, float *xout,
                                                            size_t cols, int n, uint8_t *__restrict__ panels) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, j = warp & 7, uu = tid >> 8;
    __shared__ float part[32];
    __shared__ float wmax[32];
    const float *src = x + (size_t)t * cols;
    float ss = 0.0f;
    for (size_t k = tid; k < cols; k += 1024) ss += src[k] * src[k];
    ss = warp_sum(ss);
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    float total = part[0];
#pragma unroll
    for (int i = 1; i < 32; i++) total += part[i];
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)cols), eps)));
    const size_t units = (cols + 255) / 256;
    for (size_t u0 = 0; u0 < units; u0 += 4) {
        const size_t u = u0 + uu, k = u * 256 + (tid & 255);
        float v = 0.0f;
        if (u < units && k < cols) {
            v = __fmul_rn(src[k], __fmul_rn(scale, weight[k]));
            xout[(size_t)t * cols + k] = v;
        }
        float m = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) wmax[warp] = m;
        __syncthreads();
        m = wmax[8 * uu];
#pragma unroll
        for (int i = 1; i < 8; i++) m = fmaxf(m, wmax[8 * uu + i]);
        __syncthreads();                    // wmax is rewritten in the next round
        if (u < units) i8_digits<P>(v, m, t, n, j, lane, (tid & 255) == 0, panels + u * i8_unit_bytes(P * n));
    }
}

// weight / eps / xout: null / 0 / null for a plain conversion, or the RMS norm's
// weight [cols], its epsilon and the f32 destination [n, cols] (may be x itself).
int build_panels_i8(dwim_b200_ctx *ctx, const float *x, size_t n, size_t cols, uint8_t *panels, const float *weight, float eps,
                    float *xout) {
    if (n == 0 || cols == 0) return 0;
    if (n > I8_MAX_TOKENS) return fail(ctx, DWIM_B200_EINVAL, "int8 panels take at most %d tokens, not %zu", I8_MAX_TOKENS, n);
    const bool dependent = !ctx->weights_written;
    const int planes = i8_planes((int)n);
    if (weight) {
        auto kern = planes == 4 ? normalize_i8_kernel<4> : normalize_i8_kernel<3>;
        DWIM_CUDA(ctx, launch_dependent(dependent, kern, dim3((unsigned)n), dim3(1024), 0, ctx->stream, x, weight, eps, xout, cols, (int)n,
                                        panels));
    } else {
        auto kern = planes == 4 ? panel_i8_kernel<4> : panel_i8_kernel<3>;
        dim3 grid((unsigned)((cols + 255) / 256), (unsigned)n);
        DWIM_CUDA(ctx, launch_dependent(dependent, kern, grid, dim3(256), 0, ctx->stream, x, cols, (int)n, panels));
    }
    DWIM_LAUNCHED(ctx);
    return 0;
}

// Bytes of the GEMM's operand for n tokens (ncols = n, or 2n when an f32 activation travels as two
// columns): the f16 rows, the sub-block means, and one f32 scale per token.
size_t gemm_operand_bytes(size_t cols, size_t n, int split) {
    const size_t ncols = n * (split ? 2 : 1);
    return ncols * cols * sizeof(__half) + ncols * (cols / 256) * 16 * sizeof(__half) + ((n * sizeof(float) + 15) & ~size_t(15));
}

__device__ __forceinline__ float block_max_256(float v, float *scratch8) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();                                   // scratch8 may still be read from the reduction before
    if ((threadIdx.x & 31) == 0) scratch8[threadIdx.x >> 5] = v;
    __syncthreads();
    v = scratch8[0];
#pragma unroll
    for (int i = 1; i < 8; i++) v = fmaxf(v, scratch8[i]);
    return v;
}
__device__ __forceinline__ float block_sum_256(float v, float *scratch8) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch8[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = scratch8[0];
#pragma unroll
    for (int i = 1; i < 8; i++) s += scratch8[i];      // warp order: the same sum on every thread
    return s;
}

// One block of 256 threads per token row; the row passes through shared memory
// (cols floats of dynamic shared memory).
//   NORM: the row is first normalized by its root mean square and multiplied
//   by `weight` (Cpu::rmsnorm, gpu/cpu.rs:157-166: v * (scale * w) with
//   scale = 1 / sqrt(sum(v^2) / dim + eps)); the f32 result goes to `xout`.
// Then the row is scaled by a power of two 2^-e, chosen per token so that its
// largest magnitude lands in [4, 8): whatever the activations' range, nothing
// is clamped, an activation down to 2^-16 of the token's largest keeps its
// full f16 precision (and, for f32 inputs, the f16 remainder its share), and
// the product's epilogue multiplies the token's results by 2^e (tok_scale)
// again.  (Rows of typical normalized activations, largest magnitude 4 to 8,
// are not scaled at all.  Scaling them up instead, to just below f16's
// maximum, was measured to slow the tensor-core kernel by half: the same
// kernel on larger operand magnitudes runs into the power limit earlier.)  A thread takes
// four consecutive activations per round, eight threads a 32-wide sub-block,
// 64 a unit, the block four units.
template <bool NORM, bool ALIGNED>   // ALIGNED: x (and xout, weight) are 16-byte aligned (a wrapped caller's pointer need not be)
__global__ void __launch_bounds__(256) gemm_operand_kernel(const float *x, const float *__restrict__ weight, float eps,
                                                           float *xout, size_t cols, size_t units, int split,
                                                           __half *__restrict__ x16, __half *__restrict__ means,
                                                           float *__restrict__ tok_scale) {
    // as the small-M prologues: let the product's kernel begin (it streams weights first),
    // wait for the kernel ahead, which may still read the operand or write x
    griddep_launch();
    griddep_wait();
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch8[8];
    const int t = blockIdx.x, k = threadIdx.x;
    const float *src = x + (size_t)t * cols;
    float amax = 0.0f, ssq = 0.0f;
    for (size_t at = (size_t)k * 4; at < cols; at += 1024) {
        float4 v;
        if (ALIGNED) v = *reinterpret_cast<const float4 *>(src + at);
        else v = make_float4(src[at], src[at + 1], src[at + 2], src[at + 3]);
        *reinterpret_cast<float4 *>(row + at) = v;
        if (NORM) ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        else amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fmaxf(fabsf(v.z), fabsf(v.w)), amax));
    }
    if (NORM) {
        const float total = block_sum_256(ssq, scratch8);
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)cols), eps)));
        float *dst = xout + (size_t)t * cols;
        for (size_t at = (size_t)k * 4; at < cols; at += 1024) {
            float4 v = *reinterpret_cast<float4 *>(row + at), w;
            if (ALIGNED) w = *reinterpret_cast<const float4 *>(weight + at);
            else w = make_float4(weight[at], weight[at + 1], weight[at + 2], weight[at + 3]);
            v.x = __fmul_rn(v.x, __fmul_rn(scale, w.x));
            v.y = __fmul_rn(v.y, __fmul_rn(scale, w.y));
            v.z = __fmul_rn(v.z, __fmul_rn(scale, w.z));
            v.w = __fmul_rn(v.w, __fmul_rn(scale, w.w));
            *reinterpret_cast<float4 *>(row + at) = v;
            if (ALIGNED) *reinterpret_cast<float4 *>(dst + at) = v;
            else { dst[at] = v.x; dst[at + 1] = v.y; dst[at + 2] = v.z; dst[at + 3] = v.w; }
            amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fmaxf(fabsf(v.z), fabsf(v.w)), amax));
        }
    }
    amax = block_max_256(amax, scratch8);
    // amax in [2^(b-127), 2^(b-126)) for its biased exponent b; e = b - 127 - 2, kept where 2^e and
    // 2^-e are normal floats (a row of zeros, subnormals or infinities takes the nearest end)
    int e = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 129;
    e = amax > 0.0f ? max(-100, min(100, e)) : 0;
    const float down = __uint_as_float((uint32_t)(127 - e) << 23);
    if (k == 0) tok_scale[t] = __uint_as_float((uint32_t)(127 + e) << 23);
    const size_t col = split ? 2 * (size_t)t : (size_t)t;
    for (size_t at = (size_t)k * 4; at < cols; at += 1024) {
        const float4 v = *reinterpret_cast<float4 *>(row + at);
        const float f[4] = {v.x * down, v.y * down, v.z * down, v.w * down};
        __half hi[4], lo[4];
        float sh = 0.0f, sl = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            hi[i] = to_f16_clamped(f[i]);
            lo[i] = to_f16_clamped(f[i] - __half2float(hi[i]));
            sh += __half2float(hi[i]);
            sl += __half2float(lo[i]);
        }
        // a group of four goes out in the order (0, 2, 1, 3): the order the weights' bytes decode in
        auto pack = [](const __half (&h)[4]) {
            uint2 r;
            r.x = (uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[2]) << 16);
            r.y = (uint32_t)__half_as_ushort(h[1]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
            return r;
        };
        *reinterpret_cast<uint2 *>(x16 + col * cols + at) = pack(hi);
        if (split) *reinterpret_cast<uint2 *>(x16 + (col + 1) * cols + at) = pack(lo);
        // sub-block sums over the eight threads that share it (cols is whole units: whole warps take part)
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            sh += __shfl_xor_sync(0xffffffffu, sh, o);
            sl += __shfl_xor_sync(0xffffffffu, sl, o);
        }
        if ((k & 7) == 0) {
            const size_t u = at >> 8;
            const int j = (int)(at & 255) >> 5;
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
}

// x: the activations [n, cols]; weight / eps / xout: null / 0 / null for a plain conversion, or the
// RMS-norm's weight [cols], its epsilon and the f32 destination [n, cols] (xout may be x itself).
int build_gemm_operand(dwim_b200_ctx *ctx, const float *x, size_t n, size_t cols, int split, __half *out, const float *weight,
                       float eps, float *xout) {
    if (n == 0 || cols == 0) return 0;
    if (cols % 256) return fail(ctx, DWIM_B200_EINVAL, "GEMM operand: %zu columns are not whole 256-weight units", cols);
    const size_t units = cols / 256, ncols = n * (split ? 2 : 1);
    __half *means = out + ncols * cols;
    float *tok_scale = reinterpret_cast<float *>(means + ncols * units * 16);
    const size_t smem = cols * sizeof(float);
    if (smem > 200 * 1024) return fail(ctx, DWIM_B200_EINVAL, "GEMM operand: rows of %zu activations are too long", cols);
    const bool norm = weight != nullptr;
    const bool aligned = reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(weight) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(xout) % 16 == 0;
    auto kern = norm ? (aligned ? gemm_operand_kernel<true, true> : gemm_operand_kernel<true, false>)
                     : (aligned ? gemm_operand_kernel<false, true> : gemm_operand_kernel<false, false>);
    if (smem > 48 * 1024) DWIM_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    DWIM_CUDA(ctx, launch_dependent(!ctx->weights_written, kern, dim3((unsigned)n), dim3(256), smem, ctx->stream, x, weight, eps,
                                    xout, cols, units, split, out, means, tok_scale));
    DWIM_LAUNCHED(ctx);
    return 0;
}

}  // namespace dwim
