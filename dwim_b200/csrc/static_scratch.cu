// A matmul entry point that allocates nothing.
//
// Who needs it: callers that hold their GPU memory in an arena sized once at
// start-up (the engine fits its context to the memory that is free,
// inference/memory.rs:33-46, and then must not grow), and callers inside a
// region where cudaMalloc is not allowed or would synchronize the device.
// dwim_b200_matmul keeps the 16-bit operand form of the activations in a
// buffer it allocates on first use; here that scratch is a fixed array in the
// library's own image instead.
//
// Every GPU on which a context is opened holds the array from then until the
// process ends (STATIC_SCRATCH_BYTES per device: the module that contains it is
// loaded, and the array's address looked up, by dwim_b200_open, so that no
// call of this entry point allocates or loads anything).  All calls share it
// and it keeps the last call's contents: every byte a call reads it has
// written itself first (the prologue rewrites each panel in full), so nothing
// has to start at zero — but two calls that overlap on the GPU (two contexts,
// two streams) would race on it.  Calls on one context are ordered by its
// stream.
#include "common.cuh"

namespace {

constexpr size_t STATIC_SCRATCH_BYTES = 1u << 20;   // 1 MiB

static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

}  // namespace

namespace dwim {
// Called by dwim_b200_open with the context's device current.  In host code the
// array's name is only a handle for the runtime, not an address a kernel could
// use: the device address comes from cudaGetSymbolAddress, per device.
int static_scratch_prepare(dwim_b200_ctx *ctx) {
    void *p = nullptr;
    DWIM_CUDA(ctx, cudaGetSymbolAddress(&p, g_static_scratch));
    ctx->static_scratch = p;
    return 0;
}
}  // namespace dwim

extern "C" int dwim_b200_matmul_static(dwim_b200_ctx *ctx, float *out, const dwim_b200_weight *w, const float *x, size_t n) {
    DWIM_DEVICE(ctx);
    using namespace dwim;
    if (!ctx || !w) return DWIM_B200_EINVAL;
    const WeightView &v = w->v;
    if (n == 0 || v.rows == 0) return 0;
    if (!out || !x) return fail(ctx, DWIM_B200_EINVAL, "matmul_static: null pointer");
    if (out == x) return fail(ctx, DWIM_B200_EINVAL, "matmul_static: output aliases input");
    if (v.fmt == BF16) return fail(ctx, DWIM_B200_EFORMAT, "matmul_static: bf16 weights need no scratch: use matmul");
    if (n > (size_t)I8_MAX_TOKENS)
        return fail(ctx, DWIM_B200_EINVAL, "matmul_static: %zu tokens, at most %d", n, I8_MAX_TOKENS);
    if (!gemv_takes_i8(v, n))
        return fail(ctx, DWIM_B200_EFORMAT, "matmul_static: no small-M kernel takes format %d with %zu columns", v.fmt, v.cols);
    // the int8 digit-plane operand, as dwim_b200_matmul builds it for up to eight tokens
    const size_t need = panel_i8_bytes(v.cols, n);
    if (need > STATIC_SCRATCH_BYTES)
        return fail(ctx, DWIM_B200_EINVAL,
                    "matmul_static: %zu tokens of %zu columns need %zu bytes of scratch, the fixed array holds %zu", n,
                    v.cols, need, STATIC_SCRATCH_BYTES);
    void *scratch = ctx->static_scratch;
    int rc = build_panels_i8(ctx, x, n, v.cols, (uint8_t *)scratch);
    if (rc) return rc;
    return gemv_small_i8(ctx, v, (const uint8_t *)scratch, (int)n, 0, out_local(out, v.rows), nullptr, EPI_STORE);
}
