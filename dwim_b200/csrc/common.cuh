// Handles behind the C ABI and the helpers every translation unit shares.
#pragma once
#include <stdlib.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/dwim_b200.h"
#include "formats.cuh"

// Forms of an activation buffer's 16-bit shadow (cf. `Form`,
// gpu/cuda/mod.rs:108-126: the reference keeps an f16 copy beside the f32 one
// so that consecutive matmuls on one input convert it once).
enum ShadowKind : int {
    SHADOW_NONE = 0,
    SHADOW_GEMM,            // f16 rows, sub-block means and token scales, for the tensor-core kernels
    SHADOW_PANEL_I8         // int8 digit planes per 256-wide unit, for the small-M kernel
};

constexpr int DWIM_MAX_WORLD = 8;

struct dwim_b200_buffer {
    float *data = nullptr;
    size_t len = 0, cap = 0;
    bool owned = true;
    // A buffer shared with the other ranks of a group (dwim_b200_shared_alloc /
    // _connect, peer.cu): every rank's copy as mapped into this process
    // (sh_peer[sh_rank] == data), and behind this rank's data its flag block
    // (the barrier's epoch counter and one arrival word per source rank).
    int sh_world = 0, sh_rank = 0;
    float *sh_peer[DWIM_MAX_WORLD] = {};
    bool sh_opened[DWIM_MAX_WORLD] = {};
    size_t sh_flag_offset = 0;   // bytes from data to the flag block (the same on every rank)
    bool bf16_exact = false;     // every value is exactly a bf16 (write_bf16)
    // shadow
    void *shadow = nullptr;
    size_t shadow_cap = 0;       // bytes
    int shadow_kind = SHADOW_NONE;
    size_t shadow_cols = 0;      // K the shadow was built for
    int shadow_split = 0;        // 1: hi/lo column pairs, 0: single f16
};

struct dwim_b200_weight {
    dwim::WeightView v{};
    void *quants_alloc = nullptr;
    void *scales_alloc = nullptr;
};

struct dwim_b200_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    bool stream_owned = true;        // false: the caller's stream, adopted by dwim_b200_open_on_stream
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    uint32_t *status = nullptr;      // device word: bounded waits report here
    uint32_t *status_host = nullptr; // pinned
    uint64_t launches = 0;
    char name[256] = {0};
    char err[512] = {0};
    // the GEMM path's lazily created state
    void *gemm_state = nullptr;
    // A kernel on the stream has written weight memory since the last small-M launch
    // (an upload's repack): that launch must be an ordinary one, because a
    // programmatic dependent streams weights before it waits for the kernels ahead.
    bool weights_written = false;
    // 1: f32 activations go to the tensor-core kernels as one f16 column (dwim_b200_activation_precision)
    int act_f16 = 0;
    // the dense pair kernel's weight panel: f16 value and remainder of the dequantized rows, the rows' scales (gemm.cu)
    __half *pair_hi = nullptr, *pair_lo = nullptr;
    float *pair_scale = nullptr;
    size_t pair_cap = 0;             // f16 elements in each of the two
    // argmax's result slots: device keys, their pinned host copy (neighbours.cu), created on request
    unsigned long long *argmax_dev = nullptr, *argmax_host = nullptr;
    size_t argmax_cap = 0;
    // the peer all-reduce's mailbox and mappings (peer.cu), created on request
    void *peer_state = nullptr;
    // device address of the fixed scratch array of dwim_b200_matmul_static (static_scratch.cu)
    void *static_scratch = nullptr;
};

namespace dwim {

// Where a product's rows go: the same rows of one destination (the usual case)
// or of every rank's copy of a shared buffer (the row-sharded product writes
// its slice of the full result straight into its peers' memory).
struct OutSpec {
    float *dst[DWIM_MAX_WORLD];
    int world;        // destinations in use
    size_t pitch;     // floats between consecutive tokens in a destination
    size_t row0;      // destination row of the product's first row
    // scatter (the K-sharded product's partial sums, each row to the rank that owns it): when
    // scatter_per > 0, row r goes to dst[r / scatter_per] alone, at row (r % scatter_per) of that
    // destination's slot for this rank (row0 is then the slot's offset in floats, pitch = scatter_per)
    size_t scatter_per;
};
inline OutSpec out_local(float *out, size_t rows) {
    OutSpec o{};
    o.dst[0] = out;
    o.world = 1;
    o.pitch = rows;
    o.row0 = 0;
    o.scatter_per = 0;
    return o;
}

inline int fail(dwim_b200_ctx *ctx, int code, const char *fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof ctx->err, fmt, ap);
        va_end(ap);
    }
    return code;
}

#define DWIM_CUDA(ctx, expr)                                                                   \
    do {                                                                                       \
        cudaError_t e_ = (expr);                                                               \
        if (e_ != cudaSuccess)                                                                 \
            return dwim::fail(ctx, e_ == cudaErrorMemoryAllocation ? DWIM_B200_ENOMEM : DWIM_B200_ECUDA, \
                              "%s: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)

// Launches `kern` so that it may begin while the kernel ahead of it in the
// stream still runs (programmatic dependent launch).  Only for kernels that
// call griddep_wait() (ptx.cuh) before they touch anything an earlier kernel
// may read or write.  DWIM_B200_NO_PDL in the environment turns it off.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(bool allow, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    static const bool on = getenv("DWIM_B200_NO_PDL") == nullptr;
    const bool pdl = on && allow;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

// Every entry point works on its context's device, whatever device the calling thread had
// current: an engine drives several GPUs from one thread, or one context from several threads.
#define DWIM_DEVICE(ctx)                            \
    do {                                            \
        if (ctx) cudaSetDevice((ctx)->device);      \
    } while (0)

#define DWIM_LAUNCHED(ctx)                                                                     \
    do {                                                                                       \
        (ctx)->launches++;                                                                     \
        cudaError_t e_ = cudaGetLastError();                                                   \
        if (e_ != cudaSuccess)                                                                 \
            return dwim::fail(ctx, DWIM_B200_ECUDA, "kernel launch: %s (%s:%d)",               \
                              cudaGetErrorString(e_), __FILE__, __LINE__);                     \
    } while (0)

// codec.cu
int repack_to_device(dwim_b200_ctx *ctx, int fmt, size_t rows, size_t cols, const uint8_t *file_dev,
                     uint8_t *quants, __half *scales);
int dequantize_device(dwim_b200_ctx *ctx, const WeightView &w, float *out_dev);
int quantize_device(dwim_b200_ctx *ctx, int fmt, size_t rows, size_t cols, const float *w_dev, uint8_t *file_dev);

// prologue.cu
// int8 panels: per unit of 256 activations one blob of i8_unit_bytes(nc), nc = planes * tokens columns
// (column = 4*token + plane for one and two tokens, plane*tokens + token for three to eight):
//   [sub-block j (8)][column][32 digits]        256*nc B
//   [column][a_0..a_7 | b_0..b_7]                16*nc B   the digits' sums per sub-block, 128*a + b
//   [column] float                                4*nc B   what one unit of the plane's digit is worth
// rounded up to 16 bytes.
constexpr int I8_MAX_TOKENS = 8;
constexpr int i8_planes(int n) { return n <= 2 ? 4 : 3; }   // digit planes per token
constexpr int i8_unit_bytes(int nc) { return (276 * nc + 15) & ~15; }   // whole 16-byte steps: bulk copies, 128-bit loads
size_t panel_i8_bytes(size_t cols, size_t n);
int build_panels_i8(dwim_b200_ctx *ctx, const float *x, size_t n, size_t cols, uint8_t *panels, const float *weight = nullptr,
                    float eps = 0.0f, float *xout = nullptr);
// Tokens above which the tensor-core GEMM takes over from the small-M kernel (for the formats it takes).
constexpr size_t DWIM_SMALL_M_MAX = I8_MAX_TOKENS;
size_t gemm_operand_bytes(size_t cols, size_t n, int split);
int build_gemm_operand(dwim_b200_ctx *ctx, const float *x, size_t n, size_t cols, int split, __half *out,
                       const float *weight = nullptr, float eps = 0.0f, float *xout = nullptr);

// gemv.cu
enum Epilogue : int { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2 };
// One launch: tokens [t0, t0 + n_tokens) of a panel array holding ncols_total
// columns, the launch's first at col0.  aux is the `up` product for EPI_SWIGLU.
bool gemv_takes_i8(const WeightView &w, size_t n);
// n_tokens tokens (at most eight) whose results are tokens [t0, t0 + n_tokens) of out and aux.
int gemv_small_i8(dwim_b200_ctx *ctx, const WeightView &w, const uint8_t *panels, int n_tokens, size_t t0, const OutSpec &out,
                  const float *aux, int epilogue, const WeightView *up = nullptr);
void peer_release(dwim_b200_ctx *ctx);
void shared_release(dwim_b200_buffer *buf);
// neighbours.cu
int matmul_bf16(dwim_b200_ctx *ctx, const WeightView &w, const float *x, size_t n, const OutSpec &out, const float *aux, int epi);
// static_scratch.cu
int static_scratch_prepare(dwim_b200_ctx *ctx);

}  // namespace dwim
