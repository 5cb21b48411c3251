// A small all-reduce over peer memory, for the partial sums of tensor-parallel
// decode (one or a few tokens: kilobytes, where a library collective's latency
// exceeds the product it follows).
//
// Every rank (one process per GPU) owns a mailbox in its own memory: two sets
// (alternating by call) of `world` slots of `cap` floats, and for every set,
// source rank and chunk one 32-bit flag.  The mailboxes are mapped into every
// peer with CUDA IPC.  A call with epoch e, on rank r, is one kernel whose
// CTA c owns chunk c of the vector:
//   1. it stores its chunk of the local vector into slot r of every rank's
//      mailbox (plain stores over NVLink; its own included),
//   2. makes them visible (__threadfence_system) and writes e into flag
//      (r, c) of every mailbox,
//   3. waits until flags (q, c) of its own mailbox hold e for every q (a
//      bounded spin: on time-out it records a code in the context's status
//      word and goes on, so that the kernel always ends),
//   4. adds the world slots' chunk in rank order (the same order, hence the
//      same bits, on every rank) into the local vector.
// No rank reads another's memory (plain one-to-one stores only), and a slot is reused
// only two calls later: a rank can be writing call e+1 while a slower peer
// still adds up call e, but not call e+2, which needs that peer's flag of e+1.
#include "common.cuh"
#include "ptx.cuh"

namespace {

constexpr int PEER_MAX_WORLD = 8;
constexpr int PEER_CHUNK = 1024;          // floats per CTA
constexpr int PEER_THREADS = 256;

struct PeerState {
    int world = 0, rank = 0;
    size_t cap = 0;                       // floats per slot
    size_t chunks = 0;                    // cap / PEER_CHUNK
    uint8_t *mine = nullptr;              // this rank's mailbox
    uint8_t *box[PEER_MAX_WORLD] = {};    // every rank's mailbox as mapped here (box[rank] == mine)
    bool opened[PEER_MAX_WORLD] = {};
    uint32_t epoch = 0;
};

size_t slots_bytes(const PeerState &p) { return 2 * (size_t)p.world * p.cap * sizeof(float); }
size_t flags_bytes(const PeerState &p) { return 2 * (size_t)p.world * p.chunks * sizeof(uint32_t); }

struct PeerArgs {
    float *x;
    size_t n;
    int world, rank;
    size_t cap, chunks;
    uint32_t epoch;
    uint8_t *box[PEER_MAX_WORLD];
    uint32_t *status;
};

__device__ __forceinline__ float *slot_of(uint8_t *box, const PeerArgs &a, int set, int src) {
    return reinterpret_cast<float *>(box) + ((size_t)set * a.world + src) * a.cap;
}
__device__ __forceinline__ uint32_t *flag_of(uint8_t *box, const PeerArgs &a, int set, int src, size_t chunk) {
    uint32_t *flags = reinterpret_cast<uint32_t *>(box + 2 * (size_t)a.world * a.cap * sizeof(float));
    return flags + ((size_t)set * a.world + src) * a.chunks + chunk;
}

__global__ void __launch_bounds__(PEER_THREADS) peer_allreduce_kernel(const PeerArgs a) {
    // a programmatic dependent: the vector comes from the product just ahead
    dwim::griddep_launch();
    dwim::griddep_wait();
    const size_t chunk = blockIdx.x, first = chunk * PEER_CHUNK;
    const int set = a.epoch & 1;
    // 1. this chunk of the local vector into slot `rank` of every mailbox
    for (int p = 0; p < a.world; p++) {
        float *dst = slot_of(a.box[p], a, set, a.rank) + first;
        for (size_t i = threadIdx.x; i < PEER_CHUNK && first + i < a.n; i += PEER_THREADS) dst[i] = a.x[first + i];
    }
    // 2. visible everywhere before the flags say so
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < (unsigned)a.world) {
        volatile uint32_t *f = flag_of(a.box[threadIdx.x], a, set, a.rank, chunk);
        *f = a.epoch;
    }
    // 3. every rank's chunk has arrived here (bounded wait)
    if (threadIdx.x < (unsigned)a.world) {
        volatile uint32_t *f = flag_of(a.box[a.rank], a, set, (int)threadIdx.x, chunk);
        const uint64_t start = dwim::globaltimer();
        while (*f != a.epoch) {
            if (dwim::globaltimer() - start > dwim::WAIT_LIMIT_NS) {
                atomicOr(a.status, 0x10000u);
                break;
            }
        }
    }
    __syncthreads();
    __threadfence_system();
    // 4. the sum, in rank order
    for (size_t i = threadIdx.x; i < PEER_CHUNK && first + i < a.n; i += PEER_THREADS) {
        float s = 0.0f;
        for (int q = 0; q < a.world; q++) s += reinterpret_cast<volatile float *>(slot_of(a.box[a.rank], a, set, q))[first + i];
        a.x[first + i] = s;
    }
}

PeerState *state(dwim_b200_ctx *ctx) { return static_cast<PeerState *>(ctx->peer_state); }

}  // namespace

namespace dwim {
void peer_release(dwim_b200_ctx *ctx) {
    PeerState *p = state(ctx);
    if (!p) return;
    for (int r = 0; r < p->world; r++)
        if (p->opened[r]) cudaIpcCloseMemHandle(p->box[r]);
    if (p->mine) cudaFree(p->mine);
    delete p;
    ctx->peer_state = nullptr;
}
}  // namespace dwim

extern "C" int dwim_b200_peer_create(dwim_b200_ctx *ctx, int world, int rank, size_t cap, void *handle, size_t handle_bytes) {
    using namespace dwim;
    if (!ctx || !handle) return DWIM_B200_EINVAL;
    if (world < 1 || world > PEER_MAX_WORLD || rank < 0 || rank >= world || cap == 0)
        return fail(ctx, DWIM_B200_EINVAL, "peer_create: world %d rank %d cap %zu", world, rank, cap);
    if (handle_bytes < sizeof(cudaIpcMemHandle_t))
        return fail(ctx, DWIM_B200_EINVAL, "peer_create: the handle needs %zu bytes", sizeof(cudaIpcMemHandle_t));
    if (ctx->peer_state) return fail(ctx, DWIM_B200_EINVAL, "peer_create: this context has a mailbox already");
    PeerState *p = new PeerState;
    p->world = world;
    p->rank = rank;
    p->cap = (cap + PEER_CHUNK - 1) / PEER_CHUNK * PEER_CHUNK;
    p->chunks = p->cap / PEER_CHUNK;
    const size_t bytes = slots_bytes(*p) + flags_bytes(*p);
    cudaError_t e = cudaMalloc(&p->mine, bytes);
    if (e == cudaSuccess) e = cudaMemsetAsync(p->mine, 0, bytes, ctx->stream);   // flags start below every epoch
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p->mine);
    if (e != cudaSuccess) {
        if (p->mine) cudaFree(p->mine);
        delete p;
        return fail(ctx, e == cudaErrorMemoryAllocation ? DWIM_B200_ENOMEM : DWIM_B200_ECUDA, "peer_create: %s", cudaGetErrorString(e));
    }
    memcpy(handle, &h, sizeof h);
    p->box[rank] = p->mine;
    ctx->peer_state = p;
    return 0;
}

extern "C" size_t dwim_b200_peer_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

extern "C" int dwim_b200_peer_connect(dwim_b200_ctx *ctx, const void *handles, size_t handle_bytes) {
    using namespace dwim;
    if (!ctx || !handles) return DWIM_B200_EINVAL;
    PeerState *p = state(ctx);
    if (!p) return fail(ctx, DWIM_B200_EINVAL, "peer_connect: no mailbox (peer_create first)");
    if (handle_bytes < sizeof(cudaIpcMemHandle_t)) return fail(ctx, DWIM_B200_EINVAL, "peer_connect: short handles");
    for (int r = 0; r < p->world; r++) {
        if (r == p->rank || p->opened[r]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const uint8_t *>(handles) + (size_t)r * handle_bytes, sizeof h);
        void *ptr = nullptr;
        DWIM_CUDA(ctx, cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        p->box[r] = static_cast<uint8_t *>(ptr);
        p->opened[r] = true;
    }
    return 0;
}

extern "C" int dwim_b200_peer_allreduce(dwim_b200_ctx *ctx, dwim_b200_buffer *buf, size_t n) {
    using namespace dwim;
    if (!ctx || !buf) return DWIM_B200_EINVAL;
    PeerState *p = state(ctx);
    if (!p) return fail(ctx, DWIM_B200_EINVAL, "peer_allreduce: no mailbox");
    if (n > buf->len || n > p->cap) return fail(ctx, DWIM_B200_EINVAL, "peer_allreduce: %zu floats, buffer %zu, mailbox %zu", n, buf->len, p->cap);
    for (int r = 0; r < p->world; r++)
        if (!p->box[r]) return fail(ctx, DWIM_B200_EINVAL, "peer_allreduce: rank %d is not connected", r);
    if (n == 0) return 0;
    PeerArgs a{};
    a.x = buf->data;
    a.n = n;
    a.world = p->world;
    a.rank = p->rank;
    a.cap = p->cap;
    a.chunks = p->chunks;
    a.epoch = ++p->epoch;
    for (int r = 0; r < p->world; r++) a.box[r] = p->box[r];
    a.status = ctx->status;
    const unsigned grid = (unsigned)((n + PEER_CHUNK - 1) / PEER_CHUNK);
    DWIM_CUDA(ctx, launch_dependent(!ctx->weights_written, peer_allreduce_kernel, dim3(grid), dim3(PEER_THREADS), 0, ctx->stream, a));
    DWIM_LAUNCHED(ctx);
    buf->shadow_kind = SHADOW_NONE;
    buf->bf16_exact = false;
    return 0;
}
