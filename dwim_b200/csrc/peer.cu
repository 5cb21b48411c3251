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

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
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
    // 2. visible everywhere before the flags say so: every thread fences its own stores, the
    //    block meets, and the threads that write the flags release what they have seen
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < (unsigned)a.world) {
        __threadfence_system();
        st_release_sys(flag_of(a.box[threadIdx.x], a, set, a.rank, chunk), a.epoch);
    }
    // 3. every rank's chunk has arrived here (bounded wait)
    if (threadIdx.x < (unsigned)a.world) {
        const uint32_t *f = flag_of(a.box[a.rank], a, set, (int)threadIdx.x, chunk);
        const uint64_t start = dwim::globaltimer();
        while (ld_acquire_sys(f) != a.epoch) {
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
    DWIM_DEVICE(ctx);
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
    DWIM_DEVICE(ctx);
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
    DWIM_DEVICE(ctx);
    using namespace dwim;
    if (!ctx || !buf) return DWIM_B200_EINVAL;
    PeerState *p = state(ctx);
    if (!p) return fail(ctx, DWIM_B200_EINVAL, "peer_allreduce: no mailbox");
    if (n > buf->len || n > p->cap) return fail(ctx, DWIM_B200_EINVAL, "peer_allreduce: %zu floats, buffer %zu, mailbox %zu", n, buf->len, p->cap);
    for (int r = 0; r < p->world; r++)
        if (!p->box[r]) return fail(ctx, DWIM_B200_EINVAL, "peer_allreduce: rank %d is not connected", r);
    if (n == 0) return 0;
    // The call's epoch is a kernel argument: a captured launch would replay one epoch for ever
    // and stop waiting for its peers.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    DWIM_CUDA(ctx, cudaStreamIsCapturing(ctx->stream, &cap));
    if (cap != cudaStreamCaptureStatusNone)
        return fail(ctx, DWIM_B200_EINVAL, "peer_allreduce: not inside a stream capture (the epoch is a launch argument)");
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

// ---- buffers shared by the ranks of a group, and their barrier ------------------------
// A row-sharded product writes its rows of the full, token-major result into
// every rank's copy of the output (dwim_b200_matmul_gather: plain stores from
// the product's epilogue, over NVLink for the peers' copies), so the exchange
// runs while the rest of the product is still being computed.  What remains
// of the all-gather is a barrier: every rank must know that all slices have
// arrived in its copy.
//
// A shared buffer is `len` floats followed (256-byte aligned) by a flag block:
//   word 0        this rank's barrier count (advanced by the barrier kernel
//                 itself, so a captured launch can be replayed)
//   words 16..23  arrival word of source rank q: the highest barrier count q
//                 has signalled here
// The barrier kernel (one block) runs after the product in stream order: it
// waits for the kernel ahead (all its stores, remote ones included, are then
// complete), fences, writes its new count into its arrival word on every rank
// with a system-scope release, and waits (bounded) until every arrival word of
// its own block has reached that count.
namespace {

constexpr size_t SH_FLAG_BYTES = 256;
constexpr int SH_ARRIVE_WORD = 16;

struct BarrierArgs {
    uint32_t *flags[DWIM_MAX_WORLD];   // every rank's flag block as mapped here
    int world, rank;
    uint32_t *status;
};

__global__ void __launch_bounds__(32) shared_barrier_kernel(const BarrierArgs a) {
    dwim::griddep_launch();
    dwim::griddep_wait();           // the product ahead has completed: its stores have left this GPU
    __shared__ uint32_t count;
    if (threadIdx.x == 0) {
        count = a.flags[a.rank][0] + 1;
        a.flags[a.rank][0] = count;
    }
    __syncwarp();
    const uint32_t c = *(volatile uint32_t *)&count;
    if (threadIdx.x < (unsigned)a.world) {
        __threadfence_system();
        st_release_sys(a.flags[threadIdx.x] + SH_ARRIVE_WORD + a.rank, c);
        const uint32_t *f = a.flags[a.rank] + SH_ARRIVE_WORD + threadIdx.x;
        const uint64_t start = dwim::globaltimer();
        // a peer may already be a barrier ahead: at least c, not exactly c
        while ((int32_t)(ld_acquire_sys(f) - c) < 0) {
            if (dwim::globaltimer() - start > dwim::WAIT_LIMIT_NS) {
                atomicOr(a.status, 0x20000u);
                break;
            }
        }
    }
    __syncwarp();
    __threadfence_system();
}

}  // namespace

namespace dwim {
void shared_release(dwim_b200_buffer *b) {
    for (int r = 0; r < b->sh_world; r++)
        if (b->sh_opened[r]) cudaIpcCloseMemHandle(b->sh_peer[r]);
    b->sh_world = 0;
}
}  // namespace dwim

extern "C" int dwim_b200_shared_alloc(dwim_b200_ctx *ctx, size_t len, dwim_b200_buffer **out, void *handle, size_t handle_bytes) {
    DWIM_DEVICE(ctx);
    using namespace dwim;
    if (!ctx || !out || !handle) return DWIM_B200_EINVAL;
    *out = nullptr;
    if (len == 0) return fail(ctx, DWIM_B200_EINVAL, "shared_alloc: empty buffer");
    if (handle_bytes < sizeof(cudaIpcMemHandle_t))
        return fail(ctx, DWIM_B200_EINVAL, "shared_alloc: the handle needs %zu bytes", sizeof(cudaIpcMemHandle_t));
    dwim_b200_buffer *b = new dwim_b200_buffer();
    b->len = b->cap = len;
    b->sh_flag_offset = (len * sizeof(float) + 255) / 256 * 256;
    const size_t bytes = b->sh_flag_offset + SH_FLAG_BYTES;
    cudaError_t e = cudaMalloc(&b->data, bytes);
    if (e == cudaSuccess) e = cudaMemsetAsync(b->data, 0, bytes, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, b->data);
    if (e != cudaSuccess) {
        if (b->data) cudaFree(b->data);
        delete b;
        cudaGetLastError();
        return fail(ctx, e == cudaErrorMemoryAllocation ? DWIM_B200_ENOMEM : DWIM_B200_ECUDA, "shared_alloc: %s", cudaGetErrorString(e));
    }
    memcpy(handle, &h, sizeof h);
    *out = b;
    return 0;
}

extern "C" int dwim_b200_shared_connect(dwim_b200_ctx *ctx, dwim_b200_buffer *buf, int world, int rank, const void *handles,
                                        size_t handle_bytes) {
    DWIM_DEVICE(ctx);
    using namespace dwim;
    if (!ctx || !buf) return DWIM_B200_EINVAL;
    if (world < 1 || world > DWIM_MAX_WORLD || rank < 0 || rank >= world)
        return fail(ctx, DWIM_B200_EINVAL, "shared_connect: world %d rank %d", world, rank);
    if (buf->sh_flag_offset == 0) return fail(ctx, DWIM_B200_EINVAL, "shared_connect: not a buffer of shared_alloc");
    if (buf->sh_world) return fail(ctx, DWIM_B200_EINVAL, "shared_connect: connected already");
    if (world > 1 && (!handles || handle_bytes < sizeof(cudaIpcMemHandle_t)))
        return fail(ctx, DWIM_B200_EINVAL, "shared_connect: short handles");
    for (int r = 0; r < world; r++) {
        if (r == rank) {
            buf->sh_peer[r] = buf->data;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const uint8_t *>(handles) + (size_t)r * handle_bytes, sizeof h);
        void *ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            buf->sh_world = r;          // what has been opened so far
            buf->sh_rank = rank;
            shared_release(buf);
            cudaGetLastError();
            return fail(ctx, DWIM_B200_ECUDA, "shared_connect: mapping rank %d's copy: %s", r, cudaGetErrorString(e));
        }
        buf->sh_peer[r] = static_cast<float *>(ptr);
        buf->sh_opened[r] = true;
    }
    buf->sh_world = world;
    buf->sh_rank = rank;
    return 0;
}

extern "C" int dwim_b200_shared_connect_local(dwim_b200_ctx *ctx, dwim_b200_buffer *buf, int world, int rank,
                                              dwim_b200_buffer *const *copies) {
    DWIM_DEVICE(ctx);
    using namespace dwim;
    if (!ctx || !buf || !copies) return DWIM_B200_EINVAL;
    if (world < 1 || world > DWIM_MAX_WORLD || rank < 0 || rank >= world)
        return fail(ctx, DWIM_B200_EINVAL, "shared_connect_local: world %d rank %d", world, rank);
    if (buf->sh_flag_offset == 0) return fail(ctx, DWIM_B200_EINVAL, "shared_connect_local: not a buffer of shared_alloc");
    if (buf->sh_world) return fail(ctx, DWIM_B200_EINVAL, "shared_connect_local: connected already");
    for (int r = 0; r < world; r++) {
        const dwim_b200_buffer *c = r == rank ? buf : copies[r];
        if (!c || c->sh_flag_offset != buf->sh_flag_offset || c->cap != buf->cap)
            return fail(ctx, DWIM_B200_EINVAL, "shared_connect_local: rank %d's copy is not a shared buffer of the same size", r);
    }
    for (int r = 0; r < world; r++) buf->sh_peer[r] = r == rank ? buf->data : copies[r]->data;   // nothing to unmap later
    buf->sh_world = world;
    buf->sh_rank = rank;
    return 0;
}

extern "C" int dwim_b200_shared_barrier(dwim_b200_ctx *ctx, dwim_b200_buffer *buf) {
    DWIM_DEVICE(ctx);
    using namespace dwim;
    if (!ctx || !buf) return DWIM_B200_EINVAL;
    if (buf->sh_world < 1) return fail(ctx, DWIM_B200_EINVAL, "shared_barrier: not a connected shared buffer");
    BarrierArgs a{};
    a.world = buf->sh_world;
    a.rank = buf->sh_rank;
    a.status = ctx->status;
    for (int r = 0; r < buf->sh_world; r++)
        a.flags[r] = reinterpret_cast<uint32_t *>(reinterpret_cast<uint8_t *>(buf->sh_peer[r]) + buf->sh_flag_offset);
    DWIM_CUDA(ctx, launch_dependent(!ctx->weights_written, shared_barrier_kernel, dim3(1), dim3(32), 0, ctx->stream, a));
    DWIM_LAUNCHED(ctx);
    return 0;
}

// ---- the K-sharded product: partial sums scattered to the rows' owners, reduced, gathered --------
// The closing product of a tensor-parallel block (the feed-forward block's down
// projection, an attention block's output projection) is split along K: every
// rank multiplies its K slice of W with its slice of the activations and holds
// a partial sum of the whole [n, rows] result.  Rows are owned by ranks in
// slices of `per` = ceil(rows / world).  dwim_b200_matmul_scatter's epilogue
// stores each partial sum straight into its row's owner: slot `rank` of the
// owner's copy of the shared `slots` buffer ([world][n][per] floats), by plain
// stores over NVLink while other tiles multiply.  After a barrier,
// dwim_b200_reduce_gather adds a rank's own rows over the slots in rank order
// (the same bits on every rank) and stores the sums into every rank's copy of
// the shared result; a second barrier closes the exchange.
namespace {

struct ReduceArgs {
    const float *slots;                 // this rank's copy: [world][n][per]
    float *out[DWIM_MAX_WORLD];         // every rank's copy of the result [n][rows]
    size_t n, rows, per, begin, mine;   // mine = rows this rank owns, from `begin`
    int world;
};

__global__ void __launch_bounds__(256) reduce_gather_kernel(const __grid_constant__ ReduceArgs a) {
    dwim::griddep_launch();
    dwim::griddep_wait();
    const size_t total = a.n * a.mine;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / a.mine, r = i - t * a.mine;
        float sum = 0.0f;
        for (int q = 0; q < a.world; q++) sum += a.slots[((size_t)q * a.n + t) * a.per + r];
        const size_t at = t * a.rows + a.begin + r;
#pragma unroll
        for (int p = 0; p < DWIM_MAX_WORLD; p++)
            if (p < a.world) a.out[p][at] = sum;
    }
}

}  // namespace

namespace dwim {
int product_into(dwim_b200_ctx *ctx, const OutSpec &out, size_t out_len, const dwim_b200_weight *w, dwim_b200_buffer *x,
                 const char *what);
}

extern "C" int dwim_b200_matmul_scatter(dwim_b200_ctx *ctx, dwim_b200_buffer *slots, const dwim_b200_weight *w, dwim_b200_buffer *x) {
    DWIM_DEVICE(ctx);
    using namespace dwim;
    if (!ctx || !slots || !w || !x) return DWIM_B200_EINVAL;
    if (slots->sh_world < 1) return fail(ctx, DWIM_B200_EINVAL, "matmul_scatter: the slots are not a connected shared buffer");
    const size_t rows = w->v.rows, cols = w->v.cols;
    if (cols == 0 || x->len % cols) return fail(ctx, DWIM_B200_EINVAL, "matmul_scatter: input of %zu floats is not rows of %zu", x->len, cols);
    const size_t n = x->len / cols, world = (size_t)slots->sh_world, per = (rows + world - 1) / world;
    if (slots->len != world * n * per)
        return fail(ctx, DWIM_B200_EINVAL, "matmul_scatter: slots of %zu floats, %zu ranks x %zu tokens x %zu rows need %zu", slots->len,
                    world, n, per, world * n * per);
    OutSpec o{};
    o.world = slots->sh_world;
    for (int r = 0; r < slots->sh_world; r++) o.dst[r] = slots->sh_peer[r];   // by owner rank
    o.pitch = per;
    o.row0 = (size_t)slots->sh_rank * n * per;                                // this rank's slot in every owner's copy
    o.scatter_per = per;
    // the product checks its output's length against tokens x pitch
    return product_into(ctx, o, n * per, w, x, "matmul_scatter");
}

extern "C" int dwim_b200_reduce_gather(dwim_b200_ctx *ctx, dwim_b200_buffer *out, const dwim_b200_buffer *slots, size_t n, size_t rows) {
    DWIM_DEVICE(ctx);
    using namespace dwim;
    if (!ctx || !out || !slots) return DWIM_B200_EINVAL;
    if (out->sh_world < 1 || slots->sh_world != out->sh_world || slots->sh_rank != out->sh_rank)
        return fail(ctx, DWIM_B200_EINVAL, "reduce_gather: out and slots are not shared buffers of one group");
    const size_t world = (size_t)out->sh_world, per = (rows + world - 1) / world;
    if (out->len != n * rows || slots->len != world * n * per)
        return fail(ctx, DWIM_B200_EINVAL, "reduce_gather: out of %zu and slots of %zu floats for [%zu, %zu] over %zu ranks", out->len,
                    slots->len, n, rows, world);
    ReduceArgs a{};
    a.slots = slots->data;
    // every rank's copy, in ring order from this rank on (the ranks' stores then head for different GPUs)
    for (int k = 0; k < out->sh_world; k++) a.out[k] = out->sh_peer[(out->sh_rank + k) % out->sh_world];
    a.n = n;
    a.rows = rows;
    a.per = per;
    a.begin = (size_t)out->sh_rank * per;
    a.mine = a.begin >= rows ? 0 : (rows - a.begin < per ? rows - a.begin : per);
    a.world = out->sh_world;
    out->shadow_kind = SHADOW_NONE;
    out->bf16_exact = false;
    if (n * a.mine == 0) return 0;
    size_t blocks = (n * a.mine + 255) / 256, cap = (size_t)ctx->sm_count * 8;
    DWIM_CUDA(ctx, launch_dependent(!ctx->weights_written, reduce_gather_kernel, dim3((unsigned)(blocks < cap ? blocks : cap)), dim3(256), 0,
                                    ctx->stream, a));
    DWIM_LAUNCHED(ctx);
    return 0;
}
