// Exchange of sharded outputs by peer stores over NVLink.
//
// The reference is single-device; this is the second multi-GPU form of
// Linear::forward (rusty-graph/src/lib.rs:69-70) next to the NCCL all-gather in
// shard.cu.  Every rank owns an "arena": one device allocation with the same
// layout on all ranks, exported with a CUDA IPC handle and mapped by the others.
// A rank computes its output columns and stores them into its own y AND into
// the same place of every other rank's y.  Where the tensor-core kernel runs,
// that happens in its epilogue (gemm_tc.cu); the other kernels are followed by
// a copy kernel.  Ranks keep step at the START of every operation: the first kernel of an operation (the digit
// pre-pass, the wait kernel) runs after everything this rank enqueued before has completed, tells the other ranks so
// with one add per rank, and waits for theirs (internal.h, peer_sync_block).  No fence stands between a
// kernel's stores and its exit: the kernel boundary orders them.
//
// All ranks must enqueue the same sequence of pushing operations on an arena.
// Waits are bounded (RUSTY_PEER_WAIT_MS, default 5000): a rank that never
// signals makes the others report RUSTY_CUDA_ERR_TIMEOUT at their next
// rusty_cuda_sync instead of hanging.  No load ever reads a peer's memory.
#include <cstdlib>
#include <cstring>
#include <new>

#include "internal.h"
#include "tc_common.cuh"

using namespace rusty;
using namespace rusty_tc;

namespace {

constexpr size_t ARENA_CTL_BYTES = 4096;  // control block in front of the data region

__global__ void peer_wait_kernel(const PeerPush pp) {
    pdl_launch_dependents();
    pdl_wait();
    peer_sync_block(pp, 0, 31);   // one warp
}

// Copies rows [0,M) x bytes [0,row_bytes) of a local slice (rows ld_bytes apart) to the same addresses of every
// other arena.  VEC = bytes per thread access.
template <int VEC>
__global__ void __launch_bounds__(256) peer_push_kernel(const uint8_t* __restrict__ src, int M, size_t row_bytes, size_t ld_bytes,
                                                        const PeerPush pp) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t per_row = row_bytes / VEC;
    const size_t total = (size_t)M * per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t m = i / per_row, v = i % per_row;
        const uint8_t* s = src + m * ld_bytes + v * VEC;
        if constexpr (VEC == 16) {
            const uint4 val = *reinterpret_cast<const uint4*>(s);
            for (int g = 0; g < pp.nranks; ++g)
                if (g != pp.rank) *reinterpret_cast<uint4*>(const_cast<uint8_t*>(s) + pp.delta[g]) = val;
        } else if constexpr (VEC == 4) {
            const uint32_t val = *reinterpret_cast<const uint32_t*>(s);
            for (int g = 0; g < pp.nranks; ++g)
                if (g != pp.rank) *reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(s) + pp.delta[g]) = val;
        } else {
            const uint16_t val = *reinterpret_cast<const uint16_t*>(s);
            for (int g = 0; g < pp.nranks; ++g)
                if (g != pp.rank) *reinterpret_cast<uint16_t*>(const_cast<uint8_t*>(s) + pp.delta[g]) = val;
        }
    }
    // no signal here: the next operation's first kernel meets the other ranks once this kernel has completed
}

}  // namespace

struct rusty_cuda_arena {
    rusty_cuda_ctx* ctx = nullptr;
    uint8_t* base = nullptr;  // control block, then the data region
    size_t data_bytes = 0;
    int nranks = 1, rank = 0;
    bool attached = false;
    void* opened[PEER_MAX_RANKS] = {};  // mappings of the other ranks' arenas (to close)
    PeerPush pp{};
};

namespace rusty {
const PeerPush* arena_push_state(const rusty_cuda_arena* arena) { return arena && arena->attached ? &arena->pp : nullptr; }
bool arena_holds(const rusty_cuda_arena* arena, const void* ptr, size_t bytes) {
    const uint8_t* lo = arena->base + ARENA_CTL_BYTES;
    const uint8_t* p = (const uint8_t*)ptr;
    return p >= lo && p <= lo + arena->data_bytes && bytes <= (size_t)(lo + arena->data_bytes - p);
}
rusty_cuda_ctx* arena_ctx(const rusty_cuda_arena* arena) { return arena ? arena->ctx : nullptr; }
}  // namespace rusty

extern "C" {

int rusty_cuda_arena_create(rusty_cuda_ctx* ctx, size_t bytes, int nranks, int rank, rusty_cuda_arena** out) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!out) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "arena_create: null out pointer");
    *out = nullptr;
    if (nranks < 1 || nranks > PEER_MAX_RANKS || rank < 0 || rank >= nranks)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "arena_create: rank %d of %d (at most %d ranks)", rank, nranks, PEER_MAX_RANKS);
    DeviceGuard g(ctx->device);
    rusty_cuda_arena* a = new (std::nothrow) rusty_cuda_arena();
    if (!a) return fail(ctx, RUSTY_CUDA_ERR_MEMORY_ALLOCATION, "arena_create: host allocation failed");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, ARENA_CTL_BYTES + bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        delete a;
        return fail(ctx, RUSTY_CUDA_ERR_MEMORY_ALLOCATION, "arena_create: cudaMalloc(%zu) failed", ARENA_CTL_BYTES + bytes);
    }
    // flags, epoch and the arrival counter start at zero; finish before any peer can map and write the block
    e = cudaMemset(p, 0, ARENA_CTL_BYTES);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(p);
        delete a;
        return check_cuda(ctx, e, "arena_create: clearing the control block");
    }
    a->ctx = ctx;
    a->base = (uint8_t*)p;
    a->data_bytes = bytes;
    a->nranks = nranks;
    a->rank = rank;
    a->pp.nranks = nranks;
    a->pp.rank = rank;
    a->pp.ctl = (unsigned int*)p;
    a->pp.peer_ctl[rank] = (unsigned int*)p;
    a->pp.delta[rank] = 0;
    a->pp.status = ctx->status_dev;
    const char* ms = getenv("RUSTY_PEER_WAIT_MS");
    long long lim = ms ? atoll(ms) : 5000;
    if (lim < 1) lim = 1;
    a->pp.wait_ns = (unsigned long long)lim * 1000000ull;
    a->attached = nranks == 1;
    *out = a;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_arena_export(const rusty_cuda_arena* arena, void* handle64) {
    if (!arena || !handle64) return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "arena_export: null argument");
    DeviceGuard g(arena->ctx->device);
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == RUSTY_CUDA_IPC_HANDLE_BYTES, "IPC handle size");
    cudaError_t e = cudaIpcGetMemHandle(&h, arena->base);
    if (e != cudaSuccess) return check_cuda(arena->ctx, e, "arena_export: cudaIpcGetMemHandle");
    memcpy(handle64, &h, sizeof(h));
    return RUSTY_CUDA_OK;
}

int rusty_cuda_arena_attach(rusty_cuda_arena* arena, const void* handles) {
    if (!arena || !handles) return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "arena_attach: null argument");
    rusty_cuda_ctx* ctx = arena->ctx;
    if (arena->attached) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "arena_attach: already attached");
    DeviceGuard g(ctx->device);
    for (int r = 0; r < arena->nranks; ++r) {
        if (r == arena->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char*)handles + (size_t)r * sizeof(h), sizeof(h));
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int q = 0; q < r; ++q)
                if (arena->opened[q]) {
                    cudaIpcCloseMemHandle(arena->opened[q]);
                    arena->opened[q] = nullptr;
                }
            return check_cuda(ctx, e, "arena_attach: cudaIpcOpenMemHandle (ranks must be separate processes on one node)");
        }
        arena->opened[r] = p;
        arena->pp.peer_ctl[r] = (unsigned int*)p;
        arena->pp.delta[r] = (long long)((intptr_t)p - (intptr_t)arena->base);
    }
    arena->attached = true;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_arena_buf(rusty_cuda_arena* arena, size_t offset, size_t bytes, rusty_cuda_buf** out) {
    if (!arena || !out) return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "arena_buf: null argument");
    *out = nullptr;
    if (offset % 256 != 0 || offset > arena->data_bytes || bytes > arena->data_bytes - offset)
        return fail(arena->ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "arena_buf: [%zu, +%zu) not inside %zu bytes (offsets are multiples of 256)",
                    offset, bytes, arena->data_bytes);
    rusty_cuda_buf* b = new (std::nothrow) rusty_cuda_buf();
    if (!b) return fail(arena->ctx, RUSTY_CUDA_ERR_MEMORY_ALLOCATION, "arena_buf: host allocation failed");
    b->ctx = arena->ctx;
    b->ptr = arena->base + ARENA_CTL_BYTES + offset;
    b->bytes = bytes;
    b->borrowed = true;
    *out = b;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_arena_wait(rusty_cuda_ctx* ctx, rusty_cuda_arena* arena) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!arena || arena->ctx != ctx) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "arena_wait: null arena or arena of another context");
    if (arena->nranks == 1) return RUSTY_CUDA_OK;
    if (!arena->attached) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "arena_wait: arena not attached");
    DeviceGuard g(ctx->device);
    cudaError_t e = launch_pdl(peer_wait_kernel, dim3(1), dim3(32), 0, ctx->stream, arena->pp);
    if (e != cudaSuccess) return check_cuda(ctx, e, "peer_wait");
    return after_launch(ctx, "peer_wait");
}

int rusty_cuda_arena_destroy(rusty_cuda_arena* arena) {
    if (!arena) return RUSTY_CUDA_OK;
    DeviceGuard g(arena->ctx->device);
    cudaStreamSynchronize(arena->ctx->stream);
    for (int r = 0; r < PEER_MAX_RANKS; ++r)
        if (arena->opened[r]) cudaIpcCloseMemHandle(arena->opened[r]);
    cudaFree(arena->base);
    delete arena;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_qlinear_forward_pushed(rusty_cuda_ctx* ctx, rusty_cuda_arena* arena, const rusty_cuda_qlinear* ql_shard,
                                      const rusty_cuda_buf* x, int x_dtype, uint32_t M, rusty_cuda_buf* y_full, int y_dtype) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!arena || !ql_shard || !x || !y_full) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_pushed: null argument");
    if (arena->ctx != ctx) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_pushed: arena of another context");
    if (!arena->attached) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_pushed: arena not attached");
    const size_t ys = y_dtype == RUSTY_CUDA_BF16 ? 2 : y_dtype == RUSTY_CUDA_F32 ? 4 : 0;
    if (!ys) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DATA_TYPE, "qlinear_forward_pushed: y must be f32 or bf16");
    const int G = arena->nranks;
    // with the pair activation a shard of Nl rows yields Nl/2 columns; col0 keeps counting rows of the whole weight
    const uint32_t Nl = ql_shard->N, col0 = Nl * (uint32_t)arena->rank;
    const uint32_t Nl_out = ql_shard->act ? Nl / 2 : Nl, N = Nl_out * (uint32_t)G, col0_out = ql_shard->act ? col0 / 2 : col0;
    const uint8_t* lo = arena->base + ARENA_CTL_BYTES;
    const uint8_t* yp = (const uint8_t*)y_full->ptr;
    if (yp < lo || yp > lo + arena->data_bytes || y_full->bytes > (size_t)(lo + arena->data_bytes - yp))
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_pushed: y is not a buffer of this arena");
    if (y_full->bytes < (size_t)M * N * ys)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_forward_pushed: y holds %zu bytes, [%u,%u] needs %zu", y_full->bytes, M, N,
                    (size_t)M * N * ys);
    if (M == 0 || Nl == 0) return RUSTY_CUDA_OK;
    static const bool unfused = getenv("RUSTY_PUSH_UNFUSED") != nullptr;  // development aid: always use the copy kernel
    if (G > 1 && !unfused && qlinear_pushes_fused(ql_shard, x_dtype, M, y_dtype)) {
        if (!qlinear_meets_in_kernel(ql_shard, x_dtype, M, y_dtype)) {   // the bf16 kernel: the meeting as a kernel in front
            DeviceGuard g(ctx->device);
            cudaError_t e = launch_pdl(peer_wait_kernel, dim3(1), dim3(32), 0, ctx->stream, arena->pp);
            if (e != cudaSuccess) return check_cuda(ctx, e, "peer_wait");
            int rc = after_launch(ctx, "peer_wait");
            if (rc) return rc;
        }
        return qlinear_forward_cols(ctx, ql_shard, x, x_dtype, M, y_full, y_dtype, N, col0, &arena->pp);
    }
    // Other kernels: wait, compute this rank's columns in place, copy them to the peers and signal.
    DeviceGuard g(ctx->device);
    if (G > 1) {
        cudaError_t e = launch_pdl(peer_wait_kernel, dim3(1), dim3(32), 0, ctx->stream, arena->pp);
        if (e != cudaSuccess) return check_cuda(ctx, e, "peer_wait");
        int rc = after_launch(ctx, "peer_wait");
        if (rc) return rc;
    }
    int rc = qlinear_forward_cols(ctx, ql_shard, x, x_dtype, M, y_full, y_dtype, N, col0, nullptr);
    if (rc || G == 1) return rc;
    const uint8_t* slice = yp + (size_t)col0_out * ys;
    const size_t row_bytes = (size_t)Nl_out * ys, ld_bytes = (size_t)N * ys;
    const int vec = (row_bytes % 16 == 0 && ld_bytes % 16 == 0 && ((uintptr_t)slice & 15) == 0) ? 16 : (int)(ys == 4 ? 4 : 2);
    const size_t work = (size_t)M * (row_bytes / vec);
    size_t blocks = (work + 255) / 256, cap = (size_t)ctx->sm_count * 4;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    cudaError_t e;
    if (vec == 16)
        e = launch_pdl(peer_push_kernel<16>, dim3((unsigned)blocks), dim3(256), 0, ctx->stream, slice, (int)M, row_bytes, ld_bytes, arena->pp);
    else if (vec == 4)
        e = launch_pdl(peer_push_kernel<4>, dim3((unsigned)blocks), dim3(256), 0, ctx->stream, slice, (int)M, row_bytes, ld_bytes, arena->pp);
    else
        e = launch_pdl(peer_push_kernel<2>, dim3((unsigned)blocks), dim3(256), 0, ctx->stream, slice, (int)M, row_bytes, ld_bytes, arena->pp);
    if (e != cudaSuccess) return check_cuda(ctx, e, "peer_push");
    return after_launch(ctx, "peer_push");
}

int rusty_cuda_qlinear_forward_pushed_batch(rusty_cuda_ctx* ctx, rusty_cuda_arena* arena, size_t n,
                                            const rusty_cuda_qlinear* const* ql_shards, const rusty_cuda_buf* const* xs, int x_dtype,
                                            uint32_t M, rusty_cuda_buf* const* ys, int y_dtype) {
    RUSTY_REQUIRE_CTX(ctx);
    if (n && (!ql_shards || !xs || !ys)) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_pushed_batch: null array");
    for (size_t i = 0; i < n; ++i) {
        int rc = rusty_cuda_qlinear_forward_pushed(ctx, arena, ql_shards[i], xs[i], x_dtype, M, ys[i], y_dtype);
        if (rc) return rc;
    }
    return RUSTY_CUDA_OK;
}

}  // extern "C"
