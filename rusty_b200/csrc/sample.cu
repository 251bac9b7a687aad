// The step after the LM head: greedy token choice on the device.
//
// The reference reads the logits back and takes the arg-max on the host
// (rusty-loader/src/tokenizer.rs:151-158: Iterator::max_by, so the LAST of
// several equal maxima wins; an empty row gives 0), or runs the single-thread
// WGSL `top_k` (rusty-backend/src/kernels.wgsl:168-188).  Here one block per
// activation row scans the logits once; with output-feature shards every rank
// scans its own columns and the per-rank candidates (value, global index)
// travel instead of the logits: M x 8 bytes per rank rather than M x N/G x 4.
#include "internal.h"
#include "tc_common.cuh"

using namespace rusty;
using namespace rusty_tc;

namespace {

constexpr int AM_THREADS = 1024;

struct Cand {
    float v;
    unsigned int i;
};
// a beats b: larger value, or the same value at a later index (max_by keeps the last maximum)
__device__ __forceinline__ bool beats(const Cand& a, const Cand& b, bool b_valid) {
    return !b_valid || a.v > b.v || (a.v == b.v && a.i > b.i);
}

// best of row m of x[M, ld] over columns [0, n), indices reported as col0 + column; NaN never wins.
// valid == false: no candidate (empty row or all NaN).
__device__ __forceinline__ void row_argmax(const float* __restrict__ x, int n, unsigned int col0, Cand& best, bool& valid) {
    __shared__ float s_v[AM_THREADS / 32];
    __shared__ unsigned int s_i[AM_THREADS / 32];
    __shared__ int s_ok[AM_THREADS / 32];
    Cand c{0.0f, 0u};
    bool ok = false;
    for (int j = threadIdx.x; j < n; j += AM_THREADS) {
        const float v = x[j];
        if (v != v) continue;
        const Cand t{v, col0 + (unsigned int)j};
        if (beats(t, c, ok)) {
            c = t;
            ok = true;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, c.v, off);
        const unsigned int oi = __shfl_xor_sync(0xffffffffu, c.i, off);
        const int ook = __shfl_xor_sync(0xffffffffu, (int)ok, off);
        const Cand o{ov, oi};
        if (ook && beats(o, c, ok)) {
            c = o;
            ok = true;
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        s_v[warp] = c.v;
        s_i[warp] = c.i;
        s_ok[warp] = ok;
    }
    __syncthreads();
    if (warp == 0) {
        c = Cand{s_v[lane], s_i[lane]};
        ok = s_ok[lane] != 0;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, c.v, off);
            const unsigned int oi = __shfl_xor_sync(0xffffffffu, c.i, off);
            const int ook = __shfl_xor_sync(0xffffffffu, (int)ok, off);
            const Cand o{ov, oi};
            if (ook && beats(o, c, ok)) {
                c = o;
                ok = true;
            }
        }
    }
    best = c;
    valid = ok;  // meaningful in thread 0
}

// out_idx[m] = arg-max of row m (0 when the row has no candidate); out_val[m] (optional) = the maximum.
__global__ void __launch_bounds__(AM_THREADS) argmax_rows_kernel(const float* __restrict__ x, int n, size_t ld,
                                                                 unsigned int* __restrict__ out_idx, float* __restrict__ out_val) {
    pdl_launch_dependents();
    pdl_wait();
    Cand best;
    bool valid;
    row_argmax(x + (size_t)blockIdx.x * ld, n, 0u, best, valid);
    if (threadIdx.x == 0) {
        out_idx[blockIdx.x] = valid ? best.i : 0u;
        if (out_val) out_val[blockIdx.x] = valid ? best.v : __int_as_float(0xff800000);  // -inf
    }
}

// Sharded form, first half: this rank's candidate of every row goes into slot `rank` of the candidate table of EVERY
// rank's arena ([G][M] x {value bits, index + 1}; index + 1 == 0 means "no candidate"), then the CTA signals.
__global__ void __launch_bounds__(AM_THREADS) argmax_rows_push_kernel(const float* __restrict__ x, int n, size_t ld, unsigned int col0,
                                                                      uint2* __restrict__ table, int M, const PeerPush pp) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x < 32) peer_sync_block(pp, (int)blockIdx.x, 32);  // the table of the previous step has been consumed everywhere
    __syncthreads();
    for (int m = blockIdx.x; m < M; m += gridDim.x) {
        Cand best;
        bool valid;
        row_argmax(x + (size_t)m * ld, n, col0, best, valid);
        if (threadIdx.x == 0) {
            const uint2 e = make_uint2(__float_as_uint(best.v), valid ? best.i + 1u : 0u);
            uint2* slot = table + (size_t)pp.rank * M + m;
            *slot = e;
#pragma unroll
            for (int g = 0; g < PEER_MAX_RANKS; ++g)
                if (g < pp.nranks && g != pp.rank) *reinterpret_cast<uint2*>(reinterpret_cast<char*>(slot) + pp.delta[g]) = e;
        }
        __syncthreads();   // row_argmax reuses its shared scratch
    }
}

// Second half: once every rank's candidates have landed, the best of the G candidates of each row.
__global__ void __launch_bounds__(256) argmax_finish_kernel(const uint2* __restrict__ table, int M, int G, unsigned int* __restrict__ out_idx,
                                                            float* __restrict__ out_val, const PeerPush pp) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x < 32) peer_sync_block(pp, (int)blockIdx.x, 33);
    __syncthreads();
    for (int m = blockIdx.x * blockDim.x + threadIdx.x; m < M; m += gridDim.x * blockDim.x) {
        Cand c{0.0f, 0u};
        bool ok = false;
        for (int g = 0; g < G; ++g) {
            const uint2 e = __ldcg(table + (size_t)g * M + m);
            if (e.y == 0u) continue;
            const Cand t{__uint_as_float(e.x), e.y - 1u};
            if (beats(t, c, ok)) {
                c = t;
                ok = true;
            }
        }
        out_idx[m] = ok ? c.i : 0u;
        if (out_val) out_val[m] = ok ? c.v : __int_as_float(0xff800000);
    }
    // counted like a pushing kernel: the next table write of any rank waits until every rank has read this one
}

}  // namespace

namespace rusty {
// peer.cu: the exchange state of an arena, and whether [ptr, ptr + bytes) lies in its data region
const PeerPush* arena_push_state(const rusty_cuda_arena* arena);
bool arena_holds(const rusty_cuda_arena* arena, const void* ptr, size_t bytes);
rusty_cuda_ctx* arena_ctx(const rusty_cuda_arena* arena);
}  // namespace rusty

extern "C" {

int rusty_cuda_argmax_rows_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* logits, uint32_t M, uint32_t N, rusty_cuda_buf* out_idx,
                               rusty_cuda_buf* out_val) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!logits || !out_idx) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "argmax_rows: null buffer");
    if (logits->bytes < (size_t)M * N * 4 || out_idx->bytes < (size_t)M * 4 || (out_val && out_val->bytes < (size_t)M * 4))
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "argmax_rows: [%u,%u] logits need %zu bytes, indices (and values) %zu", M, N,
                    (size_t)M * N * 4, (size_t)M * 4);
    if (M == 0) return RUSTY_CUDA_OK;
    DeviceGuard g(ctx->device);
    cudaError_t e = launch_pdl(argmax_rows_kernel, dim3(M), dim3(AM_THREADS), 0, ctx->stream, (const float*)logits->ptr, (int)N, (size_t)N,
                               (unsigned int*)out_idx->ptr, out_val ? (float*)out_val->ptr : (float*)nullptr);
    if (e != cudaSuccess) return check_cuda(ctx, e, "argmax_rows");
    return after_launch(ctx, "argmax_rows");
}

int rusty_cuda_argmax_rows_sharded(rusty_cuda_ctx* ctx, rusty_cuda_arena* arena, const rusty_cuda_buf* logits_shard, uint32_t M,
                                   uint32_t Nl, rusty_cuda_buf* table, rusty_cuda_buf* out_idx, rusty_cuda_buf* out_val) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!arena || !logits_shard || !table || !out_idx) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "argmax_rows_sharded: null argument");
    if (arena_ctx(arena) != ctx) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "argmax_rows_sharded: arena of another context");
    const PeerPush* pp = arena_push_state(arena);
    if (!pp) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "argmax_rows_sharded: arena not attached");
    const int G = pp->nranks < 1 ? 1 : pp->nranks;
    if (logits_shard->bytes < (size_t)M * Nl * 4 || out_idx->bytes < (size_t)M * 4 || (out_val && out_val->bytes < (size_t)M * 4))
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "argmax_rows_sharded: buffers too small for [%u,%u]", M, Nl);
    if (table->bytes < (size_t)G * M * 8 || !arena_holds(arena, table->ptr, (size_t)G * M * 8))
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "argmax_rows_sharded: the candidate table ([%d][%u] x 8 bytes) must be a buffer of the arena", G, M);
    if (M == 0) return RUSTY_CUDA_OK;
    DeviceGuard g(ctx->device);
    const unsigned int col0 = (unsigned int)pp->rank * Nl;
    cudaError_t e = launch_pdl(argmax_rows_push_kernel, dim3(M < (uint32_t)PEER_SYNC_SLOTS ? M : (uint32_t)PEER_SYNC_SLOTS), dim3(AM_THREADS), 0, ctx->stream, (const float*)logits_shard->ptr, (int)Nl,
                               (size_t)Nl, col0, (uint2*)table->ptr, (int)M, *pp);
    if (e != cudaSuccess) return check_cuda(ctx, e, "argmax_rows_push");
    int rc = after_launch(ctx, "argmax_rows_push");
    if (rc) return rc;
    unsigned blocks = (M + 255) / 256;
    if (blocks > (unsigned)PEER_SYNC_SLOTS) blocks = PEER_SYNC_SLOTS;
    e = launch_pdl(argmax_finish_kernel, dim3(blocks), dim3(256), 0, ctx->stream, (const uint2*)table->ptr, (int)M, G,
                   (unsigned int*)out_idx->ptr, out_val ? (float*)out_val->ptr : (float*)nullptr, *pp);
    if (e != cudaSuccess) return check_cuda(ctx, e, "argmax_finish");
    return after_launch(ctx, "argmax_finish");
}

}  // extern "C"
