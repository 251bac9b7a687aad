// The step after the LM head, k > 1: the k largest logits of every row, on the device.
//
// WGSL `top_k` (rusty-backend/src/kernels.wgsl:168-188) is one thread running k rounds of "first index of the largest
// value not taken yet" (strict `>`, each round starting from max_v = -1e9 and max_idx = 0): the result is the k
// largest values in descending order, equal values in ascending index order; a value that is not > -1e9 (NaN
// included) is never taken, and a round that finds nothing reports index 0.  Same result here, computed per row by
// one block: an 8-bit radix select over order-preserving keys finds the k-th largest key in four passes over the row,
// a fifth pass collects the winners, and a bitonic sort in shared memory orders them.  With output-feature shards
// every rank selects from its own columns and only k (key, index) pairs per row and rank cross NVLink; every rank
// then merges the G x k candidates.  The reference's temperature / top-p Sampler (rusty-loader/src/tokenizer.rs:
// 149-204) needs exactly these k pairs when used with a top-k cut-off.
#include "internal.h"
#include "tc_common.cuh"

using namespace rusty;
using namespace rusty_tc;

namespace {

constexpr int TK_THREADS = 1024;
constexpr int TK_MAX_K = 1024;          // single device: one sort element per thread
constexpr int TK_MAX_MERGE = 2048;      // sharded: G * k candidates per row

// Larger float <=> larger key; 0 = "not a candidate" (NaN, or not > -1e9 as in the shader).  -0.0 counts as +0.0.
__device__ __forceinline__ uint32_t key_of(float v) {
    if (!(v > -1e9f)) return 0u;
    uint32_t b = __float_as_uint(v);
    if (v == 0.0f) b = 0u;
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float value_of(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key ^ 0x80000000u) : ~key);
}
// sort item: key in the high word, inverted index in the low word: descending order of the 64-bit item is descending
// value, then ascending index.  0 = empty.
__device__ __forceinline__ unsigned long long item_of(uint32_t key, uint32_t idx) {
    return ((unsigned long long)key << 32) | (unsigned long long)(0xffffffffu - idx);
}

// descending bitonic sort of P (power of two, <= blockDim.x * per) items in shared memory
__device__ __forceinline__ void bitonic_desc(unsigned long long* a, int P) {
    for (int size = 2; size <= P; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int t = threadIdx.x; t < P / 2; t += blockDim.x) {
                const int lo = 2 * t - (t & (stride - 1));   // index with bit `stride` clear
                const int hi = lo + stride;
                const bool desc = (lo & size) == 0;
                const unsigned long long x = a[lo], y = a[hi];
                if ((x < y) == desc) {
                    a[lo] = y;
                    a[hi] = x;
                }
            }
        }
    }
    __syncthreads();
}

// One block per row (rows b, b + grid, ...).  Writes the row's k winners, sorted, as items into `items_out`
// ([M][k], zero-padded) and, when out_idx is given, as indices / values.  table != null: the items also go into slot
// `rank` of every rank's candidate table ([G][M][k]).
__global__ void __launch_bounds__(TK_THREADS) topk_rows_kernel(const float* __restrict__ x, int n, size_t ld, unsigned int col0, int k, int M,
                                                               unsigned int* __restrict__ out_idx, float* __restrict__ out_val,
                                                               unsigned long long* __restrict__ table, const PeerPush pp) {
    __shared__ unsigned int hist[TK_THREADS / 32][256];
    __shared__ unsigned long long cand[TK_MAX_K];
    __shared__ unsigned int s_prefix, s_need, s_kk, s_eq, s_cnt, s_run;
    __shared__ unsigned int s_warp[TK_THREADS / 32];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_launch_dependents();
    pdl_wait();
    if (table) {
        if (tid < 32) peer_sync_block(pp, (int)blockIdx.x, 34);   // the table of the previous step has been merged everywhere
        __syncthreads();
    }
    for (int m = blockIdx.x; m < M; m += gridDim.x) {
        const float* row = x + (size_t)m * ld;
        if (tid == 0) {
            s_prefix = 0u;
            s_need = (unsigned)k;
            s_kk = 0u;
        }
        uint32_t mask = 0u;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = tid; i < (TK_THREADS / 32) * 256; i += TK_THREADS) (&hist[0][0])[i] = 0u;
            __syncthreads();
            const uint32_t prefix = s_prefix;
            for (int j0 = 0; j0 < n; j0 += TK_THREADS) {
                const int j = j0 + tid;
                const uint32_t key = j < n ? key_of(row[j]) : 0u;
                const bool in = key != 0u && (key & mask) == prefix;
                const uint32_t d = (key >> shift) & 255u;
                // lanes of the warp that hit the same bin add once
                const unsigned peers = __match_any_sync(0xffffffffu, in ? d : 256u + (uint32_t)lane);
                if (in && (unsigned)lane == (unsigned)(__ffs(peers) - 1)) hist[warp][d] += (unsigned)__popc(peers);
                __syncwarp();
            }
            __syncthreads();
            if (tid < 256) {
                unsigned s = 0;
#pragma unroll 8
                for (int w = 0; w < TK_THREADS / 32; ++w) s += hist[w][tid];
                hist[0][tid] = s;
            }
            __syncthreads();
            if (tid == 0) {
                if (pass == 0) {
                    unsigned total = 0;
                    for (int d = 0; d < 256; ++d) total += hist[0][d];
                    s_kk = total < (unsigned)k ? total : (unsigned)k;
                    s_need = s_kk;
                }
                unsigned need = s_need, cum = 0;
                if (need > 0) {
                    int d = 255;
                    for (; d > 0; --d) {
                        if (cum + hist[0][d] >= need) break;
                        cum += hist[0][d];
                    }
                    s_need = need - cum;                 // how many of this bin are still wanted
                    s_prefix = prefix | ((uint32_t)d << shift);
                    s_eq = hist[0][d];                   // after the last pass: elements equal to the k-th key
                }
            }
            mask |= 0xffu << shift;
            __syncthreads();
        }
        const unsigned kk = s_kk, need_eq = s_need, count_eq = s_eq;
        const uint32_t T = s_prefix;
        for (int i = tid; i < TK_MAX_K; i += TK_THREADS) cand[i] = 0ull;
        if (tid == 0) {
            s_cnt = 0u;
            s_run = 0u;
        }
        __syncthreads();
        if (kk > 0) {
            // everything above the k-th key, and the equals when all of them are wanted
            const bool all_eq = count_eq == need_eq;
            for (int j = tid; j < n; j += TK_THREADS) {
                const uint32_t key = key_of(row[j]);
                if (key > T || (all_eq && key == T)) cand[atomicAdd(&s_cnt, 1u)] = item_of(key, col0 + (uint32_t)j);
            }
            __syncthreads();
            if (!all_eq) {
                // more equals than wanted: the first need_eq of them in index order (a block-wide ordered count per
                // chunk of 1024 consecutive elements; stops once enough are found)
                for (int j0 = 0; j0 < n; j0 += TK_THREADS) {
                    const int j = j0 + tid;
                    const bool eq = j < n && key_of(row[j]) == T;
                    const unsigned bal = __ballot_sync(0xffffffffu, eq);
                    if (lane == 0) s_warp[warp] = (unsigned)__popc(bal);
                    __syncthreads();
                    unsigned before = s_run;
                    for (int w = 0; w < warp; ++w) before += s_warp[w];
                    const unsigned rank_eq = before + (unsigned)__popc(bal & ((1u << lane) - 1u));
                    if (eq && rank_eq < need_eq) cand[kk - need_eq + rank_eq] = item_of(T, col0 + (uint32_t)j);
                    __syncthreads();
                    if (tid == 0) {
                        unsigned tot = 0;
                        for (int w = 0; w < TK_THREADS / 32; ++w) tot += s_warp[w];
                        s_run += tot;
                    }
                    __syncthreads();
                    if (s_run >= need_eq) break;
                }
            }
            int P = 1;
            while (P < (int)kk) P <<= 1;
            bitonic_desc(cand, P);
        }
        __syncthreads();
        for (int i = tid; i < k; i += TK_THREADS) {
            const unsigned long long it = cand[i];
            if (out_idx) {
                out_idx[(size_t)m * k + i] = it ? 0xffffffffu - (uint32_t)(it & 0xffffffffull) : 0u;
                if (out_val) out_val[(size_t)m * k + i] = it ? value_of((uint32_t)(it >> 32)) : __int_as_float(0xff800000);
            }
            if (table) {
                unsigned long long* slot = table + ((size_t)pp.rank * M + m) * k + i;
                *slot = it;
                for (int g = 0; g < pp.nranks; ++g)
                    if (g != pp.rank) *reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(slot) + pp.delta[g]) = it;
            }
        }
        __syncthreads();
    }
}

// Sharded, second half: once every rank's candidates have landed, the best k of the G x k items of each row.
__global__ void __launch_bounds__(TK_THREADS) topk_merge_kernel(const unsigned long long* __restrict__ table, int M, int G, int k,
                                                                unsigned int* __restrict__ out_idx, float* __restrict__ out_val,
                                                                const PeerPush pp) {
    __shared__ unsigned long long items[TK_MAX_MERGE];
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x < 32) peer_sync_block(pp, (int)blockIdx.x, 35);
    __syncthreads();
    const int total = G * k;
    int P = 1;
    while (P < total) P <<= 1;
    for (int m = blockIdx.x; m < M; m += gridDim.x) {
        for (int i = threadIdx.x; i < P; i += blockDim.x) {
            unsigned long long it = 0ull;
            if (i < total) {
                const int g = i / k, j = i - g * k;
                it = __ldcg(table + ((size_t)g * M + m) * k + j);
            }
            items[i] = it;
        }
        bitonic_desc(items, P);
        for (int i = threadIdx.x; i < k; i += blockDim.x) {
            const unsigned long long it = items[i];
            out_idx[(size_t)m * k + i] = it ? 0xffffffffu - (uint32_t)(it & 0xffffffffull) : 0u;
            if (out_val) out_val[(size_t)m * k + i] = it ? value_of((uint32_t)(it >> 32)) : __int_as_float(0xff800000);
        }
        __syncthreads();
    }
    // like the arg-max table: the next table write of any rank waits until every rank has merged this one
}

// Soft-max statistics of every row at a temperature: the largest logit and sum_j exp((x_j - max) / T), what
// Sampler::sample (rusty-loader/src/tokenizer.rs:161-170) computes before it sorts.  With these two numbers and the
// row's top-k pairs the host can walk the nucleus without ever seeing the other logits.  Tree sum in f32 (the
// reference adds sequentially); NaN logits are skipped.
__global__ void __launch_bounds__(TK_THREADS) softmax_stats_rows_kernel(const float* __restrict__ x, int n, size_t ld, int M, float inv_t,
                                                                        float* __restrict__ out_max, float* __restrict__ out_sum) {
    __shared__ float red[TK_THREADS / 32];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_launch_dependents();
    pdl_wait();
    for (int m = blockIdx.x; m < M; m += gridDim.x) {
        const float* row = x + (size_t)m * ld;
        float mx = __int_as_float(0xff800000);
        for (int j = tid; j < n; j += TK_THREADS) {
            const float v = row[j];
            if (v == v) mx = fmaxf(mx, v);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        if (lane == 0) red[warp] = mx;
        __syncthreads();
        mx = red[lane];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        __syncthreads();
        float sum = 0.0f;
        for (int j = tid; j < n; j += TK_THREADS) {
            const float v = row[j];
            if (v == v) sum += expf((v - mx) * inv_t);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (lane == 0) red[warp] = sum;
        __syncthreads();
        sum = red[lane];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (tid == 0) {
            out_max[m] = mx;
            out_sum[m] = sum;
        }
        __syncthreads();
    }
}

}  // namespace

namespace rusty {
const PeerPush* arena_push_state(const rusty_cuda_arena* arena);
bool arena_holds(const rusty_cuda_arena* arena, const void* ptr, size_t bytes);
rusty_cuda_ctx* arena_ctx(const rusty_cuda_arena* arena);
}  // namespace rusty

extern "C" {

int rusty_cuda_top_k_rows_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* logits, uint32_t M, uint32_t N, uint32_t k, rusty_cuda_buf* out_idx,
                              rusty_cuda_buf* out_val) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!logits || !out_idx) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "top_k_rows: null buffer");
    if (k == 0 || k > (uint32_t)TK_MAX_K) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "top_k_rows: k=%u must lie in 1..%d", k, TK_MAX_K);
    if (N > 0x7fffffffu) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "top_k_rows: N=%u too large", N);
    if (logits->bytes < (size_t)M * N * 4 || out_idx->bytes < (size_t)M * k * 4 || (out_val && out_val->bytes < (size_t)M * k * 4))
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "top_k_rows: [%u,%u] logits need %zu bytes, [%u,%u] indices (and values) %zu", M, N,
                    (size_t)M * N * 4, M, k, (size_t)M * k * 4);
    if (M == 0) return RUSTY_CUDA_OK;
    DeviceGuard g(ctx->device);
    const unsigned blocks = M < (uint32_t)ctx->sm_count ? M : (unsigned)ctx->sm_count;
    cudaError_t e = launch_pdl(topk_rows_kernel, dim3(blocks), dim3(TK_THREADS), 0, ctx->stream, (const float*)logits->ptr, (int)N, (size_t)N, 0u,
                               (int)k, (int)M, (unsigned int*)out_idx->ptr, out_val ? (float*)out_val->ptr : (float*)nullptr,
                               (unsigned long long*)nullptr, PeerPush{});
    if (e != cudaSuccess) return check_cuda(ctx, e, "top_k_rows");
    return after_launch(ctx, "top_k_rows");
}

int rusty_cuda_softmax_stats_rows_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* logits, uint32_t M, uint32_t N, float temperature,
                                      rusty_cuda_buf* out_max, rusty_cuda_buf* out_sum) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!logits || !out_max || !out_sum) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "softmax_stats_rows: null buffer");
    if (!(temperature > 0.0f)) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "softmax_stats_rows: temperature must be > 0 (greedy choice is argmax_rows)");
    if (N > 0x7fffffffu) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "softmax_stats_rows: N=%u too large", N);
    if (logits->bytes < (size_t)M * N * 4 || out_max->bytes < (size_t)M * 4 || out_sum->bytes < (size_t)M * 4)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "softmax_stats_rows: [%u,%u] logits need %zu bytes, the outputs %zu each", M, N,
                    (size_t)M * N * 4, (size_t)M * 4);
    if (M == 0) return RUSTY_CUDA_OK;
    DeviceGuard g(ctx->device);
    const unsigned blocks = M < (uint32_t)ctx->sm_count ? M : (unsigned)ctx->sm_count;
    cudaError_t e = launch_pdl(softmax_stats_rows_kernel, dim3(blocks), dim3(TK_THREADS), 0, ctx->stream, (const float*)logits->ptr, (int)N, (size_t)N,
                               (int)M, 1.0f / temperature, (float*)out_max->ptr, (float*)out_sum->ptr);
    if (e != cudaSuccess) return check_cuda(ctx, e, "softmax_stats_rows");
    return after_launch(ctx, "softmax_stats_rows");
}

int rusty_cuda_top_k_rows_sharded(rusty_cuda_ctx* ctx, rusty_cuda_arena* arena, const rusty_cuda_buf* logits_shard, uint32_t M, uint32_t Nl,
                                  uint32_t k, rusty_cuda_buf* table, rusty_cuda_buf* out_idx, rusty_cuda_buf* out_val) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!arena || !logits_shard || !table || !out_idx) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "top_k_rows_sharded: null argument");
    if (arena_ctx(arena) != ctx) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "top_k_rows_sharded: arena of another context");
    const PeerPush* pp = arena_push_state(arena);
    if (!pp) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "top_k_rows_sharded: arena not attached");
    const int G = pp->nranks < 1 ? 1 : pp->nranks;
    if (k == 0 || (size_t)k * G > (size_t)TK_MAX_MERGE || k > (uint32_t)TK_MAX_K)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "top_k_rows_sharded: k=%u x %d ranks must lie in 1..%d", k, G, TK_MAX_MERGE);
    if ((uint64_t)Nl * (uint64_t)G > 0x7fffffffull) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "top_k_rows_sharded: N too large");
    if (logits_shard->bytes < (size_t)M * Nl * 4 || out_idx->bytes < (size_t)M * k * 4 || (out_val && out_val->bytes < (size_t)M * k * 4))
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "top_k_rows_sharded: buffers too small for [%u,%u], k=%u", M, Nl, k);
    const size_t table_b = (size_t)G * M * k * 8;
    if (table->bytes < table_b || !arena_holds(arena, table->ptr, table_b))
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "top_k_rows_sharded: the candidate table ([%d][%u][%u] x 8 bytes) must be a buffer of the arena", G, M, k);
    if (M == 0) return RUSTY_CUDA_OK;
    DeviceGuard g(ctx->device);
    const unsigned blocks = M < (uint32_t)PEER_SYNC_SLOTS ? M : (unsigned)PEER_SYNC_SLOTS;
    cudaError_t e = launch_pdl(topk_rows_kernel, dim3(blocks), dim3(TK_THREADS), 0, ctx->stream, (const float*)logits_shard->ptr, (int)Nl, (size_t)Nl,
                               (unsigned int)pp->rank * Nl, (int)k, (int)M, (unsigned int*)nullptr, (float*)nullptr,
                               (unsigned long long*)table->ptr, *pp);
    if (e != cudaSuccess) return check_cuda(ctx, e, "top_k_rows_push");
    int rc = after_launch(ctx, "top_k_rows_push");
    if (rc) return rc;
    e = launch_pdl(topk_merge_kernel, dim3(blocks), dim3(TK_THREADS), 0, ctx->stream, (const unsigned long long*)table->ptr, (int)M, G, (int)k,
                   (unsigned int*)out_idx->ptr, out_val ? (float*)out_val->ptr : (float*)nullptr, *pp);
    if (e != cudaSuccess) return check_cuda(ctx, e, "top_k_merge");
    return after_launch(ctx, "top_k_merge");
}

}  // extern "C"
