// The two steps in front of the quantised Linears of a layer: RMSNorm (plain and with the residual add) and the
// Embedding row gather.
//
// RMSNorm follows rusty-backend/src/kernels.wgsl:81-102 (rms_norm) and :570-597 (rms_norm_residual):
//   ss = sum_i v_i^2 / size;  inv_rms = 1 / sqrt(ss + eps);  out_i = v_i * inv_rms * weight_i,   v = x (+ residual)
// with eps = 1e-5 there.  The reference shader normalises row 0 only (`if (row >= 1u) return`) and its residual form
// treats the whole tensor as one row; here every row of x[M, K] is normalised on its own, which is what RMSNorm::forward
// (rusty-graph/src/lib.rs:148-170) is meant to compute.  The sum of squares is accumulated in f32 by a tree over the
// row's threads instead of the shader's single sequential loop: results agree to a few ulp of f32, not bit for bit.
//
// Embedding follows Embedding::forward (rusty-graph/src/lib.rs:121-135): out[t, :] = table[ids[t], :].  The reference
// copies the whole table to the host for every call and indexes a slice there (an id >= vocab panics); here the ids
// live in a device buffer, rows are gathered on the device, and an id >= vocab writes a row of zeros and raises a
// flag that the next rusty_cuda_sync reports as InvalidOperation.
#include <cstdio>

#include "internal.h"
#include "tc_common.cuh"

using namespace rusty;
using namespace rusty_tc;

namespace {

constexpr int RN_THREADS = 256;

__device__ __forceinline__ float block_sum_256(float v, float* red) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[threadIdx.x & 7];
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
    return t;
}

// One block per row; two passes over the row (the second one hits L2).  K % 4 == 0.
__global__ void __launch_bounds__(RN_THREADS) rms_norm_rows_kernel(const float* __restrict__ x, const float* __restrict__ residual,
                                                                   const float* __restrict__ weight, float* __restrict__ out,
                                                                   float* __restrict__ sum_out, int K, float eps) {
    __shared__ float red[RN_THREADS / 32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * K;
    float ss = 0.0f;
    for (int k = threadIdx.x * 4; k < K; k += RN_THREADS * 4) {
        float4 v = *reinterpret_cast<const float4*>(x + row + k);
        if (residual) {
            const float4 r = *reinterpret_cast<const float4*>(residual + row + k);
            v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
            // the sum is the layer's new residual stream; without a buffer for it, it is parked in out
            *reinterpret_cast<float4*>((sum_out ? sum_out : out) + row + k) = v;
        }
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = block_sum_256(ss, red);
    const float inv_rms = 1.0f / sqrtf(ss / (float)K + eps);
    const float* src = residual ? (sum_out ? sum_out : out) : x;   // this thread re-reads what it wrote itself
    for (int k = threadIdx.x * 4; k < K; k += RN_THREADS * 4) {
        const float4 v = *reinterpret_cast<const float4*>(src + row + k);
        const float4 w = *reinterpret_cast<const float4*>(weight + k);
        float4 o;
        o.x = v.x * inv_rms * w.x; o.y = v.y * inv_rms * w.y; o.z = v.z * inv_rms * w.z; o.w = v.w * inv_rms * w.w;
        *reinterpret_cast<float4*>(out + row + k) = o;
    }
}

// out[t, :] = table[ids[t], :], 16 bytes per thread access; dim % 4 == 0.
__global__ void __launch_bounds__(256) embedding_rows_kernel(const float* __restrict__ table, const uint32_t* __restrict__ ids,
                                                             float* __restrict__ out, size_t n_ids, uint32_t vocab, uint32_t dim,
                                                             rusty_cuda_dev_status* status) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t per_row = dim / 4, total = n_ids * per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / per_row, c = i - t * per_row;
        const uint32_t id = __ldg(ids + t);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (id < vocab) {
            v = __ldg(reinterpret_cast<const float4*>(table + (size_t)id * dim) + c);
        } else if (c == 0) {
            if (atomicExch(&status->bad_index_flag, 1u) == 0u) status->bad_index_value = id;
        }
        reinterpret_cast<float4*>(out + t * dim)[c] = v;
    }
}

}  // namespace

namespace rusty {

int launch_rms_norm(rusty_cuda_ctx* ctx, const float* x, const float* residual, const float* weight, float* out, float* sum_out,
                    uint32_t M, uint32_t K, float eps) {
    cudaError_t e = launch_pdl(rms_norm_rows_kernel, dim3(M), dim3(RN_THREADS), 0, ctx->stream, x, residual, weight, out, sum_out, (int)K, eps);
    if (e != cudaSuccess) return check_cuda(ctx, e, "rms_norm");
    return after_launch(ctx, "rms_norm");
}

}  // namespace rusty

extern "C" {

int rusty_cuda_rms_norm_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* x, const rusty_cuda_buf* residual, const rusty_cuda_buf* weight,
                            rusty_cuda_buf* out, rusty_cuda_buf* sum_out, uint32_t M, uint32_t K, float eps) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!x || !weight || !out) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "rms_norm: null argument");
    if (K == 0 || K % 4 != 0) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "rms_norm: the row length %u must be a positive multiple of 4", K);
    if (sum_out && !residual) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "rms_norm: sum_out without a residual");
    if (!(eps >= 0.0f)) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "rms_norm: eps must be >= 0");
    const size_t need_b = (size_t)M * K * 4;
    if (x->bytes < need_b || out->bytes < need_b || (residual && residual->bytes < need_b) || (sum_out && sum_out->bytes < need_b))
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "rms_norm: a buffer is smaller than [%u,%u] f32 (%zu bytes)", M, K, need_b);
    if (weight->bytes < (size_t)K * 4) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "rms_norm: weight holds %zu bytes, [%u] needs %zu", weight->bytes, K, (size_t)K * 4);
    if (out == x || out == residual || (sum_out && (sum_out == out || sum_out == x)))
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "rms_norm: out must not alias an input, sum_out must not alias x or out");
    if (M == 0) return RUSTY_CUDA_OK;
    DeviceGuard g(ctx->device);
    return launch_rms_norm(ctx, (const float*)x->ptr, residual ? (const float*)residual->ptr : nullptr, (const float*)weight->ptr, (float*)out->ptr,
                           sum_out ? (float*)sum_out->ptr : nullptr, M, K, eps);
}

int rusty_cuda_embedding_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* table, const rusty_cuda_buf* ids, rusty_cuda_buf* out, size_t n_ids,
                             uint32_t vocab, uint32_t dim) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!table || !ids || !out) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "embedding: null argument");
    if (dim == 0 || dim % 4 != 0) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "embedding: the row length %u must be a positive multiple of 4", dim);
    if (table->bytes < (size_t)vocab * dim * 4)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "embedding: table holds %zu bytes, [%u,%u] needs %zu", table->bytes, vocab, dim, (size_t)vocab * dim * 4);
    if (ids->bytes < n_ids * 4 || out->bytes < n_ids * (size_t)dim * 4)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "embedding: ids / out too small for %zu tokens of %u", n_ids, dim);
    if (n_ids == 0) return RUSTY_CUDA_OK;
    DeviceGuard g(ctx->device);
    const size_t work = n_ids * (dim / 4);
    size_t blocks = (work + 255) / 256, cap = (size_t)ctx->sm_count * 8;
    if (blocks > cap) blocks = cap;
    cudaError_t e = launch_pdl(embedding_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, ctx->stream, (const float*)table->ptr,
                               (const uint32_t*)ids->ptr, (float*)out->ptr, n_ids, vocab, dim, ctx->status_dev);
    if (e != cudaSuccess) return check_cuda(ctx, e, "embedding");
    return after_launch(ctx, "embedding");
}

}  // extern "C"
