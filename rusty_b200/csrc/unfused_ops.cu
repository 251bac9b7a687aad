// The four unfused operators of the path, one CUDA kernel each, behind the
// same entry points rusty-backend's ComputeEngine exposes:
//   matmul            (WGSL matmul_tiled,      kernels.wgsl:16-54)
//   matmul_bt         (WGSL matmul_bt,         kernels.wgsl:234-242)
//   dequantize        (WGSL dequantize,        kernels.wgsl:156-166)
//   affine_dequantize (WGSL affine_dequantize, kernels.wgsl:385-400)
//
// Numerics contract kept by these kernels:
//   * both matmuls keep ONE accumulator per output and add the products in
//     ascending k, exactly the shaders' order, using fused multiply-add; the
//     result is bit-identical to the shader arithmetic evaluated with FMA
//     contraction (which WGSL permits) and within a few ulp of the uncontracted
//     evaluation.
//   * affine_dequantize rounds the multiply and the add separately
//     (__fmul_rn / __fadd_rn), bit-identical to the uncontracted shader text.
//   * dequantize is exact integer unpacking.
#include <cuda_bf16.h>

#include "internal.h"

namespace {

// ---------------------------------------------------------------------------
// f32 matmul, register-tiled.  Block tile 64x64, 256 threads, each thread a
// 4x4 patch; k advances in steps of 16 through shared memory.  Every output's
// accumulator sees k = 0,1,2,... in order.
// B_IS_NK == false: b is [K,N] (matmul_tiled);  true: b is [N,K] (matmul_bt).
// ---------------------------------------------------------------------------
constexpr int TM = 64, TN = 64, TK = 16;

template <bool B_IS_NK>
__global__ void __launch_bounds__(256) matmul_f32_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                         float* __restrict__ out, uint32_t M, uint32_t K, uint32_t N) {
    __shared__ float sa[TK][TM + 4];  // sa[k][m]
    __shared__ float sb[TK][TN + 4];  // sb[k][n]
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;  // 16x16 threads, 4x4 outputs each
    const uint32_t m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (uint32_t k0 = 0; k0 < K; k0 += TK) {
        // a tile: 64 rows x 16 k, a is [M,K] row-major: consecutive threads walk k.
#pragma unroll
        for (int i = tid; i < TM * TK; i += 256) {
            int m = i / TK, k = i % TK;
            uint32_t gm = m0 + m, gk = k0 + k;
            sa[k][m] = (gm < M && gk < K) ? a[(size_t)gm * K + gk] : 0.0f;
        }
        if (B_IS_NK) {
#pragma unroll
            for (int i = tid; i < TN * TK; i += 256) {
                int n = i / TK, k = i % TK;
                uint32_t gn = n0 + n, gk = k0 + k;
                sb[k][n] = (gn < N && gk < K) ? b[(size_t)gn * K + gk] : 0.0f;
            }
        } else {
#pragma unroll
            for (int i = tid; i < TN * TK; i += 256) {
                int k = i / TN, n = i % TN;
                uint32_t gn = n0 + n, gk = k0 + k;
                sb[k][n] = (gn < N && gk < K) ? b[(size_t)gk * N + gn] : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sa[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = sb[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t gn = n0 + tx * 4 + j;
            if (gn < N) out[(size_t)gm * N + gn] = acc[i][j];
        }
    }
}

// ---------------------------------------------------------------------------
// dequantize: word i -> four unsigned bytes, least significant first, as f32.
// `limit_words` = min(dispatched threads, words in the input buffer).
// One thread per word; four guarded stores, as the shader does.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) dequantize_u8_kernel(const uint32_t* __restrict__ in, size_t limit_words,
                                                            float* __restrict__ out, size_t n_out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < limit_words; i += stride) {
        uint32_t p = in[i];
        size_t base = i * 4;
        if (base + 3 < n_out) {
            float4 v = make_float4((float)(p & 0xFFu), (float)((p >> 8) & 0xFFu), (float)((p >> 16) & 0xFFu),
                                   (float)((p >> 24) & 0xFFu));
            *reinterpret_cast<float4*>(out + base) = v;
        } else {
            if (base < n_out) out[base] = (float)(p & 0xFFu);
            if (base + 1 < n_out) out[base + 1] = (float)((p >> 8) & 0xFFu);
            if (base + 2 < n_out) out[base + 2] = (float)((p >> 16) & 0xFFu);
        }
    }
}

// ---------------------------------------------------------------------------
// affine_dequantize: out[i] = f32(u8[i]) * scales[i/64] + biases[i/64].
// One thread per 16 consecutive elements (one 128-bit load, four 128-bit
// stores); 16 divides 64 so a thread's elements share one group.  The scalar
// tail covers n not a multiple of 16.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) affine_dequantize_g64_kernel(const uint8_t* __restrict__ w,
                                                                    const float* __restrict__ scales,
                                                                    const float* __restrict__ biases,
                                                                    float* __restrict__ out, size_t n) {
    size_t nvec = n / 16;
    size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t v = t; v < nvec; v += stride) {
        uint4 p = reinterpret_cast<const uint4*>(w)[v];
        size_t g = v / 4;
        float s = scales[g], b = biases[g];
        uint32_t words[4] = {p.x, p.y, p.z, p.w};
        float4* o = reinterpret_cast<float4*>(out + v * 16);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t x = words[q];
            float4 r;
            r.x = __fadd_rn(__fmul_rn((float)(x & 0xFFu), s), b);
            r.y = __fadd_rn(__fmul_rn((float)((x >> 8) & 0xFFu), s), b);
            r.z = __fadd_rn(__fmul_rn((float)((x >> 16) & 0xFFu), s), b);
            r.w = __fadd_rn(__fmul_rn((float)((x >> 24) & 0xFFu), s), b);
            o[q] = r;
        }
    }
    for (size_t i = nvec * 16 + t; i < n; i += stride) {
        size_t g = i / 64;
        out[i] = __fadd_rn(__fmul_rn((float)w[i], scales[g]), biases[g]);
    }
}

__global__ void __launch_bounds__(256) add_f32_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                      float* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = __fadd_rn(a[i], b[i]);
}

// out[n][k] = in[k][n] for a [K, N] matrix of bytes or of f32: 32 x 32 tiles through shared memory (padded against bank
// conflicts).
template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T* __restrict__ in, T* __restrict__ out, uint32_t K, uint32_t N) {
    __shared__ T tile[32][33];
    const uint32_t n0 = blockIdx.x * 32u, k0 = blockIdx.y * 32u;
    const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;   // 32 x 8 threads
    for (uint32_t r = ty; r < 32u; r += 8u) {
        const uint32_t k = k0 + r, n = n0 + tx;
        tile[r][tx] = (k < K && n < N) ? in[(size_t)k * N + n] : T(0);
    }
    __syncthreads();
    for (uint32_t r = ty; r < 32u; r += 8u) {
        const uint32_t n = n0 + r, k = k0 + tx;
        if (n < N && k < K) out[(size_t)n * K + k] = tile[tx][r];
    }
}

// out = a + b with a and out of the output type of a Linear (f32 or bf16): the residual add behind a Linear whose
// kernel has no epilogue for it.
template <typename YT>
__global__ void __launch_bounds__(256) residual_add_kernel(const YT* __restrict__ a, const YT* b, YT* out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        if constexpr (sizeof(YT) == 4) out[i] = __fadd_rn(a[i], b[i]);
        else out[i] = __float2bfloat16_rn(__bfloat162float(a[i]) + __bfloat162float(b[i]));
    }
}

// WGSL `silu` (kernels.wgsl:104-113) and `mul` (kernels.wgsl:146-151), one element per thread as there.
__global__ void __launch_bounds__(256) silu_f32_kernel(const float* __restrict__ x, float* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        const float v = x[i];
        out[i] = __fmul_rn(v, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v))));
    }
}
__global__ void __launch_bounds__(256) mul_f32_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                      float* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = __fmul_rn(a[i], b[i]);
}

}  // namespace

namespace rusty {

int launch_matmul_f32(rusty_cuda_ctx* ctx, const float* a, const float* b, float* out, uint32_t M, uint32_t K,
                      uint32_t N) {
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    matmul_f32_kernel<false><<<grid, 256, 0, ctx->stream>>>(a, b, out, M, K, N);
    return after_launch(ctx, "matmul_f32");
}

int launch_matmul_bt_f32(rusty_cuda_ctx* ctx, const float* a, const float* b, float* out, uint32_t M, uint32_t K,
                         uint32_t N) {
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    matmul_f32_kernel<true><<<grid, 256, 0, ctx->stream>>>(a, b, out, M, K, N);
    return after_launch(ctx, "matmul_bt_f32");
}

int launch_dequantize_u8(rusty_cuda_ctx* ctx, const uint32_t* in, size_t in_words, size_t n_in, float* out,
                         size_t n_out) {
    size_t u32_elements = (n_in + 3) / 4;
    size_t threads = ((u32_elements + 63) / 64) * 64;  // the reference dispatches whole workgroups of 64
    size_t limit = threads < in_words ? threads : in_words;
    if (limit == 0) return RUSTY_CUDA_OK;
    size_t blocks = (limit + 255) / 256;
    size_t cap = (size_t)ctx->sm_count * 32;
    if (blocks > cap) blocks = cap;
    dequantize_u8_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(in, limit, out, n_out);
    return after_launch(ctx, "dequantize_u8");
}

int launch_affine_dequantize_g64(rusty_cuda_ctx* ctx, const uint8_t* w, const float* scales, const float* biases,
                                 float* out, size_t n) {
    if (n == 0) return RUSTY_CUDA_OK;
    size_t work = (n + 15) / 16;
    size_t blocks = (work + 255) / 256;
    size_t cap = (size_t)ctx->sm_count * 32;
    if (blocks > cap) blocks = cap;
    affine_dequantize_g64_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(w, scales, biases, out, n);
    return after_launch(ctx, "affine_dequantize_g64");
}

int launch_transpose_u8(rusty_cuda_ctx* ctx, const uint8_t* in, uint8_t* out, uint32_t K, uint32_t N) {
    const dim3 grid((N + 31) / 32, (K + 31) / 32);
    if (grid.y > 65535u) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "transpose: K=%u too large", K);
    transpose_kernel<uint8_t><<<grid, 256, 0, ctx->stream>>>(in, out, K, N);
    return after_launch(ctx, "transpose_u8");
}

int launch_transpose_f32(rusty_cuda_ctx* ctx, const float* in, float* out, uint32_t K, uint32_t N) {
    const dim3 grid((N + 31) / 32, (K + 31) / 32);
    if (grid.y > 65535u) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "transpose: K=%u too large", K);
    transpose_kernel<float><<<grid, 256, 0, ctx->stream>>>(in, out, K, N);
    return after_launch(ctx, "transpose_f32");
}

int launch_residual_add(rusty_cuda_ctx* ctx, const void* a, const void* b, void* out, size_t n, int y_dtype) {
    size_t blocks = (n + 255) / 256, cap = (size_t)ctx->sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (y_dtype == RUSTY_CUDA_BF16)
        residual_add_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, ctx->stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, n);
    else
        residual_add_kernel<float><<<(unsigned)blocks, 256, 0, ctx->stream>>>((const float*)a, (const float*)b, (float*)out, n);
    return after_launch(ctx, "residual_add");
}

}  // namespace rusty

using namespace rusty;

static int need(rusty_cuda_ctx* ctx, const char* op, const char* name, const rusty_cuda_buf* b, size_t bytes) {
    if (!b) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "%s: buffer '%s' is null", op, name);
    if (b->bytes < bytes)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "%s: buffer '%s' holds %zu bytes, the given dimensions need %zu",
                    op, name, b->bytes, bytes);
    return RUSTY_CUDA_OK;
}

extern "C" {

int rusty_cuda_matmul_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* a, const rusty_cuda_buf* b, rusty_cuda_buf* out,
                          uint32_t M, uint32_t K, uint32_t N) {
    RUSTY_REQUIRE_CTX(ctx);
    int rc;
    if ((rc = need(ctx, "matmul", "a", a, (size_t)M * K * 4))) return rc;
    if ((rc = need(ctx, "matmul", "b", b, (size_t)K * N * 4))) return rc;
    if ((rc = need(ctx, "matmul", "out", out, (size_t)M * N * 4))) return rc;
    if (M == 0 || N == 0) return RUSTY_CUDA_OK;
    if ((M + TM - 1) / TM > 65535) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "matmul: M=%u too large", M);
    DeviceGuard g(ctx->device);
    return launch_matmul_f32(ctx, (const float*)a->ptr, (const float*)b->ptr, (float*)out->ptr, M, K, N);
}

int rusty_cuda_matmul_bt_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* a, const rusty_cuda_buf* b,
                             rusty_cuda_buf* out, uint32_t M, uint32_t K, uint32_t N) {
    RUSTY_REQUIRE_CTX(ctx);
    int rc;
    if ((rc = need(ctx, "matmul_bt", "a", a, (size_t)M * K * 4))) return rc;
    if ((rc = need(ctx, "matmul_bt", "b", b, (size_t)N * K * 4))) return rc;
    if ((rc = need(ctx, "matmul_bt", "out", out, (size_t)M * N * 4))) return rc;
    if (M == 0 || N == 0) return RUSTY_CUDA_OK;
    if ((M + TM - 1) / TM > 65535) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "matmul_bt: M=%u too large", M);
    DeviceGuard g(ctx->device);
    return launch_matmul_bt_f32(ctx, (const float*)a->ptr, (const float*)b->ptr, (float*)out->ptr, M, K, N);
}

int rusty_cuda_add_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* a, const rusty_cuda_buf* b, rusty_cuda_buf* out,
                       size_t n) {
    RUSTY_REQUIRE_CTX(ctx);
    int rc;
    if ((rc = need(ctx, "add", "a", a, n * 4))) return rc;
    if ((rc = need(ctx, "add", "b", b, n * 4))) return rc;
    if ((rc = need(ctx, "add", "out", out, n * 4))) return rc;
    if (n == 0) return RUSTY_CUDA_OK;
    DeviceGuard g(ctx->device);
    size_t blocks = (n + 255) / 256, cap = (size_t)ctx->sm_count * 16;
    if (blocks > cap) blocks = cap;
    add_f32_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>((const float*)a->ptr, (const float*)b->ptr, (float*)out->ptr, n);
    return after_launch(ctx, "add_f32");
}

int rusty_cuda_silu_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* x, rusty_cuda_buf* out, size_t n) {
    RUSTY_REQUIRE_CTX(ctx);
    int rc;
    if ((rc = need(ctx, "silu", "x", x, n * 4))) return rc;
    if ((rc = need(ctx, "silu", "out", out, n * 4))) return rc;
    if (n == 0) return RUSTY_CUDA_OK;
    DeviceGuard g(ctx->device);
    size_t blocks = (n + 255) / 256, cap = (size_t)ctx->sm_count * 16;
    if (blocks > cap) blocks = cap;
    silu_f32_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>((const float*)x->ptr, (float*)out->ptr, n);
    return after_launch(ctx, "silu_f32");
}

int rusty_cuda_mul_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* a, const rusty_cuda_buf* b, rusty_cuda_buf* out,
                       size_t n) {
    RUSTY_REQUIRE_CTX(ctx);
    int rc;
    if ((rc = need(ctx, "mul", "a", a, n * 4))) return rc;
    if ((rc = need(ctx, "mul", "b", b, n * 4))) return rc;
    if ((rc = need(ctx, "mul", "out", out, n * 4))) return rc;
    if (n == 0) return RUSTY_CUDA_OK;
    DeviceGuard g(ctx->device);
    size_t blocks = (n + 255) / 256, cap = (size_t)ctx->sm_count * 16;
    if (blocks > cap) blocks = cap;
    mul_f32_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>((const float*)a->ptr, (const float*)b->ptr, (float*)out->ptr, n);
    return after_launch(ctx, "mul_f32");
}

int rusty_cuda_dequantize_u8(rusty_cuda_ctx* ctx, const rusty_cuda_buf* in, rusty_cuda_buf* out, size_t n_in) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!in || !out) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "dequantize: null buffer");
    DeviceGuard g(ctx->device);
    // arrayLength() of the shader's two runtime-sized arrays.
    return launch_dequantize_u8(ctx, (const uint32_t*)in->ptr, in->bytes / 4, n_in, (float*)out->ptr, out->bytes / 4);
}

int rusty_cuda_affine_dequantize_g64(rusty_cuda_ctx* ctx, const rusty_cuda_buf* weight, const rusty_cuda_buf* scales,
                                     const rusty_cuda_buf* biases, rusty_cuda_buf* out, size_t n) {
    RUSTY_REQUIRE_CTX(ctx);
    int rc;
    size_t groups = (n + 63) / 64;
    if ((rc = need(ctx, "affine_dequantize", "weight", weight, n))) return rc;
    if ((rc = need(ctx, "affine_dequantize", "scales", scales, groups * 4))) return rc;
    if ((rc = need(ctx, "affine_dequantize", "biases", biases, groups * 4))) return rc;
    if ((rc = need(ctx, "affine_dequantize", "out", out, n * 4))) return rc;
    DeviceGuard g(ctx->device);
    return launch_affine_dequantize_g64(ctx, (const uint8_t*)weight->ptr, scales ? (const float*)scales->ptr : nullptr,
                                        (const float*)biases->ptr, (float*)out->ptr, n);
}

}  // extern "C"
