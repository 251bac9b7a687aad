// Fused int8-weight GEMV for decode (few activation rows): reads each 1-byte
// weight and its scale from HBM once, dequantises in registers, accumulates in
// fp32 on the CUDA cores.
//
// Replaces, for a Linear whose weight stays quantised, the reference's
// "affine_dequantize at load (kernels.wgsl:385-400) + f32 matmul per forward
// (kernels.wgsl:16-54 / :234-242)"; the arithmetic it must agree with is
//   mode SYM_ROW   : y[m,n] = sum_k x[m,k] * (f32(q[n,k]) * scale[n])
//   mode AFFINE_G64: y[m,n] = sum_k x[m,k] * (f32(u[n,k]) * s[g] + b[g]),  g = (n*K+k)/64
//
// Layout NK ([out,in], rows contiguous along k) kernel:
//   * one warp owns R consecutive weight rows and walks the whole of K; lane l
//     takes the 16 bytes at k = 512*c + 16*l of every 512-byte chunk c with one
//     128-bit non-allocating load per row, several chunks in flight;
//   * x is staged once per block in shared memory as f32, permuted so that the
//     four float4 a lane needs per chunk are conflict-free to read;
//   * bytes -> f32 by byte-permute into the mantissa of 2^23 and one subtract
//     (exact for all 256 values), then one FMA per activation row;
//   * a warp-shuffle tree finishes each dot product; lane 0 applies the row
//     scale (SYM_ROW) and stores.
// Layout KN ([in,out], rusty's own Linear orientation) kernel: a thread owns 16
// consecutive output features and a slice of k; the block reduces the slices
// through shared memory.
#include "tc_common.cuh"

namespace {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int CHUNK = 512;  // k-elements one warp covers per step (32 lanes x 16 bytes)

__device__ __forceinline__ uint4 ld_stream_16B(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Four bytes of `w` -> four floats.  SIGNED: the bytes are int8 (two's
// complement); flipping the top bit makes them offset-binary u = q + 128, the
// permute drops u into the low mantissa byte of 2^23 (0x4B000000), and
// subtracting 2^23 + 128 leaves q exactly.  Unsigned: subtract 2^23 only.
template <bool SIGNED>
__device__ __forceinline__ void bytes4_to_f32(uint32_t w, float (&f)[4]) {
    if (SIGNED) w ^= 0x80808080u;
    const float magic = SIGNED ? 8388736.0f : 8388608.0f;
    f[0] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650)) - magic;
    f[1] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7651)) - magic;
    f[2] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7652)) - magic;
    f[3] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7653)) - magic;
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ void store_out(T* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// Position (in floats) inside the permuted x stage of element k of row m.
// Per row: nchunks chunks of 512; per chunk four planes j (which float4 of the
// lane's 16 values) of 32 lanes x 4 floats.
__device__ __forceinline__ int xs_index(int m, int nchunks, int k) {
    int c = k / CHUNK, within = k % CHUNK;
    int l = within / 16, j = (within % 16) / 4, e = within % 4;
    return (((m * nchunks + c) * 4 + j) * 32 + l) * 4 + e;
}

// ---------------------------------------------------------------------------
// NK kernel.  MB activation rows per pass, R weight rows per warp, U chunks in
// flight.  AFFINE: mode AFFINE_G64 (u8, per-64 scale+bias) else SYM_ROW.
// Dynamic shared memory: MB * nchunks*512 floats of x, then (AFFINE only)
// MB * nchunks*32 floats holding the sum of each lane's 16 x values.
// ---------------------------------------------------------------------------
template <int MB, int R, int U, bool AFFINE, typename XT, typename YT>
__global__ void __launch_bounds__(GEMV_THREADS, (MB <= 2 ? 2 : 1))
gemv_nk_kernel(const uint8_t* __restrict__ W, const float* __restrict__ scales, const float* __restrict__ biases,
               const XT* __restrict__ x, YT* __restrict__ y, int M, int N, int K, int ldy, int y_col0, int act) {
    extern __shared__ __align__(16) float smem[];
    const int nchunks = (K + CHUNK - 1) / CHUNK;
    float* xs = smem;
    float* xsum = smem + (size_t)MB * nchunks * CHUNK;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ngroups = (N + R - 1) / R;
    const int gstride = gridDim.x * GEMV_WARPS;

    // Let the next kernel in the stream start (programmatic dependent launch), and put this warp's first batch of
    // weight bytes in flight BEFORE waiting for the previous kernel: weights never depend on it, x and y may.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    auto load_batch = [&](int g, int c0, uint4 (&dst)[U][R]) {
        const int n0 = g * R;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (c0 + u) * CHUNK + lane * 16;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int n = n0 + r < N ? n0 + r : N - 1;  // clamp: a duplicate row is read, its result dropped
                dst[u][r] = (k < K && g < ngroups) ? ld_stream_16B(W + (size_t)n * K + k) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    int g = blockIdx.x * GEMV_WARPS + warp, c0 = 0;
    uint4 wnext[U][R];
    load_batch(g, c0, wnext);
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- stage x (zero-filled beyond M and beyond K) ----
    for (int i = tid; i < MB * nchunks * CHUNK; i += GEMV_THREADS) {
        int m = i / (nchunks * CHUNK), k = i % (nchunks * CHUNK);
        float v = (m < M && k < K) ? to_f32<XT>(x[(size_t)m * K + k]) : 0.0f;
        xs[xs_index(m, nchunks, k)] = v;
    }
    __syncthreads();
    if (AFFINE) {
        for (int i = tid; i < MB * nchunks * 32; i += GEMV_THREADS) {
            int l = i % 32, mc = i / 32;  // mc = m*nchunks + c
            float s = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float4 v = *reinterpret_cast<const float4*>(xs + ((size_t)(mc * 4 + j) * 32 + l) * 4);
                s += (v.x + v.y) + (v.z + v.w);
            }
            xsum[i] = s;
        }
        __syncthreads();
    }

    float acc[R][MB];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[r][m] = 0.0f;

    while (g < ngroups) {
        // take the batch that is in flight, then put the following one in flight before computing
        uint4 wv[U][R];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int r = 0; r < R; ++r) wv[u][r] = wnext[u][r];
        const int cur_g = g, cur_c0 = c0;
        c0 += U;
        if (c0 >= nchunks) {
            c0 = 0;
            g += gstride;
        }
        load_batch(g, c0, wnext);
        const int n0 = cur_g * R;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = cur_c0 + u;
            const int k = c * CHUNK + lane * 16;
            if (c >= nchunks) break;
            const bool live = k < K;
            float sc[R], bi[R];
            if (AFFINE) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    int n = n0 + r < N ? n0 + r : N - 1;
                    size_t grp = ((size_t)n * K + k) / 64;
                    sc[r] = live ? __ldg(scales + grp) : 0.0f;
                    bi[r] = live ? __ldg(biases + grp) : 0.0f;
                }
            }
            float part[R][MB];
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MB; ++m) part[r][m] = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float4 xv[MB];
#pragma unroll
                for (int m = 0; m < MB; ++m)
                    xv[m] = *reinterpret_cast<const float4*>(xs + ((size_t)((m * nchunks + c) * 4 + j) * 32 + lane) * 4);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint32_t word = j == 0 ? wv[u][r].x : j == 1 ? wv[u][r].y : j == 2 ? wv[u][r].z : wv[u][r].w;
                    float f[4];
                    bytes4_to_f32<!AFFINE>(word, f);
#pragma unroll
                    for (int m = 0; m < MB; ++m) {
                        float* a = AFFINE ? &part[r][m] : &acc[r][m];
                        *a = fmaf(xv[m].x, f[0], *a);
                        *a = fmaf(xv[m].y, f[1], *a);
                        *a = fmaf(xv[m].z, f[2], *a);
                        *a = fmaf(xv[m].w, f[3], *a);
                    }
                }
            }
            if (AFFINE) {
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    float sx = xsum[(m * nchunks + c) * 32 + lane];
#pragma unroll
                    for (int r = 0; r < R; ++r) acc[r][m] += sc[r] * part[r][m] + bi[r] * sx;
                }
            }
        }
        if (cur_c0 + U >= nchunks) {
            // ---- the rows of this group are complete: warp reduction and store ----
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    float v = acc[r][m];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                    acc[r][m] = v;
                }
            if (lane == 0 && act) {
                // the warp's two rows are one (gate, up) pair: y[m, pair] = silu(x.gate) * (x.up), as MLP::forward composes it
                static_assert(R == 2, "pairs need two rows per warp");
                if (n0 + 1 < N) {
                    const float s0 = AFFINE ? 1.0f : __ldg(scales + n0), s1 = AFFINE ? 1.0f : __ldg(scales + n0 + 1);
#pragma unroll
                    for (int m = 0; m < MB; ++m)
                        if (m < M) {
                            const float g = AFFINE ? acc[0][m] : acc[0][m] * s0, u = AFFINE ? acc[1][m] : acc[1][m] * s1;
                            store_out<YT>(y + (size_t)m * ldy + ((y_col0 + n0) >> 1), (g * (1.0f / (1.0f + expf(-g)))) * u);
                        }
                }
            } else if (lane == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    int n = n0 + r;
                    if (n >= N) continue;
                    float s = AFFINE ? 1.0f : __ldg(scales + n);
#pragma unroll
                    for (int m = 0; m < MB; ++m)
                        if (m < M) store_out<YT>(y + (size_t)m * ldy + y_col0 + n, AFFINE ? acc[r][m] : acc[r][m] * s);
                }
            }
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MB; ++m) acc[r][m] = 0.0f;
        }
    }
}

// ---------------------------------------------------------------------------
// KN kernel ([in,out] storage).  Block = 256 threads = 4 column groups of 16
// output features (one 128-bit load spans 16 features of one k) x 64 k-slices.
// Each thread walks k = slice, slice+64, ... with U loads in flight, keeping
// 16 x MB accumulators; slices are then summed through shared memory in a
// fixed order.  AFFINE groups run along n inside a k-row (N % 64 == 0).
// ---------------------------------------------------------------------------
constexpr int KN_THREADS = 256;
constexpr int KN_COLG = 4;               // column groups per block
constexpr int KN_COLS = KN_COLG * 16;    // output features per block
constexpr int KN_SLICES = 64;            // k-slices per block

template <int MB, int U, bool AFFINE, typename XT, typename YT>
__global__ void __launch_bounds__(KN_THREADS)
gemv_kn_kernel(const uint8_t* __restrict__ W, const float* __restrict__ scales, const float* __restrict__ biases,
               const XT* __restrict__ x, YT* __restrict__ y, int M, int N, int K, int ldy, int y_col0) {
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;                             // [MB][K]
    float* red = smem + (size_t)MB * K;           // [KN_SLICES][MB][KN_COLS]
    const int tid = threadIdx.x;
    const int cg = tid % KN_COLG, slice = tid / KN_COLG;
    const int n_base = blockIdx.x * KN_COLS + cg * 16;

    for (int i = tid; i < MB * K; i += KN_THREADS) {
        int m = i / K, k = i % K;
        xs[i] = m < M ? to_f32<XT>(x[(size_t)m * K + k]) : 0.0f;
    }
    __syncthreads();

    float acc[MB][16];
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[m][e] = 0.0f;

    const bool col_live = n_base < N;  // N % 16 == 0 is required, so a group is all-in or all-out
    if (col_live) {
        for (int k0 = slice; k0 < K; k0 += KN_SLICES * U) {
            uint4 wv[U];
            float sc[U], bi[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                int k = k0 + u * KN_SLICES;
                if (k < K) {
                    wv[u] = ld_stream_16B(W + (size_t)k * N + n_base);
                    if (AFFINE) {
                        size_t grp = ((size_t)k * N + n_base) / 64;
                        sc[u] = __ldg(scales + grp);
                        bi[u] = __ldg(biases + grp);
                    }
                } else {
                    wv[u] = make_uint4(0, 0, 0, 0);
                    sc[u] = bi[u] = 0.0f;
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                int k = k0 + u * KN_SLICES;
                if (k >= K) break;
                float f[16];
                {
                    float t[4];
                    bytes4_to_f32<!AFFINE>(wv[u].x, t); f[0] = t[0]; f[1] = t[1]; f[2] = t[2]; f[3] = t[3];
                    bytes4_to_f32<!AFFINE>(wv[u].y, t); f[4] = t[0]; f[5] = t[1]; f[6] = t[2]; f[7] = t[3];
                    bytes4_to_f32<!AFFINE>(wv[u].z, t); f[8] = t[0]; f[9] = t[1]; f[10] = t[2]; f[11] = t[3];
                    bytes4_to_f32<!AFFINE>(wv[u].w, t); f[12] = t[0]; f[13] = t[1]; f[14] = t[2]; f[15] = t[3];
                }
                if (AFFINE) {
#pragma unroll
                    for (int e = 0; e < 16; ++e) f[e] = fmaf(f[e], sc[u], bi[u]);
                }
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    float xv = xs[m * K + k];
#pragma unroll
                    for (int e = 0; e < 16; ++e) acc[m][e] = fmaf(xv, f[e], acc[m][e]);
                }
            }
        }
    }
    // ---- reduce the 16 k-slices ----
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int e = 0; e < 16; ++e) red[((size_t)slice * MB + m) * KN_COLS + cg * 16 + e] = acc[m][e];
    __syncthreads();
    for (int i = tid; i < MB * KN_COLS; i += KN_THREADS) {
        int m = i / KN_COLS, col = i % KN_COLS;
        int n = blockIdx.x * KN_COLS + col;
        if (n >= N || m >= M) continue;
        float s = 0.0f;
#pragma unroll
        for (int sl = 0; sl < KN_SLICES; ++sl) s += red[((size_t)sl * MB + m) * KN_COLS + col];
        if (!AFFINE) s *= __ldg(scales + n);
        store_out<YT>(y + (size_t)m * ldy + y_col0 + n, s);
    }
}

template <int MB, bool AFFINE, typename XT, typename YT>
int launch_nk(rusty_cuda_ctx* ctx, const rusty::QLinearArgs& a, const void* x, void* y, int M) {
    constexpr int R = 2, U = 4;
    const int nchunks = (a.K + CHUNK - 1) / CHUNK;
    size_t smem = (size_t)MB * nchunks * CHUNK * 4 + (AFFINE ? (size_t)MB * nchunks * 32 * 4 : 0);
    auto kern = gemv_nk_kernel<MB, R, U, AFFINE, XT, YT>;
    {
        cudaError_t e = rusty::ensure_dynamic_smem((const void*)kern, ctx->device, smem);
        if (e != cudaSuccess) return rusty::check_cuda(ctx, e, "gemv_nk: cudaFuncSetAttribute");
    }
    int ngroups = (a.N + R - 1) / R;
    int blocks = (ngroups + GEMV_WARPS - 1) / GEMV_WARPS;
    // one CTA per SM for short problems (so that the next kernel's CTA fits beside it and prefetches its weights
    // while this one drains), two when every warp has several row groups to stream
    int per_sm = (smem <= 100 * 1024 && MB <= 2 && ngroups >= 4 * ctx->sm_count * GEMV_WARPS) ? 2 : 1;
    int max_blocks = ctx->sm_count * per_sm;
    if (blocks > max_blocks) blocks = max_blocks;
    cudaError_t le = rusty_tc::launch_pdl(kern, dim3(blocks), dim3(GEMV_THREADS), smem, ctx->stream, a.w, a.scales, a.biases,
                                          (const XT*)x, (YT*)y, M, (int)a.N, (int)a.K, (int)a.ldy, (int)a.y_col0, a.act);
    if (le != cudaSuccess) return rusty::check_cuda(ctx, le, "gemv_nk");
    return rusty::after_launch(ctx, "gemv_nk");
}

template <int MB, bool AFFINE, typename XT, typename YT>
int launch_kn(rusty_cuda_ctx* ctx, const rusty::QLinearArgs& a, const void* x, void* y, int M) {
    constexpr int U = 4;
    size_t smem = (size_t)MB * a.K * 4 + (size_t)KN_SLICES * MB * KN_COLS * 4;
    auto kern = gemv_kn_kernel<MB, U, AFFINE, XT, YT>;
    {
        cudaError_t e = rusty::ensure_dynamic_smem((const void*)kern, ctx->device, smem);
        if (e != cudaSuccess) return rusty::check_cuda(ctx, e, "gemv_kn: cudaFuncSetAttribute");
    }
    int blocks = (a.N + KN_COLS - 1) / KN_COLS;
    kern<<<blocks, KN_THREADS, smem, ctx->stream>>>(a.w, a.scales, a.biases, (const XT*)x, (YT*)y, M, (int)a.N, (int)a.K,
                                                    (int)a.ldy, (int)a.y_col0);
    return rusty::after_launch(ctx, "gemv_kn");
}

template <int MB, typename XT, typename YT>
int launch_mb(rusty_cuda_ctx* ctx, const rusty::QLinearArgs& a, const void* x, void* y, int M) {
    const bool affine = a.qmode == RUSTY_CUDA_QMODE_AFFINE_G64;
    if (a.layout == RUSTY_CUDA_LAYOUT_NK)
        return affine ? launch_nk<MB, true, XT, YT>(ctx, a, x, y, M) : launch_nk<MB, false, XT, YT>(ctx, a, x, y, M);
    if constexpr (MB <= 2)
        return affine ? launch_kn<MB, true, XT, YT>(ctx, a, x, y, M) : launch_kn<MB, false, XT, YT>(ctx, a, x, y, M);
    else
        return rusty::fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "gemv: [in,out] weights take at most two rows per pass");
}

template <typename XT, typename YT>
int launch_typed(rusty_cuda_ctx* ctx, const rusty::QLinearArgs& a) {
    // Largest row block whose x stage fits shared memory; rows beyond it take
    // further passes (the weight is then re-read, from L2 when it fits there).
    const size_t budget = ctx->smem_optin > 8192 ? ctx->smem_optin - 8192 : 0;
    auto stage_bytes = [&](int mb) -> size_t {
        if (a.layout == RUSTY_CUDA_LAYOUT_NK) {
            size_t nch = (a.K + CHUNK - 1) / CHUNK;
            return (size_t)mb * nch * CHUNK * 4 + (size_t)mb * nch * 32 * 4;
        }
        return (size_t)mb * a.K * 4 + (size_t)KN_SLICES * mb * KN_COLS * 4;
    };
    // [out,in]: up to eight activation rows share one pass over the weights (the reference's affine layout has no
    // tensor-core kernel for f32 activations, so decode batches are passes of this kernel: 32 rows = 4 passes)
    int mb_max = a.layout == RUSTY_CUDA_LAYOUT_NK ? 8 : 2;
    while (mb_max > 1 && stage_bytes(mb_max) > budget) mb_max >>= 1;
    if (stage_bytes(mb_max) > budget)
        return rusty::fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "gemv: K=%u does not fit the shared-memory stage", a.K);
    uint32_t m0 = 0;
    while (m0 < a.M) {
        int rows = (int)(a.M - m0);
        int mb = rows >= 8 && mb_max >= 8 ? 8 : rows >= 4 && mb_max >= 4 ? 4 : rows >= 2 && mb_max >= 2 ? 2 : 1;
        if (rows > mb) rows = mb;
        const void* xp = (const char*)a.x + (size_t)m0 * a.K * sizeof(XT);
        void* yp = (char*)a.y + (size_t)m0 * a.ldy * sizeof(YT);
        int rc = mb == 8   ? launch_mb<8, XT, YT>(ctx, a, xp, yp, rows)
                 : mb == 4 ? launch_mb<4, XT, YT>(ctx, a, xp, yp, rows)
                 : mb == 2 ? launch_mb<2, XT, YT>(ctx, a, xp, yp, rows)
                           : launch_mb<1, XT, YT>(ctx, a, xp, yp, rows);
        if (rc) return rc;
        m0 += rows;
    }
    return RUSTY_CUDA_OK;
}

}  // namespace

namespace rusty {

bool gemv_supported(const rusty_cuda_ctx*, const QLinearArgs& a) {
    if (a.qmode == QMODE_AFFINE_GC) return false;   // that re-layout exists for gemv_mma only
    if (a.layout == RUSTY_CUDA_LAYOUT_NK) return a.K % 16 == 0;
    if (a.act) return false;  // pairs are rows of an [out,in] matrix
    return a.N % 16 == 0;
}

int launch_gemv(rusty_cuda_ctx* ctx, const QLinearArgs& a) {
    const bool xb = a.x_dtype == RUSTY_CUDA_BF16, yb = a.y_dtype == RUSTY_CUDA_BF16;
    if (xb) return yb ? launch_typed<__nv_bfloat16, __nv_bfloat16>(ctx, a) : launch_typed<__nv_bfloat16, float>(ctx, a);
    return yb ? launch_typed<float, __nv_bfloat16>(ctx, a) : launch_typed<float, float>(ctx, a);
}

}  // namespace rusty
