// Fused int8-weight GEMV for one or two activation rows, weights staged by TMA.
//
// Same arithmetic as gemv.cu (mode SYM_ROW, [out,in] storage):
//     y[m,n] = scale[n] * sum_k x[m,k] * f32(q[n,k])
// standing in for the reference's dequantise-at-load + f32 matmul per forward
// (rusty-loader/src/lib.rs:155-218, rusty-backend/src/kernels.wgsl:234-242).
//
// A decode-sized weight matrix is only a few microseconds of HBM traffic, so
// what matters is how many bytes are in flight and how early they start:
//   * whole weight rows are contiguous, so a tile of consecutive rows (~16 KB)
//     is ONE bulk copy (cp.async.bulk, no tensor map) into a ring of shared-
//     memory stages; one thread keeps the ring full — ~100 KB in flight per CTA
//     without spending a register on it;
//   * the copies start before griddepcontrol.wait: weights never depend on the
//     previous kernel, so with two CTAs per SM (one per kernel) this kernel's
//     weights land while the previous kernel is still finishing; only x (read
//     after the wait, kept in registers for the whole kernel) and y depend on it;
//   * eight compute warps split K: lane l of warp w owns the 16-byte chunks
//     w*32 + l (+256 j) of every row; bytes -> f32 by byte-permute + subtract;
//     one 6-shuffle butterfly folds the four row sums of a stage; a reducer warp
//     adds the eight warp partials in a fixed order, applies the row scale and
//     stores y — no block-wide barrier anywhere in the loop.
// Every mbarrier wait is bounded.
#include <cstdlib>

#include "tc_common.cuh"

using namespace rusty_tc;

namespace {

constexpr int CW = 8;                    // compute warps
constexpr int TG_THREADS = 32 * (CW + 2);  // + reducer warp + producer warp
constexpr int CHUNKS_PER_PASS = CW * 32; // 16-byte chunks the compute warps cover side by side (4096 k)
constexpr int MAXJ = 4;                  // K <= 16384

struct TgParams {
    const uint8_t* W;
    const float* scales;
    const void* x;
    void* y;
    int M, N, K;
    int rows_per_stage;   // 1, 2 or 4
    int stages;
    int tiles;
    int ldy, y_col0;
    int act;  // RUSTY_CUDA_ACT_SWIGLU_PAIRS: rows 2j, 2j+1 -> column (y_col0 + 2j) / 2
    int x_bf16, y_bf16;
    rusty_cuda_dev_status* status;
    long long* dbg;   // optional per-CTA timeline (development aid), null in normal use
};

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 :
                 : "r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}

// Four bytes (int8) -> four floats, exactly (see gemv.cu).
__device__ __forceinline__ void s8x4_to_f32(uint32_t w, float (&f)[4]) {
    w ^= 0x80808080u;
    f[0] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650)) - 8388736.0f;
    f[1] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7651)) - 8388736.0f;
    f[2] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7652)) - 8388736.0f;
    f[3] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7653)) - 8388736.0f;
}

// MB activation rows (1 or 2), NJ passes of 4096 k.
#ifdef RUSTY_TIMELINE
#define TDBG(slot) do { if (p.dbg) p.dbg[(size_t)blockIdx.x * 16 + (slot)] = (long long)globaltimer_ns(); } while (0)
#else
#define TDBG(slot) do { } while (0)
#endif

template <int MB, int NJ>
__global__ void __launch_bounds__(TG_THREADS, 2) gemv_tma_kernel(const TgParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int stage_bytes = p.rows_per_stage * p.K;
    const int stage_stride = (stage_bytes + 127) & ~127;
    uint8_t* sW = smem;
    float* sPart = reinterpret_cast<float*>(sW + (size_t)p.stages * stage_stride);   // [stages][4 rows][MB][CW]
    uint64_t* full = reinterpret_cast<uint64_t*>(sPart + (size_t)p.stages * 4 * MB * CW);
    uint64_t* done = full + p.stages;   // compute warps: stage read and partials written (count CW)
    uint64_t* freeb = done + p.stages;  // reducer: partials consumed, the stage may be refilled (count 1)
    volatile int* abort_flag = reinterpret_cast<volatile int*>(freeb + p.stages);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) TDBG(0);
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&done[s], CW);
            mbar_init(&freeb[s], 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == CW + 1) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            const uint64_t pol = policy_evict_first();
            int stage = 0;
            uint32_t phase = 0;
            for (int t = blockIdx.x; t < p.tiles; t += gridDim.x) {
                if (!mbar_wait(&freeb[stage], phase ^ 1u, abort_flag, p.status, 21)) break;
                const int row0 = t * p.rows_per_stage;
                const int rows = min(p.rows_per_stage, p.N - row0);
                const uint32_t bytes = (uint32_t)rows * (uint32_t)p.K;
                mbar_expect_tx(&full[stage], bytes);
                bulk_load(sW + (size_t)stage * stage_stride, p.W + (size_t)row0 * p.K, bytes, &full[stage], pol);
                if (++stage == p.stages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == CW) {
        // ------------------------------ reducer -------------------------------
        pdl_wait();  // y belongs to earlier kernels until now
        int stage = 0;
        uint32_t phase = 0;
        for (int t = blockIdx.x; t < p.tiles; t += gridDim.x) {
            if (!mbar_wait(&done[stage], phase, abort_flag, p.status, 22)) break;
            const int row0 = t * p.rows_per_stage;
            {
                const int r = lane / MB, m = lane % MB;
                const int n = row0 + r;
                bool live = lane < p.rows_per_stage * MB && n < p.N && m < p.M;
                float s = 0.0f;
                if (live) {
                    const float* pp = sPart + ((size_t)(stage * 4 + r) * MB + m) * CW;
#pragma unroll
                    for (int w = 0; w < CW; ++w) s += pp[w];
                    s *= __ldg(p.scales + n);
                }
                size_t col = (size_t)p.y_col0 + n;
                if (p.act) {
                    // rows r, r+1 of the tile are one (gate, up) pair (tiles hold an even number of rows): the even row's lane
                    // takes the value MB lanes further on and writes silu(gate) * up (MLP::forward composition)
                    const float up = __shfl_down_sync(0xffffffffu, s, MB);
                    live = live && !(r & 1);
                    s = __fdividef(s, 1.0f + __expf(-s)) * up;
                    col >>= 1;
                }
                if (live) {
                    if (p.y_bf16)
                        reinterpret_cast<__nv_bfloat16*>(p.y)[(size_t)m * p.ldy + col] = __float2bfloat16_rn(s);
                    else
                        reinterpret_cast<float*>(p.y)[(size_t)m * p.ldy + col] = s;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&freeb[stage]);
            if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
        if (lane == 0) TDBG(6);
    } else {
        // ------------------------------ compute -------------------------------
        pdl_wait();  // x may come from the previous kernel
        if (threadIdx.x == 0) TDBG(1);
        // this lane's activations: 16 consecutive k per pass, for the whole kernel
        float xr[MB][NJ][16];
#pragma unroll
        for (int m = 0; m < MB; ++m)
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int k = ((j * CHUNKS_PER_PASS) + warp * 32 + lane) * 16;
#pragma unroll
                for (int e4 = 0; e4 < 4; ++e4) {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (m < p.M && k + e4 * 4 < p.K) {
                        if (p.x_bf16) {
                            const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.x) +
                                                                              (size_t)m * p.K + k + e4 * 4);
                            v = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                            __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
                        } else {
                            v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x) + (size_t)m * p.K + k + e4 * 4);
                        }
                    }
                    xr[m][j][e4 * 4 + 0] = v.x;
                    xr[m][j][e4 * 4 + 1] = v.y;
                    xr[m][j][e4 * 4 + 2] = v.z;
                    xr[m][j][e4 * 4 + 3] = v.w;
                }
            }
        if (threadIdx.x == 0) TDBG(3);
        int stage = 0;
        uint32_t phase = 0;
        for (int t = blockIdx.x; t < p.tiles; t += gridDim.x) {
            if (!mbar_wait(&full[stage], phase, abort_flag, p.status, 23)) break;
            if (threadIdx.x == 0 && t == blockIdx.x) TDBG(4);
            const uint8_t* tile = sW + (size_t)stage * stage_stride;
            const int rows = min(p.rows_per_stage, p.N - t * p.rows_per_stage);
            float acc[4][MB];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int m = 0; m < MB; ++m) acc[r][m] = 0.0f;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                if (r < rows) {
#pragma unroll
                    for (int j = 0; j < NJ; ++j) {
                        const int k = ((j * CHUNKS_PER_PASS) + warp * 32 + lane) * 16;
                        if (k < p.K) {
                            const uint4 wv = *reinterpret_cast<const uint4*>(tile + (size_t)r * p.K + k);
                            const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                float f[4];
                                s8x4_to_f32(words[q], f);
#pragma unroll
                                for (int m = 0; m < MB; ++m) {
                                    acc[r][m] = fmaf(xr[m][j][q * 4 + 0], f[0], acc[r][m]);
                                    acc[r][m] = fmaf(xr[m][j][q * 4 + 1], f[1], acc[r][m]);
                                    acc[r][m] = fmaf(xr[m][j][q * 4 + 2], f[2], acc[r][m]);
                                    acc[r][m] = fmaf(xr[m][j][q * 4 + 3], f[3], acc[r][m]);
                                }
                            }
                        }
                    }
                }
            }
            // fold the lanes: after the butterfly lane 8*i holds row i's sum over this warp's k
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                const bool up16 = (lane & 16) != 0;
                float keep0 = up16 ? acc[2][m] : acc[0][m], send0 = up16 ? acc[0][m] : acc[2][m];
                float keep1 = up16 ? acc[3][m] : acc[1][m], send1 = up16 ? acc[1][m] : acc[3][m];
                keep0 += __shfl_xor_sync(0xffffffffu, send0, 16);   // lanes <16: row 0, lanes >=16: row 2
                keep1 += __shfl_xor_sync(0xffffffffu, send1, 16);   // lanes <16: row 1, lanes >=16: row 3
                const bool up8 = (lane & 8) != 0;
                float keep = up8 ? keep1 : keep0, send = up8 ? keep0 : keep1;
                keep += __shfl_xor_sync(0xffffffffu, send, 8);      // bit 3 picks row +1
                keep += __shfl_xor_sync(0xffffffffu, keep, 4);
                keep += __shfl_xor_sync(0xffffffffu, keep, 2);
                keep += __shfl_xor_sync(0xffffffffu, keep, 1);
                if ((lane & 7) == 0) {
                    const int r = ((lane >> 4) & 1) * 2 + ((lane >> 3) & 1);
                    sPart[((size_t)(stage * 4 + r) * MB + m) * CW + warp] = keep;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&done[stage]);
            if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
        if (threadIdx.x == 0) TDBG(5);
    }
}

template <int MB, int NJ>
int launch_tg(rusty_cuda_ctx* ctx, const TgParams& p, int grid, size_t smem) {
    auto kern = gemv_tma_kernel<MB, NJ>;
    {
        cudaError_t e = rusty::ensure_dynamic_smem((const void*)kern, ctx->device, smem);
        if (e != cudaSuccess) return rusty::check_cuda(ctx, e, "gemv_tma: cudaFuncSetAttribute");
    }
    cudaError_t le = launch_pdl(kern, dim3(grid), dim3(TG_THREADS), smem, ctx->stream, p);
    if (le != cudaSuccess) return rusty::check_cuda(ctx, le, "gemv_tma");
    return rusty::after_launch(ctx, "gemv_tma");
}

}  // namespace

namespace rusty {

bool gemv_tma_supported(const rusty_cuda_ctx*, const QLinearArgs& a) {
    if (a.layout != RUSTY_CUDA_LAYOUT_NK || a.qmode != RUSTY_CUDA_QMODE_SYM_ROW) return false;
    if (a.act && a.K > 8192) return false;  // a stage then holds one row: no (gate, up) pair inside a tile
    if (a.M < 1 || a.M > 2) return false;
    if (a.K % 16 != 0 || a.K > (uint32_t)((a.M == 1 ? MAXJ : 2) * CHUNKS_PER_PASS * 16)) return false;
    static const bool off = getenv("RUSTY_NO_GEMV_TMA") != nullptr;
    if (off) return false;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.x) & 15) != 0) return false;
    return true;
}

int launch_gemv_tma(rusty_cuda_ctx* ctx, const QLinearArgs& a) {
    TgParams p{};
    p.W = a.w;
    p.scales = a.scales;
    p.x = a.x;
    p.y = a.y;
    p.M = (int)a.M;
    p.N = (int)a.N;
    p.K = (int)a.K;
    p.rows_per_stage = a.K <= 4096 ? 4 : a.K <= 8192 ? 2 : 1;
    p.tiles = (p.N + p.rows_per_stage - 1) / p.rows_per_stage;
    p.ldy = (int)a.ldy;
    p.y_col0 = (int)a.y_col0;
    p.act = a.act;
    p.x_bf16 = a.x_dtype == RUSTY_CUDA_BF16;
    p.y_bf16 = a.y_dtype == RUSTY_CUDA_BF16;
    p.status = ctx->status_dev;
    p.dbg = nullptr;
    if (ctx->tc_dbg) {  // development aid: one timeline region (304 CTAs x 16 slots) per launch, round robin
        const int regions = (int)((size_t)ctx->tc_dbg_slots * 152 / 304);
        p.dbg = (long long*)ctx->tc_dbg + (size_t)(regions > 0 ? ctx->tc_dbg_seq % regions : 0) * 304 * 16;
        ctx->tc_dbg_seq++;
    }
    const int MB = a.M == 1 ? 1 : 2;
    const size_t stage_stride = ((size_t)p.rows_per_stage * p.K + 127) & ~(size_t)127;
    // a quarter of an SM's shared memory: two CTAs of this kernel (16 compute warps per SM hide the conversion and
    // shuffle latencies far better than 8) plus two of the next kernel, which prefetch while these drain
    // (long problems: two CTAs with half each, deeper rings matter more than the hand-over to the next kernel)
    const bool longrun = p.tiles >= 16 * ctx->sm_count;
    const size_t budget = (ctx->smem_optin > 8192 ? ctx->smem_optin - 8192 : 0) / (longrun ? 2 : 4);
    int stages = (int)(budget / (stage_stride + 4 * MB * CW * 4 + 24));
    if (stages > 12) stages = 12;
    if (stages < 2) return fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "gemv_tma: stage does not fit shared memory");
    p.stages = stages;
    const size_t smem = (size_t)stages * stage_stride + (size_t)stages * 4 * MB * CW * 4 + (size_t)stages * 24 + 64;
    // short problems: one CTA per SM (the next kernel's CTA moves in beside it); long ones: two per SM
    const int per_sm = 2;
    int grid = ctx->sm_count * per_sm;
    if (grid > p.tiles) grid = p.tiles;
    const int NJ = (int)((a.K + CHUNKS_PER_PASS * 16 - 1) / (CHUNKS_PER_PASS * 16));
    if (MB == 1) {
        switch (NJ) {
            case 1: return launch_tg<1, 1>(ctx, p, grid, smem);
            case 2: return launch_tg<1, 2>(ctx, p, grid, smem);
            case 3: return launch_tg<1, 3>(ctx, p, grid, smem);
            default: return launch_tg<1, 4>(ctx, p, grid, smem);
        }
    }
    switch (NJ) {
        case 1: return launch_tg<2, 1>(ctx, p, grid, smem);
        case 2: return launch_tg<2, 2>(ctx, p, grid, smem);
        default: return fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "gemv_tma: two rows need K <= 8192");
    }
}

}  // namespace rusty
