// Fused int8-weight linear on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Replaces the reference's "dequantise once at load, f32 tiled matmul per
// forward" (rusty-loader/src/lib.rs:155-218, rusty-backend/src/kernels.wgsl:16-54,
// :234-242) for batches of activation rows: y[M,N] = x[M,K] . (q[N,K] * scale[N])^T.
//
// Arithmetic.  The weights stay int8 all the way into the tensor core
// (tcgen05.mma kind::i8, int32 accumulation in tensor memory); nothing is
// dequantised in the main loop.  The activations are decomposed EXACTLY into
// D signed 7-bit digits relative to one power-of-two scale per row,
//     x[m,k] * s_m = d0 + d1/128 + d2/128^2 (+ d3/128^3),  |d0| <= 127, |d1..| <= 64,
// by a small pre-pass; each digit plane is one column block of the B operand.
// The integer dot products are exact, the digit planes are recombined in
// 64-bit integers and multiplied by 1/s_m and scale[n] once, so the result is
// the correctly rounded value of the dot product of the (digit-truncated)
// activations: D=4 (f32 activations) keeps 28 bits below the row maximum, D=3
// (bf16 activations) 21.  Results do not depend on how K is split over CTAs:
// integer partial sums are order-independent.
//
// Data movement per CTA (persistent, one per SM, warp-specialised):
//   warp 0  : TMA producer — 128x128-byte weight tiles (HBM, read once) and the
//             matching NBx128-byte digit tiles (L2) into an 8-stage smem ring,
//             128-byte swizzle, mbarrier complete_tx;
//   warp 1  : allocates TMEM, issues tcgen05.mma (M=128, N=NB, K=32) from one
//             elected lane, frees ring slots with tcgen05.commit;
//   warps 2-5: epilogue — tcgen05.ld the int32 accumulators (double-buffered in
//             TMEM), fold the digits into int64 in a shared-memory staging tile,
//             scale, store y; or, when K is split over several CTAs, add the
//             staged piece into the tile's sum in L2 with one bulk reduce and
//             convert an equal share of the rows once all pieces have arrived.
// Every mbarrier wait is bounded by a wall-clock limit; on expiry the kernel
// raises the context's timeout flag, drains and frees its TMEM.
#include <cstdlib>
#include <cstring>

#include "tc_common.cuh"

using namespace rusty_tc;

namespace {

// Kernel timeline (%globaltimer stamps per CTA), compiled in only with -DRUSTY_TIMELINE (a development build).
#ifdef RUSTY_TIMELINE
#define DBG(slot) do { if (p.dbg) p.dbg[(size_t)blockIdx.x * 16 + (slot)] = (long long)globaltimer_ns(); } while (0)
#define PDBG(cond, slot) do { if (dbg && (cond)) dbg[slot] = (long long)globaltimer_ns(); } while (0)
#else
#define DBG(slot) do { } while (0)
#define PDBG(cond, slot) do { } while (0)
#endif

constexpr int BM = 128;            // weight rows per tile = UMMA M
constexpr int BK = 128;            // k-elements (bytes) per pipeline stage
constexpr int UMMA_K = 32;         // k-elements per tcgen05.mma kind::i8
constexpr int TC_THREADS = 192;    // producer warp, MMA warp, 4 epilogue warps
constexpr int EPI_THREADS = 128;
constexpr int A_STAGE_BYTES = BM * BK;

template <typename T>
__device__ __forceinline__ void store_y(T* p, float v);
template <>
__device__ __forceinline__ void store_y<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_y<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// ----------------------------------------------------------------------------
// Pre-pass: activations -> digit planes.
// xq is [D*Mpad, K] int8, row d*Mpad + m; inv_s[m] = 1 / (s_m * 128^(D-1)).  One block per m
// (rows M..Mpad-1 are written as zeros).
// ----------------------------------------------------------------------------
template <typename XT>
__device__ __forceinline__ float x_to_f32(XT v);
template <>
__device__ __forceinline__ float x_to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float x_to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// Four consecutive activations as f32 (p is 16-byte aligned for f32, 8-byte aligned for bf16: K % 16 == 0).
template <typename XT>
__device__ __forceinline__ float4 load_row4(const XT* p);
template <>
__device__ __forceinline__ float4 load_row4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 load_row4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                       __uint_as_float(raw.y & 0xffff0000u));
}

constexpr int DIG_THREADS = 1024;  // one block per activation row; a 4096-wide row is one 16-byte load per thread

template <typename XT, int D>
__global__ void __launch_bounds__(DIG_THREADS) digitize_x_kernel(const XT* __restrict__ x, int8_t* __restrict__ xq,
                                                                 float* __restrict__ inv_s, int M, int Mpad, int K,
                                                                 const PeerPush push, long long* dbg,
                                                                 unsigned int* __restrict__ counters, int n_counters) {
    const int m = blockIdx.x;
    __shared__ float red[DIG_THREADS / 32];
    __shared__ float s_scale;
    const int tid = threadIdx.x;
    PDBG(tid == 0 && m == 0, 0);
    pdl_launch_dependents();
    pdl_wait();  // x may come from the previous kernel, and that kernel may still be reading the digit planes
    PDBG(tid == 0 && m == 0, 1);
    // arrival counters of the GEMM's shared tiles: the kernel before has finished with them, the GEMM after this
    // kernel counts from zero
    for (int i = m * DIG_THREADS + tid; i < n_counters; i += gridDim.x * DIG_THREADS) counters[i] = 0u;
    if (push.nranks > 1) {
        // x may hold columns pushed by the other ranks, and the GEMM that follows overwrites their copies of y:
        // wait until every rank has finished (and delivered) all earlier pushes
        if (tid == 0) peer_wait_all(push, 30);
        __syncthreads();
        PDBG(tid == 0 && m == 0, 3);
    }
    if (m >= M) {
        for (int k = tid * 4; k < K; k += DIG_THREADS * 4)
#pragma unroll
            for (int d = 0; d < D; ++d) *reinterpret_cast<uint32_t*>(xq + (size_t)(d * Mpad + m) * K + k) = 0u;
        return;
    }
    const XT* xr = x + (size_t)m * K;
    // Rows of up to 16384 elements stay in registers between the maximum and the digits (one trip to memory).
    constexpr int MAXV = 4;
    const bool in_regs = K <= DIG_THREADS * 4 * MAXV;
    float4 v[MAXV];
    float mx = 0.0f;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int k = (j * DIG_THREADS + tid) * 4;
            v[j] = k < K ? load_row4<XT>(xr + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const float a4[4] = {fabsf(v[j].x), fabsf(v[j].y), fabsf(v[j].z), fabsf(v[j].w)};
#pragma unroll
            for (int e = 0; e < 4; ++e) mx = (a4[e] <= 3.0e38f) ? fmaxf(mx, a4[e]) : __int_as_float(0x7f800000);
        }
    } else {
        for (int k = tid; k < K; k += DIG_THREADS) {
            float a = fabsf(x_to_f32<XT>(xr[k]));
            mx = (a <= 3.0e38f) ? fmaxf(mx, a) : __int_as_float(0x7f800000);  // NaN or inf anywhere poisons the row
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    if (tid < 32) {
        float vmax = red[tid];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, off));
        if (tid == 0) {
            // s = the power of two that puts vmax*s into [64, 128) but not above 127
            float s = 1.0f;
            if (vmax >= 1.0e-30f && vmax <= 3.0e38f) {
                const int e = (int)((__float_as_uint(vmax) >> 23) & 0xffu) - 126;  // vmax = f * 2^e, f in [0.5, 1)
                s = __uint_as_float((uint32_t)(127 + 7 - e) << 23);                 // 2^(7-e): 7-e in [-121, 106]
                if (vmax * s > 127.0f) s *= 0.5f;
            } else if (vmax > 0.0f && vmax <= 3.0e38f) {
                int e;
                frexpf(vmax, &e);
                s = ldexpf(1.0f, 7 - e > 120 ? 120 : 7 - e);  // tiny rows: any power of two that keeps |x*s| <= 127 will do
            }
            s_scale = s;
            // 1/s_m * 128^-(D-1): both powers of two, so the product is exact
            inv_s[m] = (vmax <= 3.0e38f) ? ldexpf(1.0f / s, -7 * (D - 1)) : __int_as_float(0x7fc00000);  // inf/nan poisons the row
        }
    }
    __syncthreads();
    const float s = s_scale;
    auto emit = [&](int k, const float4& f) {
        const float in4[4] = {f.x, f.y, f.z, f.w};
        uint32_t packed[D];
#pragma unroll
        for (int d = 0; d < D; ++d) packed[d] = 0u;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float r = in4[e] * s;  // exact: s is a power of two
#pragma unroll
            for (int d = 0; d < D; ++d) {
                float q = rintf(r);
                packed[d] |= ((uint32_t)(int)q & 0xFFu) << (8 * e);
                r = (r - q) * 128.0f;  // exact
            }
        }
#pragma unroll
        for (int d = 0; d < D; ++d) *reinterpret_cast<uint32_t*>(xq + (size_t)(d * Mpad + m) * K + k) = packed[d];
    };
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int k = (j * DIG_THREADS + tid) * 4;
            if (k < K) emit(k, v[j]);
        }
    } else {
        for (int k = tid * 4; k < K; k += DIG_THREADS * 4) emit(k, load_row4<XT>(xr + k));  // K % 4 == 0 (K % 16 == 0 is required by the caller)
    }
    PDBG(tid == 0 && m == 0, 2);
}

// ----------------------------------------------------------------------------
// Main kernel
// ----------------------------------------------------------------------------
struct TcParams {
    const float* scales;     // [N]
    const float* row_factor; // [Mpad]: 1/s_m * 128^-(D-1)
    int32_t* part;           // sums of tiles cut across CTAs: [sk_tiles][Mpad/2][128] x 16 bytes (two int64), zero between uses
    unsigned int* counters;  // [tiles] arrivals per cut tile (zero between uses)
    void* y;
    int M, Mpad, D, NB;      // NB = UMMA N = roundup16(D*Mpad)
    int N, K;
    int tiles, kb_total;     // row tiles, k-blocks per row tile
    // Schedule.  The last `sk_tiles` row tiles are cut stream-K fashion: their
    // sk_tiles*kb_total k-blocks form one linear space dealt out in contiguous
    // runs of `sk_per_cta` to the first `sk_ctas` CTAs.  The other tiles are
    // taken whole, tile = cta, cta + grid, ...
    int dp_tiles, sk_tiles, sk_per_cta, sk_ctas;
    int sk_ways;             // > 0: every shared tile is cut into this many near-equal pieces, one per CTA (CTA = tile * ways + piece)
    int ldy, y_col0;
    int act;                 // RUSTY_CUDA_ACT_SWIGLU_PAIRS: rows 2j, 2j+1 -> y[:, (y_col0 + 2j) / 2] = silu(gate) * up
    int stages;
    int red_bytes;           // epilogue staging area: a partial tile (Mpad x 128 x 8 bytes), at least 12 KiB
    uint32_t idesc;
    uint32_t tmem_cols;
    rusty_cuda_dev_status* status;
    long long* dbg;          // optional per-CTA timeline (16 slots each), null in normal use
    PeerPush push;           // nranks > 1: every output is also stored into the other ranks' arenas
};

// One piece of work: k-blocks [kb0, kb1) of row tile t.  nseg > 1: the tile is
// shared with other CTAs; `slot` is where this CTA parks its partial sums.
struct Segment {
    int t, kb0, kb1, nseg, slot, first_cta;
};

// Every role of the CTA walks the same segment list.
struct Sched {
    const TcParams& p;
    int g, g_end;   // position inside the stream-K space
    int dp_next;    // next whole tile
    int seg_index;
    __device__ Sched(const TcParams& pp) : p(pp) {
        const int c = blockIdx.x;
        if (p.sk_ways > 0) {
            // one piece per CTA, cut at the same places in every tile: g walks the piece's k-blocks
            const int lt = c / p.sk_ways, j = c % p.sk_ways;
            g = c < p.sk_ctas ? lt * p.kb_total + j * p.kb_total / p.sk_ways : 0;
            g_end = c < p.sk_ctas ? lt * p.kb_total + (j + 1) * p.kb_total / p.sk_ways : 0;
        } else {
            g = c < p.sk_ctas ? c * p.sk_per_cta : 0;
            g_end = c < p.sk_ctas ? min(p.sk_tiles * p.kb_total, g + p.sk_per_cta) : 0;
        }
        dp_next = c;
        seg_index = 0;
    }
    __device__ bool next(Segment& s) {
        if (g < g_end) {  // stream-K part first: its cross-CTA fix-up then overlaps the whole tiles that follow
            const int lt = g / p.kb_total;
            s.t = p.dp_tiles + lt;
            s.kb0 = g % p.kb_total;
            s.kb1 = min(p.kb_total, s.kb0 + (g_end - g));
            if (p.sk_ways > 0) {
                s.first_cta = lt * p.sk_ways;
                s.nseg = p.sk_ways;
            } else {
                s.first_cta = (lt * p.kb_total) / p.sk_per_cta;
                const int last_cta = ((lt + 1) * p.kb_total - 1) / p.sk_per_cta;
                s.nseg = last_cta - s.first_cta + 1;
            }
            // head piece (the CTA's run starts inside this tile) -> even slot, tail piece -> odd slot
            s.slot = 2 * (int)blockIdx.x + ((int)blockIdx.x * p.sk_per_cta >= lt * p.kb_total ? 0 : 1);
            g += s.kb1 - s.kb0;
            ++seg_index;
            return true;
        }
        if (dp_next < p.dp_tiles) {
            s.t = dp_next;
            s.kb0 = 0;
            s.kb1 = p.kb_total;
            s.nseg = 1;
            s.slot = 0;
            s.first_cta = 0;
            dp_next += gridDim.x;
            ++seg_index;
            return true;
        }
        return false;
    }
};

// Digits -> one exact 64-bit integer -> f32 (one rounding) -> row factor (a power
// of two, exact) -> weight scale (one rounding).
// The other ranks' arenas as byte offsets from this rank's (exchange by peer stores), kept in shared memory: indexing
// an array inside the kernel parameter with a run-time index makes the compiler copy it to local memory at every use.
struct PeerOut {
    int n;                   // number of other ranks (0: no exchange)
    const long long* delta;  // [n] in shared memory
};
// Four outputs at once: the four conversion chains (int64 -> f32, two multiplies, and for pairs a shuffle, exp and
// reciprocal) are independent and written so that they overlap; one at a time they cost ~150 ns each in the single
// warp per scheduler that runs them.  Output k is row m[k] of feature n[k]; live[k] says whether it exists.  Every lane
// of the warp must call this together, and lane parity must equal the parity of n[k] (pair epilogue).
template <typename YT>
__device__ __forceinline__ void finalize_store4(const TcParams& p, YT* y, const int (&n)[4], const int (&m)[4], const long long (&acc)[4],
                                                const float (&scale_n)[4], const float* s_rowf, const PeerOut& po, const bool (&live)[4]) {
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = __ll2float_rn(acc[k]) * s_rowf[m[k]] * scale_n[k];
    if (p.act) {
        // rows 2j / 2j+1 are gate_j / up_j: the even lane takes its neighbour's value and writes silu(gate) * up
        // (rusty-graph/src/lib.rs:317-323; silu as kernels.wgsl:104-113, with ex2.approx and an approximate reciprocal)
        float up[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) up[k] = __shfl_down_sync(0xffffffffu, v[k], 1);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = __fdividef(v[k], 1.0f + __expf(-v[k])) * up[k];
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (live[k] && !(p.act && (n[k] & 1))) {
            const int col = p.act ? (p.y_col0 + n[k]) >> 1 : p.y_col0 + n[k];
            YT* dst = y + (size_t)m[k] * p.ldy + col;
            store_y<YT>(dst, v[k]);
            // exchange fused into the epilogue: the same element of every other rank's y, over NVLink
            for (int g = 0; g < po.n; ++g) store_y<YT>(reinterpret_cast<YT*>(reinterpret_cast<char*>(dst) + po.delta[g]), v[k]);
        }
    }
}

template <typename YT>
__global__ void __launch_bounds__(TC_THREADS, 2)
qlinear_i8_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                     const __grid_constant__ TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // carve: [A stages][B stages][barriers]
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int b_stage_bytes = p.NB * BK;
    uint8_t* sA = smem;
    uint8_t* sB = smem + (size_t)p.stages * A_STAGE_BYTES;
    // epilogue staging for the bulk reduce-add of a partial tile: [Mpad/2][128] x 16 bytes
    int4* stage_red = reinterpret_cast<int4*>(sB + (size_t)p.stages * b_stage_bytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(stage_red) + (size_t)p.red_bytes);
    uint64_t* full = bars;                      // [stages]
    uint64_t* empty = bars + p.stages;          // [stages]
    uint64_t* acc_full = bars + 2 * p.stages;   // [2]
    uint64_t* acc_empty = acc_full + 2;         // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    __shared__ float s_rowf[64];  // 1/s_m * 128^-(D-1) per activation row of this pass (at most 64 rows)
    __shared__ long long s_peer_delta[PEER_MAX_RANKS];
    if (threadIdx.x == 0) {
        int k = 0;  // the other ranks, compacted (own rank left out); static indices into the parameter
#pragma unroll
        for (int g = 0; g < PEER_MAX_RANKS; ++g)
            if (g < p.push.nranks && g != p.push.rank) s_peer_delta[k++] = p.push.delta[g];
    }
    const PeerOut po = {p.push.nranks > 1 ? p.push.nranks - 1 : 0, s_peer_delta};  // visible after the set-up barrier below
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) DBG(0);
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, p.tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) DBG(1);

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
            int stage = 0;
            uint32_t phase = 0;
            int issued = 0;
            bool ok = true;
            Sched sched(p);
            Segment sg;
            // The weights do not depend on earlier kernels: start streaming them at once.  The digit planes do, so
            // the first ring-full of stages gets its weight tile now and its digit tile after pdl_wait().
            int early = 0;           // stages whose weight tile is already in flight
            int early_kb[8];
            bool waited = false;
            while (ok && sched.next(sg)) {
                for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
                    if (!waited && early < p.stages) {
                        mbar_expect_tx(&full[early], (uint32_t)(A_STAGE_BYTES + b_stage_bytes));
                        tma_load_2d(sA + (size_t)early * A_STAGE_BYTES, &map_w, kb * BK, sg.t * BM, &full[early], pol_w);
                        early_kb[early] = kb;
                        ++early;
                        ++issued;
                        if (issued == 1) DBG(2);
                        if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                        continue;
                    }
                    if (!waited) {
                        pdl_wait();
                        for (int e = 0; e < early; ++e)
                            tma_load_2d(sB + (size_t)e * b_stage_bytes, &map_x, early_kb[e] * BK, 0, &full[e], pol_x);
                        waited = true;
                    }
                    if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
                    mbar_expect_tx(&full[stage], (uint32_t)(A_STAGE_BYTES + b_stage_bytes));
                    tma_load_2d(sA + (size_t)stage * A_STAGE_BYTES, &map_w, kb * BK, sg.t * BM, &full[stage], pol_w);
                    tma_load_2d(sB + (size_t)stage * b_stage_bytes, &map_x, kb * BK, 0, &full[stage], pol_x);
                    ++issued;
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!waited) {  // fewer k-blocks than ring slots
                pdl_wait();
                for (int e = 0; e < early; ++e)
                    tma_load_2d(sB + (size_t)e * b_stage_bytes, &map_x, early_kb[e] * BK, 0, &full[e], pol_x);
            }
            DBG(3);
            if (!ok) {
                // give the copies still in flight a bounded chance to land before the CTA tears down
                for (int j = 0; j < p.stages && j < issued; ++j) {
                    const int idx = issued - 1 - j;
                    uint64_t* bar = &full[idx % p.stages];
                    const uint32_t par = (uint32_t)(idx / p.stages) & 1u;
                    const long long t0 = clock64();
                    while (!mbar_try_wait(bar, par) && clock64() - t0 < 4000000ll) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            Sched sched(p);
            Segment sg;
            for (int i = 0; ok && sched.next(sg); ++i) {
                const int ab = i & 1;
                if (!mbar_wait(&acc_empty[ab], (((uint32_t)i >> 1) & 1u) ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(ab * p.NB);
                for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
                    if (!mbar_wait(&full[stage], phase, abort_flag, p.status, 3)) { ok = false; break; }
                    tc_fence_after();
                    if (kb == sg.kb0 && i == 0) DBG(4);
                    const uint64_t da = make_smem_desc(smem_u32(sA + (size_t)stage * A_STAGE_BYTES));
                    const uint64_t db = make_smem_desc(smem_u32(sB + (size_t)stage * b_stage_bytes));
#pragma unroll
                    for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
                        // advance 32 bytes along K inside the 128-byte swizzle atom: +2 in 16-byte units
                        umma_i8(d_tmem, da + (uint64_t)(2 * k4), db + (uint64_t)(2 * k4), p.idesc, (kb > sg.kb0 || k4 > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[stage]);
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(&acc_full[ab]);
                DBG(5);
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        const int r = q * 32 + lane;            // row inside the tile
        YT* y = reinterpret_cast<YT*>(p.y);
        const int ncol = p.D * p.Mpad;          // accumulator columns in use
        pdl_wait();                             // x, y, the sums and the counters belong to earlier kernels until now
        bool ok = true;
        const int et = threadIdx.x - 64;        // 0..127 among the epilogue threads
        // per-row factors of the pre-pass: once into shared memory (a load from global memory per output costs
        // an L2 round trip each time)
        if (et < p.Mpad) s_rowf[et] = __ldcg(p.row_factor + et);
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
        int cut_t[2], cut_j[2], cut_n[2], n_cut = 0;  // shared tiles this CTA added a piece to
        bool announced = false;
        Sched sched(p);
        Segment sg;
        for (int i = 0;; ++i) {
            const bool have = ok && sched.next(sg);
            // Shared tiles: once all pieces of a tile have been added, each CTA that holds one of them turns an equal share
            // of the tile's rows into y and leaves zeros behind (the arrival counters are cleared by the next pre-pass).  All pieces are added before anybody waits here, and the
            // CTAs of the grid are resident together (one wave), so the wait cannot depend on a CTA that has not started.
            // Announce this CTA's pieces once its last shared segment is behind it (the adds complete about when the
            // weight stream ends); convert after the CTA's last whole tile, when the other pieces have arrived too.
            if (ok && n_cut > 0 && !announced && (!have || sg.nseg == 1)) {
                if (threadIdx.x == 64) {
                    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // this CTA's adds have been performed
                    __threadfence();
                    for (int e = 0; e < n_cut; ++e)
                        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.counters + cut_t[e]) : "memory");
                }
                announced = true;
            }
            for (int e = 0; ok && e < n_cut && !have; ++e) {
                const int t = cut_t[e], nseg = cut_n[e], j = cut_j[e];
                if (threadIdx.x == 64) {
                    const long long t0 = clock64();
                    while (ld_acquire_gpu_u32(p.counters + t) < (unsigned)nseg) {
                        if (*abort_flag || clock64() - t0 > WAIT_LIMIT_CYCLES) {
                            *abort_flag = 1;
                            if (atomicExch(&p.status->timeout_flag, 1u) == 0u) p.status->timeout_where = 8;
                            break;
                        }
                    }
                    DBG(10);
                }
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
                if (*abort_flag) { ok = false; break; }
                int4* tile_sum = reinterpret_cast<int4*>(p.part) + (size_t)(t - p.dp_tiles) * (p.Mpad / 2) * BM;
                // this CTA's share of the tile's rows, cut in units of two rows so that a (gate, up) pair stays together
                const int lo = 2 * (j * (BM / 2) / nseg), rows = 2 * ((j + 1) * (BM / 2) / nseg) - lo;
                const int items = rows * (p.Mpad / 2);                         // one item: a row, two activation rows
                if (rows <= 0) continue;
                // item -> (row, mp) without a division per item: start at (et % rows, et / rows), step by EPI_THREADS items
                int row = et % rows, mp = et / rows;
                const int step_row = EPI_THREADS % rows, step_mp = EPI_THREADS / rows;
                // the loop bounds are the same for every thread: the pair epilogue needs whole warps
                for (int base = 0; base < items; base += 4 * EPI_THREADS) {
                    const int it0 = base + et;
                    int4 v[4];
                    float sc[4];
                    int rw[4], mq[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {  // independent loads: one L2 round trip per batch
                        rw[u] = lo + row;
                        mq[u] = mp;
                        const bool in = it0 + u * EPI_THREADS < items && t * BM + rw[u] < p.N;
                        v[u] = in ? __ldcg(tile_sum + (size_t)mp * BM + rw[u]) : make_int4(0, 0, 0, 0);
                        sc[u] = in ? __ldg(p.scales + t * BM + rw[u]) : 0.0f;
                        row += step_row;
                        mp += step_mp;
                        if (row >= rows) {
                            row -= rows;
                            ++mp;
                        }
                    }
                    // Park the batch in this thread's slots of the staging tile (free by now) and convert in a rolled
                    // loop: code that runs once per CTA costs an instruction fetch per line, so it is kept short.
                    float* stage_sc = reinterpret_cast<float*>(stage_red + 4 * EPI_THREADS);
                    int* stage_at = reinterpret_cast<int*>(stage_sc + 4 * EPI_THREADS);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const bool live = it0 + u * EPI_THREADS < items;
                        if (live) __stcg(tile_sum + (size_t)mq[u] * BM + rw[u], make_int4(0, 0, 0, 0));
                        stage_red[u * EPI_THREADS + et] = v[u];
                        stage_sc[u * EPI_THREADS + et] = sc[u];
                        stage_at[u * EPI_THREADS + et] = (live && t * BM + rw[u] < p.N) ? (rw[u] | (mq[u] << 8)) : -1;
                    }
#pragma unroll 1
                    for (int u = 0; u < 4; u += 2) {  // two items = four outputs per trip
                        const int at0 = stage_at[u * EPI_THREADS + et], at1 = stage_at[(u + 1) * EPI_THREADS + et];
                        const bool v0 = at0 >= 0, v1 = at1 >= 0;
                        const longlong2 t0 = *reinterpret_cast<const longlong2*>(&stage_red[u * EPI_THREADS + et]);
                        const longlong2 t1 = *reinterpret_cast<const longlong2*>(&stage_red[(u + 1) * EPI_THREADS + et]);
                        const float s0 = stage_sc[u * EPI_THREADS + et], s1 = stage_sc[(u + 1) * EPI_THREADS + et];
                        const int n0 = t * BM + (at0 & 0xff), n1 = t * BM + (at1 & 0xff);
                        const int m0 = v0 ? 2 * (at0 >> 8) : 0, m1 = v1 ? 2 * (at1 >> 8) : 0;
                        const long long a4[4] = {t0.x, t0.y, t1.x, t1.y};
                        const int n4[4] = {n0, n0, n1, n1}, m4[4] = {m0, m0 + 1, m1, m1 + 1};
                        const float s4[4] = {s0, s0, s1, s1};
                        const bool l4[4] = {v0 && m0 < p.M, v0 && m0 + 1 < p.M, v1 && m1 < p.M, v1 && m1 + 1 < p.M};
                        finalize_store4<YT>(p, y, n4, m4, a4, s4, s_rowf, po, l4);
                    }
                }
                if (threadIdx.x == 64) DBG(11);
                // the batch was parked in the staging tile at slots indexed by thread, the whole tile that may follow
                // is staged there at slots indexed by row: no warp may start on it while another still reads its batch
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
            }
            if (!have || !ok) break;
            const int ab = i & 1;
            const int n = sg.t * BM + r;
            const bool row_ok = n < p.N;
            if (!mbar_wait(&acc_full[ab], ((uint32_t)i >> 1) & 1u, abort_flag, p.status, 4)) { ok = false; break; }
            tc_fence_after();
            if (threadIdx.x == 64) DBG(6 + 4 * (i & 1));
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(ab * p.NB);
            {
                // Fold the digit planes into one exact 64-bit integer per output and stage them in shared memory
                // ([m/2][row] x 16 bytes).  A whole tile is converted from there in a rolled loop (unrolled register
                // code that runs once per tile costs an instruction fetch per line and was twice as slow); a piece of
                // a shared tile is added into the tile's sum in global memory with ONE bulk reduce
                // (cp.reduce.async.bulk ... add.u64: the adds happen in L2 at line rate).
                for (int m0 = 0; m0 < p.Mpad; m0 += 8) {
                    int32_t c[4][8];
#pragma unroll
                    for (int d = 0; d < 4; ++d)
                        if (d < p.D) tmem_ld8(taddr + (uint32_t)(d * p.Mpad + m0), c[d]);
                    tmem_ld_wait();
#pragma unroll
                    for (int h = 0; h < 4; ++h) {
                        long long a0 = c[0][2 * h], a1 = c[0][2 * h + 1];
#pragma unroll
                        for (int d = 1; d < 4; ++d)
                            if (d < p.D) {
                                a0 = a0 * 128 + c[d][2 * h];
                                a1 = a1 * 128 + c[d][2 * h + 1];
                            }
                        if (!row_ok) a0 = a1 = 0;
                        int4 v;
                        v.x = (int)(a0 & 0xffffffffll);
                        v.y = (int)(a0 >> 32);
                        v.z = (int)(a1 & 0xffffffffll);
                        v.w = (int)(a1 >> 32);
                        stage_red[(size_t)(m0 / 2 + h) * BM + r] = v;
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[ab]);
                if (threadIdx.x == 64) DBG(7 + 4 * (i & 1));
                if (sg.nseg == 1) {
                    // every thread reads back only what it staged itself: no barrier needed
                    const float sc = row_ok ? __ldg(p.scales + n) : 0.0f;
#pragma unroll 1
                    for (int m = 0; m < p.M; m += 4) {  // Mpad is a multiple of 8: the staged rows m .. m+3 exist
                        const longlong2 t0 = *reinterpret_cast<const longlong2*>(&stage_red[(size_t)(m >> 1) * BM + r]);
                        const longlong2 t1 = *reinterpret_cast<const longlong2*>(&stage_red[(size_t)((m >> 1) + 1) * BM + r]);
                        const long long a4[4] = {t0.x, t0.y, t1.x, t1.y};
                        const int n4[4] = {n, n, n, n}, m4[4] = {m, m + 1, m + 2, m + 3};
                        const float s4[4] = {sc, sc, sc, sc};
                        const bool l4[4] = {row_ok, row_ok && m + 1 < p.M, row_ok && m + 2 < p.M, row_ok && m + 3 < p.M};
                        finalize_store4<YT>(p, y, n4, m4, a4, s4, s_rowf, po, l4);
                    }
                    if (threadIdx.x == 64) DBG(9 + 4 * (i & 1));
                    continue;
                }
                const int lt = sg.t - p.dp_tiles;
                int4* tile_sum = reinterpret_cast<int4*>(p.part) + (size_t)lt * (p.Mpad / 2) * BM;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // staged values -> visible to the bulk-copy engine
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
                if (threadIdx.x == 64) {
                    const uint32_t bytes = (uint32_t)(p.Mpad * 8 * BM);
                    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.u64 [%0], [%1], %2;" ::"l"(tile_sum),
                                 "r"(smem_u32(stage_red)), "r"(bytes)
                                 : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    // only until the staging tile has been read: the adds themselves complete while the next segment
                    // is folded, and are waited for (and announced) before the shared conversion below
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                }
                if (threadIdx.x == 64) DBG(8 + 4 * (i & 1));
                // The conversion of the finished sums is shared between the CTAs that hold the tile's pieces and is
                // done after the CTA's last segment (below): remember the tile and which piece this was.
                if (n_cut < 2) {
                    cut_t[n_cut] = sg.t;
                    cut_j[n_cut] = (int)blockIdx.x - sg.first_cta;
                    cut_n[n_cut] = sg.nseg;
                    ++n_cut;
                } else {
                    ok = false;  // cannot happen: a run of k-blocks starts and ends inside at most two shared tiles
                    if (threadIdx.x == 64 && atomicExch(&p.status->timeout_flag, 1u) == 0u) p.status->timeout_where = 7;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");  // the staging tile is free again (the bulk reduce has read it)
                if (threadIdx.x == 64) DBG(9 + 4 * (i & 1));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) DBG(14);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, p.tmem_cols);
    }
    if (threadIdx.x == 0) {
        peer_signal_cta_done(p.push);  // after the barrier: every store of this CTA is issued
        DBG(15);
    }
}

// ----------------------------------------------------------------------------
// Host side
// ----------------------------------------------------------------------------
// Workspace layout.  Every region is followed by a guard zone filled with a fixed byte that no kernel may touch;
// rusty_cuda_ctx_self_check reads the guards back (the tool-free stand-in for a memory checker).
constexpr size_t WS_GUARD = 1024;
constexpr unsigned char WS_GUARD_BYTE = 0xA5;
constexpr size_t WS_XQ_BYTES = 24u << 20;      // digit planes: up to 256 rows x K <= 96K
constexpr size_t WS_INVS_BYTES = 4096;
constexpr size_t WS_ACC_BYTES = 48u << 20;     // split-K partial sums
constexpr size_t WS_CNT_BYTES = 64u << 10;     // arrival counters, kept at zero between kernels (small-batch mode, prefill kernels)
constexpr size_t WS_CNT2_BYTES = 64u << 10;    // arrival counters of the GEMM with a pre-pass, which clears them
constexpr size_t WS_OFF_XQ = 0;
constexpr size_t WS_OFF_INVS = WS_OFF_XQ + WS_XQ_BYTES + WS_GUARD;
constexpr size_t WS_OFF_ACC = WS_OFF_INVS + WS_INVS_BYTES + WS_GUARD;
constexpr size_t WS_OFF_CNT = WS_OFF_ACC + WS_ACC_BYTES + WS_GUARD;
constexpr size_t WS_OFF_CNT2 = WS_OFF_CNT + WS_CNT_BYTES + WS_GUARD;
constexpr size_t WS_TOTAL = WS_OFF_CNT2 + WS_CNT2_BYTES + WS_GUARD;
constexpr size_t WS_GUARD_AT[5] = {WS_OFF_INVS - WS_GUARD, WS_OFF_ACC - WS_GUARD, WS_OFF_CNT - WS_GUARD, WS_OFF_CNT2 - WS_GUARD,
                                   WS_TOTAL - WS_GUARD};

// The schedule of one launch: how the row tiles are dealt to the CTAs.  One place for the regular entry points and the
// entry point with built-in scratch, so that their guards cannot drift apart.
//   whole tiles (tile = cta, cta + grid, ...) for the first dp_tiles tiles; the last sk_tiles tiles are cut along K.
// `sums_tiles_cap` / `counter_cap`: how many cut tiles the caller's scratch can park / how many arrival counters
// (indexed by the GLOBAL tile number) it holds.  Returns false when N needs more counters than there are.
struct TcSchedule {
    int grid, dp_tiles, sk_tiles, sk_per_cta, sk_ctas, sk_ways;
};
bool plan_tc_schedule(int tiles, int kb_total, int sm_count, int dp_percent, size_t sums_tiles_cap, size_t counter_cap,
                      TcSchedule* out) {
    if ((size_t)tiles > counter_cap) return false;
    TcSchedule s{};
    // Whole waves of row tiles are taken tile-per-CTA; the remainder (fewer tiles than SMs) is cut stream-K fashion so
    // every SM streams the same number of k-blocks.  A cut needs >= 4 k-blocks per CTA and room for the parked tiles.
    int grid = sm_count;
    if (grid > tiles * kb_total / 4) grid = tiles * kb_total / 4 > 0 ? tiles * kb_total / 4 : 1;
    s.sk_tiles = tiles % grid;
    s.dp_tiles = tiles - s.sk_tiles;
    // Whole tiles only, dealt evenly (r or r-1 per CTA), when that still keeps most SMs streaming: ~110 SMs at the
    // tensor-core rate already draw the full HBM bandwidth, and a CTA without shared tiles skips the bulk
    // reduce-add, the wait for the other pieces and the shared conversion (5-10 us at the end of the kernel).
    {
        const int r = (tiles + sm_count - 1) / sm_count;   // tiles per CTA
        const int g_dp = r > 0 ? (tiles + r - 1) / r : 0;  // CTAs that then have work
        if (s.sk_tiles > 0 && g_dp * 100 >= sm_count * dp_percent) {
            grid = g_dp;
            s.sk_tiles = 0;
            s.dp_tiles = tiles;
        }
    }
    if (s.sk_tiles > 0) {
        const int sk_work = s.sk_tiles * kb_total;
        s.sk_per_cta = (sk_work + grid - 1) / grid;
        if (s.sk_per_cta < 4) s.sk_per_cta = 4;
        // Prefer cuts that line up with tile borders (every CTA then holds one piece and a tile has exactly
        // `ways` pieces) when that keeps at least 85% of the SMs busy.
        const int ways = grid / s.sk_tiles;
        if (ways >= 1) {
            const int aligned = (kb_total + ways - 1) / ways;
            if (aligned >= 4 && (long long)s.sk_per_cta * 100 >= (long long)aligned * 85) s.sk_per_cta = aligned;
        }
        s.sk_ctas = (sk_work + s.sk_per_cta - 1) / s.sk_per_cta;
        // No whole tiles at all and room for `ways` CTAs per tile: cut every tile at the same places, so that each CTA
        // holds exactly one piece (runs of a fixed length drift across tile borders and leave most CTAs with two).
        if (s.dp_tiles == 0 && ways >= 2 && kb_total / ways >= 4) {
            s.sk_ways = ways;
            s.sk_ctas = s.sk_tiles * ways;
            s.sk_per_cta = (kb_total + ways - 1) / ways;
        }
        if ((size_t)s.sk_tiles > sums_tiles_cap) {
            s.dp_tiles = tiles;  // no room to park partial tiles: whole tiles only
            s.sk_tiles = 0;
            s.sk_per_cta = 0;
            s.sk_ctas = 0;
            s.sk_ways = 0;
            if (grid > tiles) grid = tiles;
        }
    }
    if (s.dp_tiles == 0 && s.sk_ctas > 0) grid = s.sk_ctas;
    s.grid = grid;
    *out = s;
    return true;
}

int pick_digits(int x_dtype, uint32_t rows) {
    // f32 activations: 4 planes = 28 bits below the row maximum.  Three planes (21 bits) hold the fp32 tolerance only
    // while the row's largest element stays within ~25x of its rms: with one outlier of 1000x every other element
    // keeps 11 bits and the result is ~5e-5 off.  bf16 activations carry 8 significant bits each: 3 planes.
    (void)rows;
    return x_dtype == RUSTY_CUDA_F32 ? 4 : 3;
}

template <typename XT>
cudaError_t launch_digitize(rusty_cuda_ctx* ctx, const void* x, int8_t* xq, float* inv_s, int M, int Mpad, int K, int D,
                            const PeerPush& push, long long* dbg, unsigned int* counters, int n_counters) {
    if (D == 4)
        return launch_pdl(digitize_x_kernel<XT, 4>, dim3(Mpad), dim3(DIG_THREADS), 0, ctx->stream, (const XT*)x, xq, inv_s, M, Mpad, K, push, dbg,
                          counters, n_counters);
    return launch_pdl(digitize_x_kernel<XT, 3>, dim3(Mpad), dim3(DIG_THREADS), 0, ctx->stream, (const XT*)x, xq, inv_s, M, Mpad, K, push, dbg,
                      counters, n_counters);
}

}  // namespace

namespace rusty {

int tc_workspace_reserve(rusty_cuda_ctx* ctx) {
    if (ctx->tc_ws) return RUSTY_CUDA_OK;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, WS_TOTAL);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, RUSTY_CUDA_ERR_MEMORY_ALLOCATION, "tensor-core workspace: cudaMalloc(%zu) failed", (size_t)WS_TOTAL);
    }
    e = cudaMemsetAsync(p, 0, WS_TOTAL, ctx->stream);
    for (size_t g = 0; e == cudaSuccess && g < 5; ++g) e = cudaMemsetAsync((uint8_t*)p + WS_GUARD_AT[g], WS_GUARD_BYTE, WS_GUARD, ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(p);
        return check_cuda(ctx, e, "tensor-core workspace: memset");
    }
    ctx->tc_ws = p;
    ctx->tc_ws_bytes = WS_TOTAL;
    return RUSTY_CUDA_OK;
}

// The zero-maintained part of the workspace (sums of cut tiles + arrival counters), shared by the tensor-core
// kernels: both leave zeros behind, and kernels on one stream never overlap in their epilogues.
void tc_workspace_sums(rusty_cuda_ctx* ctx, float** sums, size_t* sums_bytes, unsigned int** counters, size_t* cnt_bytes) {
    uint8_t* ws = (uint8_t*)ctx->tc_ws;
    *sums = ws ? (float*)(ws + WS_OFF_ACC) : nullptr;
    *sums_bytes = WS_ACC_BYTES;
    *counters = ws ? (unsigned int*)(ws + WS_OFF_CNT) : nullptr;
    *cnt_bytes = WS_CNT_BYTES;
}

// Reads the guard zones back (drains the stream).  Returns the index of the first damaged guard, or -1.
int tc_workspace_check_guards(rusty_cuda_ctx* ctx, cudaError_t* err) {
    *err = cudaSuccess;
    if (!ctx->tc_ws) return -1;
    std::vector<unsigned char> host(WS_GUARD);
    for (int g = 0; g < 5; ++g) {
        *err = cudaMemcpyAsync(host.data(), (uint8_t*)ctx->tc_ws + WS_GUARD_AT[g], WS_GUARD, cudaMemcpyDeviceToHost, ctx->stream);
        if (*err == cudaSuccess) *err = cudaStreamSynchronize(ctx->stream);
        if (*err != cudaSuccess) return -1;
        for (size_t i = 0; i < WS_GUARD; ++i)
            if (host[i] != WS_GUARD_BYTE) return g;
    }
    return -1;
}

void tc_workspace_release(rusty_cuda_ctx* ctx) {
    if (ctx->tc_ws) cudaFree(ctx->tc_ws);
    ctx->tc_ws = nullptr;
    ctx->tc_ws_bytes = 0;
}

uint32_t tc_min_rows() {
    // RUSTY_TC_MIN_ROWS overrides the crossover between the CUDA-core GEMV and the tensor-core kernel (tuning aid).
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("RUSTY_TC_MIN_ROWS");
        v = e ? atoi(e) : 3;
        if (v < 1) v = 1;
    }
    return (uint32_t)v;
}

bool tc_supported(const rusty_cuda_ctx* ctx, const QLinearArgs& a) {
    if (!ctx->tc_ws || !encode_tiled_fn()) return false;
    if (a.layout != RUSTY_CUDA_LAYOUT_NK || a.qmode != RUSTY_CUDA_QMODE_SYM_ROW) return false;
    if (a.K % 16 != 0 || a.K > 96 * 1024) return false;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15) != 0) return false;
    return true;
}

// The kernel pair below stores into the peers' arenas itself, except in the small-batch mode that has no pre-pass.
bool tc_pushes_fused(uint32_t M) { return M >= tc_min_rows(); }

// One launch pair (digitise + GEMM) for up to 64 activation rows.
static int launch_tc_rows(rusty_cuda_ctx* ctx, const QLinearArgs& a, const void* x, void* y, uint32_t rows) {
    const int M = (int)rows, Mpad = (M + 7) / 8 * 8;
    const int D = pick_digits(a.x_dtype, rows);
    const int NB = (D * Mpad + 15) / 16 * 16;
    uint8_t* ws = (uint8_t*)ctx->tc_ws;
    int8_t* xq = (int8_t*)ws;
    float* inv_s = (float*)(ws + WS_OFF_INVS);
    int32_t* acc = (int32_t*)(ws + WS_OFF_ACC);
    // two sets of arrival counters: one kept at zero by its users, one cleared by the pre-pass of this path
    unsigned int* counters = (unsigned int*)(ws + WS_OFF_CNT2);   // this set is cleared by the pre-pass
    if ((size_t)D * Mpad * a.K > WS_XQ_BYTES)
        return fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "tensor-core path: %d digit rows x K=%u exceed the workspace", D * Mpad, a.K);

    cudaError_t le = cudaSuccess;
    int rc = RUSTY_CUDA_OK;
    const int n_tiles = (int)((a.N + BM - 1) / BM);
    if ((size_t)n_tiles * 4 > WS_CNT_BYTES)
        return fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "tensor-core path: N=%u has more row tiles than arrival counters", a.N);
    // development aid: each launch pair writes its timeline into the next 152 x 16 slots of the attached buffer
    long long* dbg = nullptr;
    if (ctx->tc_dbg) {
        dbg = (long long*)ctx->tc_dbg + (size_t)ctx->tc_dbg_seq * 152 * 16;
        ctx->tc_dbg_seq = (ctx->tc_dbg_seq + 1) % (ctx->tc_dbg_slots > 0 ? ctx->tc_dbg_slots : 1);
    }
    PeerPush push{};
    if (a.push && a.push->nranks > 1) {
        push = *a.push;
    }
    {
        le = a.x_dtype == RUSTY_CUDA_BF16 ? launch_digitize<__nv_bfloat16>(ctx, x, xq, inv_s, M, Mpad, (int)a.K, D, push, dbg ? dbg + 150 * 16 : nullptr, counters, n_tiles)
                                          : launch_digitize<float>(ctx, x, xq, inv_s, M, Mpad, (int)a.K, D, push, dbg ? dbg + 150 * 16 : nullptr, counters, n_tiles);
        if (le != cudaSuccess) return check_cuda(ctx, le, "digitize_x");
        rc = after_launch(ctx, "digitize_x");
        if (rc) return rc;
    }

    TcParams p{};
    p.scales = a.scales;
    p.row_factor = inv_s;
    p.part = acc;
    p.counters = counters;
    p.y = y;
    p.M = M;
    p.Mpad = Mpad;
    p.D = D;
    p.NB = NB;
    p.N = (int)a.N;
    p.K = (int)a.K;
    p.tiles = (p.N + BM - 1) / BM;
    p.kb_total = (p.K + BK - 1) / BK;
    // RUSTY_TC_DP_PERCENT: least share of the SMs that whole tiles must keep streaming (default 72; 101 turns the rule off).
    static const int dp_percent = getenv("RUSTY_TC_DP_PERCENT") ? atoi(getenv("RUSTY_TC_DP_PERCENT")) : 72;
    TcSchedule sc{};
    if (!plan_tc_schedule(p.tiles, p.kb_total, ctx->sm_count, dp_percent, WS_ACC_BYTES / ((size_t)Mpad * BM * 8),
                          WS_CNT_BYTES / 4, &sc))
        return fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "tensor-core path: N=%u has more row tiles than arrival counters", a.N);
    int grid = sc.grid;
    p.dp_tiles = sc.dp_tiles;
    p.sk_tiles = sc.sk_tiles;
    p.sk_per_cta = sc.sk_per_cta;
    p.sk_ctas = sc.sk_ctas;
    p.sk_ways = sc.sk_ways;
    p.ldy = (int)a.ldy;
    p.y_col0 = (int)a.y_col0;
    p.act = a.act;
    p.status = ctx->status_dev;
    p.dbg = dbg;
    p.push = push;
    // int8 x int8 -> int32, both K-major: c_format=S32(2)@4, a_format=INT8(1)@7, b_format=INT8(1)@10, N>>3 @17, M>>4 @24
    p.idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    uint32_t cols = 32;
    while (cols < (uint32_t)(2 * NB)) cols <<= 1;
    p.tmem_cols = cols;
    const int b_stage = NB * BK;
    // Half of the SM's shared memory at most, so that the next kernel's CTA can move in beside this one and
    // prefetch its weights while this one drains (RUSTY_TC_FULL_SMEM=1: take it all, 8 stages).
    static const bool full_smem = getenv("RUSTY_TC_FULL_SMEM") != nullptr;
    size_t budget = ctx->smem_optin > 4096 ? ctx->smem_optin - 4096 : 0;
    if (!full_smem && NB <= 32 && 4 * A_STAGE_BYTES + 4096 <= budget / 2)
        budget = budget / 2 - 1024;  // narrow batches: leave room for the next kernel's CTA on the SM
    // epilogue staging of a partial tile; the shared finalize parks 4 x 128 sums, scales and positions there (12 KiB)
    const size_t red_bytes = (size_t)Mpad * 8 * BM > 12288 ? (size_t)Mpad * 8 * BM : (size_t)12288;
    int stages = budget > red_bytes + 2048
                     ? (int)((budget - 1024 - 512 - red_bytes) / (size_t)(A_STAGE_BYTES + b_stage))
                     : 0;
    if (stages > 8) stages = 8;
    if (stages < 2) return fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "tensor-core path: tile does not fit shared memory");
    p.stages = stages;
    p.red_bytes = (int)red_bytes;
    const size_t smem = 1024 + (size_t)stages * (A_STAGE_BYTES + b_stage) + red_bytes + (size_t)(2 * stages + 4) * 8 + 256;

    CUtensorMap map_w, map_x;
    if (!make_map_u8(&map_w, a.w, a.N, a.K, BM) ||
        !make_map_u8(&map_x, xq, (uint64_t)D * Mpad, a.K, (uint32_t)NB))
        return fail(ctx, RUSTY_CUDA_ERR_KERNEL_EXECUTION, "tensor-core path: cuTensorMapEncodeTiled failed");

    const bool yb = a.y_dtype == RUSTY_CUDA_BF16;

    auto kern = yb ? qlinear_i8_tc_kernel<__nv_bfloat16> : qlinear_i8_tc_kernel<float>;
    {
        cudaError_t e = ensure_dynamic_smem((const void*)kern, ctx->device, smem);
        if (e != cudaSuccess) return check_cuda(ctx, e, "qlinear_i8_tc: cudaFuncSetAttribute");
    }
    le = launch_pdl(kern, dim3(grid), dim3(TC_THREADS), smem, ctx->stream, map_w, map_x, p);
    if (le != cudaSuccess) return check_cuda(ctx, le, "qlinear_i8_tc");
    return after_launch(ctx, "qlinear_i8_tc");
}

int launch_tc(rusty_cuda_ctx* ctx, const QLinearArgs& a) {
    const size_t xs = a.x_dtype == RUSTY_CUDA_BF16 ? 2 : 4, ys = a.y_dtype == RUSTY_CUDA_BF16 ? 2 : 4;
    for (uint32_t m0 = 0; m0 < a.M; m0 += 64) {
        uint32_t rows = a.M - m0 < 64 ? a.M - m0 : 64;
        int rc = launch_tc_rows(ctx, a, (const char*)a.x + (size_t)m0 * a.K * xs, (char*)a.y + (size_t)m0 * a.ldy * ys, rows);
        if (rc) return rc;
    }
    return RUSTY_CUDA_OK;
}

}  // namespace rusty

#ifdef RUSTY_TIMELINE
// Development builds only (-DRUSTY_TIMELINE; not part of the C ABI): point the kernels' timeline (%globaltimer stamps,
// one region of 152 x 16 int64 slots per launch pair, round robin) at a caller buffer, or detach it with NULL.
extern "C" RUSTY_CUDA_API int rusty_cuda_debug_set_timeline(rusty_cuda_ctx* ctx, rusty_cuda_buf* buf) {
    if (!ctx) return RUSTY_CUDA_ERR_INVALID_OPERATION;
    ctx->tc_dbg = buf ? buf->ptr : nullptr;
    ctx->tc_dbg_seq = 0;
    ctx->tc_dbg_slots = buf ? (int)(buf->bytes / (152 * 16 * 8)) : 0;
    return RUSTY_CUDA_OK;
}
#endif

// ----------------------------------------------------------------------------
// Entry point for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: inside a
// latency-critical serving loop whose memory was carved up front, or under an
// allocator that owns every byte of the device and treats a foreign allocation
// as a leak.  For them the tensor-core kernel's scratch (digit planes of the
// activations, per-row factors, sums of K-cut tiles, arrival counters, status
// word) lives in the fixed array below, which every GPU that loads this library
// holds until the process exits.
// ----------------------------------------------------------------------------
namespace {

constexpr uint32_t STATIC_MAX_ROWS = 8;       // activation rows per call
constexpr uint32_t STATIC_MAX_K = 8192;       // input features
constexpr uint32_t STATIC_MAX_N = 262144;     // output features: one arrival counter per 128-row tile, indexed by tile number
constexpr int STATIC_MAX_CTAS = 160;          // CTAs launched at most (one per SM)
constexpr size_t ST_XQ_BYTES = (size_t)4 * 8 * STATIC_MAX_K;            // 4 digit planes x 8 padded rows
constexpr size_t ST_FACTOR_BYTES = 256;
constexpr size_t ST_SUMS_TILES = STATIC_MAX_CTAS;                        // cut tiles parked at most (fewer than CTAs)
constexpr size_t ST_SUMS_BYTES = ST_SUMS_TILES * 8 * 8 * BM;            // one parked 8-row tile (int64) per cut tile
constexpr size_t ST_CNT_BYTES = (size_t)(STATIC_MAX_N / BM) * 4;        // 2048 counters
constexpr size_t ST_STATUS_BYTES = 256;
constexpr size_t ST_TOTAL = ST_XQ_BYTES + ST_FACTOR_BYTES + ST_SUMS_BYTES + ST_CNT_BYTES + ST_STATUS_BYTES;  // ~1.5 MiB
static_assert(ST_CNT_BYTES / 4 * BM == STATIC_MAX_N, "one arrival counter per row tile up to STATIC_MAX_N");
static_assert(STATIC_MAX_N % BM == 0, "the N cap is a whole number of row tiles");

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[ST_TOTAL];

struct StaticDev {
    bool ready = false;
    unsigned char* base = nullptr;
    int sm_count = 0;
    size_t smem_optin = 0;
};
std::mutex g_static_mu;
StaticDev g_static_dev[64];

int static_status_to_code(unsigned int timeout_flag, unsigned int timeout_where) {
    if (timeout_flag == 0u) return RUSTY_CUDA_OK;
    return rusty::fail(nullptr, RUSTY_CUDA_ERR_TIMEOUT, "qlinear_i8_forward_static: a bounded device-side wait gave up (site %u); y is incomplete",
                       timeout_where);
}

}  // namespace

extern "C" RUSTY_CUDA_API int rusty_cuda_qlinear_i8_forward_static(const void* w_i8, const float* scales, const float* x_f32,
                                                                   float* y_f32, uint32_t M, uint32_t N, uint32_t K,
                                                                   void* stream) {
    using namespace rusty;
    if (!w_i8 || !scales || !x_f32 || !y_f32)
        return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_i8_forward_static: null pointer");
    if (M == 0 || N == 0) return RUSTY_CUDA_OK;
    if (M > STATIC_MAX_ROWS || K > STATIC_MAX_K || K == 0 || K % 16 != 0 || N > STATIC_MAX_N)
        return fail(nullptr, RUSTY_CUDA_ERR_INVALID_DIMENSIONS,
                    "qlinear_i8_forward_static: M=%u N=%u K=%u outside the fixed scratch (M <= %u, N <= %u, K <= %u, K %% 16 == 0)", M,
                    N, K, STATIC_MAX_ROWS, STATIC_MAX_N, STATIC_MAX_K);
    if ((reinterpret_cast<uintptr_t>(w_i8) & 15) != 0)
        return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_i8_forward_static: weights must be 16-byte aligned");
    if (!encode_tiled_fn())
        return fail(nullptr, RUSTY_CUDA_ERR_UNSUPPORTED, "qlinear_i8_forward_static: cuTensorMapEncodeTiled is not available");
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return check_cuda(nullptr, e == cudaSuccess ? cudaErrorInvalidDevice : e, "cudaGetDevice");
    StaticDev sd;
    {
        // First call on a device: look up where the array lives ON THAT DEVICE (it must be current) and read
        // two device attributes.  Nothing is allocated.  Do this once before any stream capture.
        std::lock_guard<std::mutex> lk(g_static_mu);
        StaticDev& slot = g_static_dev[dev];
        if (!slot.ready) {
            void* ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (e != cudaSuccess) return check_cuda(nullptr, e, "cudaGetSymbolAddress(static scratch)");
            int sms = 0, optin = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (e == cudaSuccess) e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
            if (e != cudaSuccess) return check_cuda(nullptr, e, "cudaDeviceGetAttribute");
            slot.base = (unsigned char*)ptr;
            slot.sm_count = sms;
            slot.smem_optin = (size_t)optin;
            slot.ready = true;
        }
        sd = slot;
    }
    cudaStream_t st = (cudaStream_t)stream;
    int8_t* xq = (int8_t*)sd.base;
    float* factor = (float*)(sd.base + ST_XQ_BYTES);
    unsigned char* zeroed = sd.base + ST_XQ_BYTES + ST_FACTOR_BYTES;  // sums, counters, status: must start at zero
    int32_t* sums = (int32_t*)zeroed;
    unsigned int* counters = (unsigned int*)(zeroed + ST_SUMS_BYTES);
    rusty_cuda_dev_status* status = (rusty_cuda_dev_status*)(zeroed + ST_SUMS_BYTES + ST_CNT_BYTES);
    e = cudaMemsetAsync(zeroed, 0, ST_SUMS_BYTES + ST_CNT_BYTES + ST_STATUS_BYTES, st);
    if (e != cudaSuccess) return check_cuda(nullptr, e, "qlinear_i8_forward_static: clearing the scratch");

    const int Mi = (int)M, Mpad = 8, D = 4, NB = 32;
    e = launch_pdl(digitize_x_kernel<float, 4>, dim3(Mpad), dim3(DIG_THREADS), 0, st, x_f32, xq, factor, Mi, Mpad, (int)K, PeerPush{}, (long long*)nullptr, counters, (int)((N + BM - 1) / BM));
    if (e != cudaSuccess) return check_cuda(nullptr, e, "qlinear_i8_forward_static: digitize_x");

    TcParams p{};
    p.scales = scales;
    p.row_factor = factor;
    p.part = sums;
    p.counters = counters;
    p.y = y_f32;
    p.M = Mi;
    p.Mpad = Mpad;
    p.D = D;
    p.NB = NB;
    p.N = (int)N;
    p.K = (int)K;
    p.tiles = (p.N + BM - 1) / BM;
    p.kb_total = (p.K + BK - 1) / BK;
    // the same schedule rules as the regular entry points, with this scratch's capacities
    TcSchedule sc{};
    if (!plan_tc_schedule(p.tiles, p.kb_total, sd.sm_count < STATIC_MAX_CTAS ? sd.sm_count : STATIC_MAX_CTAS,
                          /*dp_percent=*/72, ST_SUMS_TILES, ST_CNT_BYTES / 4, &sc))
        return fail(nullptr, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_i8_forward_static: N=%u has more row tiles than arrival counters", N);
    const int grid = sc.grid;
    p.dp_tiles = sc.dp_tiles;
    p.sk_tiles = sc.sk_tiles;
    p.sk_per_cta = sc.sk_per_cta;
    p.sk_ctas = sc.sk_ctas;
    p.sk_ways = sc.sk_ways;
    p.ldy = (int)N;
    p.y_col0 = 0;
    p.status = status;
    p.dbg = nullptr;
    p.idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    p.tmem_cols = 64;
    const int b_stage = NB * BK;
    const size_t red_bytes = (size_t)Mpad * 8 * BM > 12288 ? (size_t)Mpad * 8 * BM : (size_t)12288;
    const size_t budget = (sd.smem_optin > 4096 ? sd.smem_optin - 4096 : 0) / 2;
    int stages = budget > red_bytes + 4096 ? (int)((budget - 2048 - red_bytes) / (size_t)(A_STAGE_BYTES + b_stage)) : 0;
    if (stages > 8) stages = 8;
    if (stages < 2) return fail(nullptr, RUSTY_CUDA_ERR_UNSUPPORTED, "qlinear_i8_forward_static: shared memory too small");
    p.stages = stages;
    p.red_bytes = (int)red_bytes;
    const size_t smem = 1024 + (size_t)stages * (A_STAGE_BYTES + b_stage) + red_bytes + (size_t)(2 * stages + 4) * 8 + 256;
    CUtensorMap map_w, map_x;
    if (!make_map_u8(&map_w, w_i8, N, K, BM) || !make_map_u8(&map_x, xq, (uint64_t)D * Mpad, K, (uint32_t)NB))
        return fail(nullptr, RUSTY_CUDA_ERR_KERNEL_EXECUTION, "qlinear_i8_forward_static: cuTensorMapEncodeTiled failed");
    auto kern = qlinear_i8_tc_kernel<float>;
    // Raise the kernel's dynamic shared-memory limit to the device maximum: enough for this launch and never
    // below what another entry point has asked for.
    cudaFuncAttributes fa;
    e = cudaFuncGetAttributes(&fa, kern);
    if (e != cudaSuccess) return check_cuda(nullptr, e, "qlinear_i8_forward_static: cudaFuncGetAttributes");
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sd.smem_optin - fa.sharedSizeBytes));
    if (e != cudaSuccess) return check_cuda(nullptr, e, "qlinear_i8_forward_static: cudaFuncSetAttribute");
    e = launch_pdl(kern, dim3(grid), dim3(TC_THREADS), smem, st, map_w, map_x, p);
    if (e != cudaSuccess) return check_cuda(nullptr, e, "qlinear_i8_forward_static: launch");
    return RUSTY_CUDA_OK;
}

// The kernel behind the entry point above bounds every wait; when one runs out it raises a flag in the built-in scratch
// and leaves y incomplete.  This call drains `stream` and reports that flag of the most recent static forward on the
// current device (the next static forward clears it).  Allocates nothing.
extern "C" RUSTY_CUDA_API int rusty_cuda_qlinear_i8_static_status(void* stream) {
    using namespace rusty;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return check_cuda(nullptr, e == cudaSuccess ? cudaErrorInvalidDevice : e, "cudaGetDevice");
    unsigned char* base = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (g_static_dev[dev].ready) base = g_static_dev[dev].base;
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (!base) {  // no static forward has run on this device yet: nothing to report, only drain
        e = cudaStreamSynchronize(st);
        return e == cudaSuccess ? RUSTY_CUDA_OK : check_cuda(nullptr, e, "qlinear_i8_static_status: synchronize");
    }
    rusty_cuda_dev_status h{};
    e = cudaMemcpyAsync(&h, base + ST_XQ_BYTES + ST_FACTOR_BYTES + ST_SUMS_BYTES + ST_CNT_BYTES, sizeof(h), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return check_cuda(nullptr, e, "qlinear_i8_static_status");
    return static_status_to_code(h.timeout_flag, h.timeout_where);
}

// Host-side decoding of the status word, exposed for tests that have no GPU.
extern "C" RUSTY_CUDA_API int rusty_cuda_qlinear_i8_static_status_decode(unsigned int timeout_flag, unsigned int timeout_where) {
    return static_status_to_code(timeout_flag, timeout_where);
}

