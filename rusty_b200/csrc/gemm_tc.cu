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
//   warps 2-9: epilogue (four or eight warps) — tcgen05.ld the int32
//             accumulators (double-buffered in TMEM), fold the digits into
//             int64, scale, store y (whole tiles through a shared-memory
//             staging tile); or, when K is split over several CTAs, store the
//             piece as tagged 64-bit words (sum << 1 | 1) into this CTA's slot,
//             poll the other pieces' words until they are non-zero, and convert
//             an equal share of the rows (readers zero the words they used).
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
constexpr int TC_MAX_THREADS = 384;  // producer warp, MMA warp, 4 or 8 epilogue warps (<= 320 threads; 384 caps the registers at 168)
constexpr int A_TILE_BYTES = BM * BK;   // one 128-row weight tile of a stage; a stage holds tpu of them

template <typename T>
__device__ __forceinline__ void store_y(T* p, float v);
template <>
__device__ __forceinline__ void store_y<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_y<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
template <typename T>
__device__ __forceinline__ float load_y(const T* p);
template <>
__device__ __forceinline__ float load_y<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_y<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// ----------------------------------------------------------------------------
// Pre-pass: activations -> digit planes.
// xq is [D*Mpad, K] int8, row d*Mpad + m; inv_s[m] = 1 / (s_m * 128^(D-1)).  One block per m
// (rows M..Mpad-1 are written as zeros).
// ----------------------------------------------------------------------------
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

constexpr int DIG_THREADS = 512;
constexpr int DIG_MAX_BLOCKS = 32;
constexpr int DIG_MAXV = 8;   // passes of a row held in registers between the maximum and the digits

// A few fat blocks on purpose: grid = min(32, Mpad) blocks of 512 threads, R = Mpad / grid activation rows per block
// (1 or 2), 512 / R threads per row (its own named barrier).  The kernel is launched early (programmatic dependent
// launch) and parks in griddepcontrol.wait while the GEMM before it still runs; many small parked blocks pile up on the
// few SMs that GEMM left free and keep the next GEMM's CTAs from being placed there.  Thirty-two blocks of at most 64
// registers a thread fit beside a GEMM CTA on any SM and cannot fill more than eight.  Rows M..Mpad-1 are written as
// zeros.  A row of up to 16384 activations (one row per block) stays in registers between its maximum and its digits:
// one round trip to memory, all loads in flight together.
//
// NORM: the activations are RMSNorm(x [+ residual]) * weight (norm_embed.cu gives the formula and its lines in the
// reference); the row is normalised in registers between the load and the maximum, so it must fit there
// (K <= DIG_MAXV * 4 * threads of the row), and the normalised row and the sum are written out where asked for.
template <typename XT, int D, bool NORM>
__global__ void __launch_bounds__(DIG_THREADS, 2) digitize_x_kernel(const XT* __restrict__ x, int8_t* __restrict__ xq,
                                                                    float* __restrict__ inv_s, int M, int Mpad, int K, int R,
                                                                    const PeerPush push, const NormArgs nrm, long long* dbg) {
    __shared__ float red[DIG_THREADS / 32];
    __shared__ float red_ss[DIG_THREADS / 32];
    const int tid = threadIdx.x;
    const int tpr = DIG_THREADS / R;               // threads per row (512 or 256)
    const int grp = tid / tpr, tg = tid - grp * tpr;
    const int m = blockIdx.x * R + grp;
    PDBG(tid == 0 && blockIdx.x == 0, 0);
    pdl_launch_dependents();
    pdl_wait();  // x may come from the previous kernel, and that kernel may still be reading the digit planes
    PDBG(tid == 0 && blockIdx.x == 0, 1);
    if (push.nranks > 1) {
        // x may hold columns pushed by the other ranks, and the GEMM that follows overwrites their copies of y:
        // meet the other ranks (every rank has finished, and delivered, all earlier pushes)
        if (tid < 32) peer_sync_block(push, (int)blockIdx.x, 30, blockIdx.x == 0 ? dbg : nullptr);
        __syncthreads();
        PDBG(tid == 0 && blockIdx.x == 0, 3);
    }
    const int step = tpr * 4;                       // activations one pass of the row's threads covers
    if (m >= M) {
        for (int k = tg * 4; k < K; k += step)
#pragma unroll
            for (int d = 0; d < D; ++d) *reinterpret_cast<uint32_t*>(xq + (size_t)(d * Mpad + m) * K + k) = 0u;
        return;   // whole row groups leave together: the named barrier below is per group
    }
    const XT* xr = x + (size_t)m * K;
    float4 v[DIG_MAXV];
#pragma unroll
    for (int j = 0; j < DIG_MAXV; ++j) {
        const int k = tg * 4 + j * step;
        v[j] = k < K ? load_row4<XT>(xr + k) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if constexpr (NORM) {
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < DIG_MAXV; ++j) {
            const int k = tg * 4 + j * step;
            if (k < K) {
                if (nrm.residual) {
                    const float4 r = *reinterpret_cast<const float4*>(nrm.residual + (size_t)m * K + k);
                    v[j].x += r.x; v[j].y += r.y; v[j].z += r.z; v[j].w += r.w;
                    if (nrm.sum) *reinterpret_cast<float4*>(nrm.sum + (size_t)m * K + k) = v[j];
                }
                ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        if ((tid & 31) == 0) red_ss[tid >> 5] = ss;
        asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(tpr) : "memory");
        const int wpr_n = tpr / 32;
        float tot = red_ss[grp * wpr_n + (tid & (wpr_n - 1))];
        if (wpr_n == 16) tot += __shfl_xor_sync(0xffffffffu, tot, 8);
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, off);
        const float inv_rms = 1.0f / sqrtf(tot / (float)K + nrm.eps);
#pragma unroll
        for (int j = 0; j < DIG_MAXV; ++j) {
            const int k = tg * 4 + j * step;
            if (k < K) {
                const float4 w = __ldg(reinterpret_cast<const float4*>(nrm.weight + k));
                v[j].x = v[j].x * inv_rms * w.x; v[j].y = v[j].y * inv_rms * w.y;
                v[j].z = v[j].z * inv_rms * w.z; v[j].w = v[j].w * inv_rms * w.w;
                if (nrm.normed) *reinterpret_cast<float4*>(nrm.normed + (size_t)m * K + k) = v[j];
            }
        }
    }
    float mx = 0.0f;
    auto fold = [&](const float4& f) {
        const float a4[4] = {fabsf(f.x), fabsf(f.y), fabsf(f.z), fabsf(f.w)};
#pragma unroll
        for (int e = 0; e < 4; ++e) mx = (a4[e] <= 3.0e38f) ? fmaxf(mx, a4[e]) : __int_as_float(0x7f800000);  // NaN or inf anywhere poisons the row
    };
#pragma unroll
    for (int j = 0; j < DIG_MAXV; ++j) fold(v[j]);
    for (int k = tg * 4 + DIG_MAXV * step; k < K; k += step) fold(load_row4<XT>(xr + k));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(tpr) : "memory");   // the row's threads only
    const int wpr = tpr / 32;                       // warps per row: 16 or 8
    float vmax = red[grp * wpr + (tid & (wpr - 1))];
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, off));
    // s = the power of two that puts vmax*s into [64, 128) but not above 127
    int e2 = 0;
    if (vmax >= 1.0e-30f && vmax <= 3.0e38f) {
        const int e = (int)((__float_as_uint(vmax) >> 23) & 0xffu) - 126;  // vmax = f * 2^e, f in [0.5, 1)
        e2 = 7 - e;
        if (vmax * __uint_as_float((uint32_t)(127 + e2) << 23) > 127.0f) --e2;
    } else if (vmax > 0.0f && vmax <= 3.0e38f) {
        int e;
        frexpf(vmax, &e);
        e2 = 7 - e > 120 ? 120 : 7 - e;  // tiny rows: any power of two that keeps |x*s| <= 127 will do
    }
    const bool finite = vmax <= 3.0e38f;
    const float sc = finite ? __uint_as_float((uint32_t)(127 + e2) << 23) : 0.0f;
    // 1/s_m * 128^-(D-1): both powers of two, so the product is exact; inf/nan poisons the row
    if (tg == 0) inv_s[m] = finite ? ldexpf(1.0f, -e2 - 7 * (D - 1)) : __int_as_float(0x7fc00000);
    for (int k = tg * 4, i = 0; k < K; k += step, ++i) {   // one copy of the conversion code, in a loop
        float4 f = v[0];
#pragma unroll
        for (int j = 1; j < DIG_MAXV; ++j)
            if (i == j) f = v[j];
        if (i >= DIG_MAXV) f = load_row4<XT>(xr + k);
        const uint32_t w0 = digits_of<D>(f.x * sc), w1 = digits_of<D>(f.y * sc), w2 = digits_of<D>(f.z * sc), w3 = digits_of<D>(f.w * sc);
        // 4 elements x 4 digit bytes -> digit planes x 4 element bytes; byte b = digit b from the least significant,
        // byte D-1 = the top digit = plane 0
        const uint32_t t0 = __byte_perm(w0, w1, 0x5140), t1 = __byte_perm(w2, w3, 0x5140);
        const uint32_t t2 = __byte_perm(w0, w1, 0x7362), t3 = __byte_perm(w2, w3, 0x7362);
        const uint32_t by[4] = {__byte_perm(t0, t1, 0x5410), __byte_perm(t0, t1, 0x7632), __byte_perm(t2, t3, 0x5410), __byte_perm(t2, t3, 0x7632)};
#pragma unroll
        for (int d = 0; d < D; ++d) *reinterpret_cast<uint32_t*>(xq + (size_t)(d * Mpad + m) * K + k) = by[D - 1 - d];
    }
    PDBG(tid == 0 && blockIdx.x == 0, 2);
}

// ----------------------------------------------------------------------------
// Main kernel
// ----------------------------------------------------------------------------
struct TcParams {
    const float* scales;     // [N]
    const float* row_factor; // [Mpad]: 1/s_m * 128^-(D-1)
    ulonglong2* part;        // pieces of tiles cut across CTAs: slot (2*cta + head/tail) x [Mpad/2][128] x 16 bytes = two tagged
                             // int64 (value << 1 | 1: a word is valid as soon as it is not zero); all zero between launches
    void* y;
    const void* residual;    // null, or added to every output (same layout as y)
    int M, Mpad, D, NB;      // NB = UMMA N = roundup16(D*Mpad)
    int N, K;
    int tpu, bmu;            // row tiles of 128 per work unit (1 or 2: two tiles share every digit tile they multiply), rows per unit
    int tiles, kb_total;     // work units (called tiles below), k-blocks per unit
    // Schedule.  The last `sk_tiles` row tiles are cut stream-K fashion: their
    // sk_tiles*kb_total k-blocks form one linear space dealt out in contiguous
    // runs of `sk_per_cta` to the first `sk_ctas` CTAs.  The other tiles are
    // taken whole, tile = cta, cta + grid, ...
    int dp_tiles, sk_tiles, sk_per_cta, sk_ctas;
    int sk_ways;             // > 0: every shared tile is cut into this many near-equal pieces, one per CTA (CTA = tile * ways + piece)
    int ldy, y_col0;
    int act;                 // RUSTY_CUDA_ACT_SWIGLU_PAIRS: rows 2j, 2j+1 -> y[:, (y_col0 + 2j) / 2] = silu(gate) * up
    int epi_warps;           // 4 or 8 epilogue warps: two per tensor-memory lane quarter split the activation rows between them
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
            if (p.residual) v[k] += load_y<YT>(reinterpret_cast<const YT*>(p.residual) + ((size_t)m[k] * p.ldy + col));
            store_y<YT>(dst, v[k]);
            // exchange fused into the epilogue: the same element of every other rank's y, over NVLink
            for (int g = 0; g < po.n; ++g) store_y<YT>(reinterpret_cast<YT*>(reinterpret_cast<char*>(dst) + po.delta[g]), v[k]);
        }
    }
}

template <typename YT>
__global__ void __launch_bounds__(TC_MAX_THREADS, 1)
qlinear_i8_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                     const __grid_constant__ TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // carve: [A stages][B stages][barriers]
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int b_stage_bytes = p.NB * BK;
    const int a_stage_bytes = p.tpu * A_TILE_BYTES;
    uint8_t* sA = smem;
    uint8_t* sB = smem + (size_t)p.stages * a_stage_bytes;
    // epilogue staging of a whole tile's folded sums: [Mpad/2][128] x 16 bytes
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
#ifdef RUSTY_TIMELINE
    if (threadIdx.x == 0 && p.dbg) {
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        p.dbg[(size_t)blockIdx.x * 16 + 12] = (long long)smid;
    }
#endif
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], (uint32_t)p.epi_warps);
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
                        mbar_expect_tx(&full[early], (uint32_t)(a_stage_bytes + b_stage_bytes));
                        tma_load_2d(sA + (size_t)early * a_stage_bytes, &map_w, kb * BK, sg.t * p.bmu, &full[early], pol_w);
                        early_kb[early] = kb;
                        ++early;
                        ++issued;
                        if (issued == 1) DBG(2);
                        if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                        continue;
                    }
                    if (!waited) {
                        pdl_wait();
                        DBG(1);
                        for (int e = 0; e < early; ++e)
                            tma_load_2d(sB + (size_t)e * b_stage_bytes, &map_x, early_kb[e] * BK, 0, &full[e], pol_x);
                        waited = true;
                    }
                    if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
                    mbar_expect_tx(&full[stage], (uint32_t)(a_stage_bytes + b_stage_bytes));
                    tma_load_2d(sA + (size_t)stage * a_stage_bytes, &map_w, kb * BK, sg.t * p.bmu, &full[stage], pol_w);
                    tma_load_2d(sB + (size_t)stage * b_stage_bytes, &map_x, kb * BK, 0, &full[stage], pol_x);
                    ++issued;
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!waited) {  // fewer k-blocks than ring slots
                pdl_wait();
                DBG(1);
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
                const uint32_t d_tmem = tmem_base + (uint32_t)(ab * p.tpu * p.NB);   // accumulator h of the unit at + h * NB
                for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
                    if (!mbar_wait(&full[stage], phase, abort_flag, p.status, 3)) { ok = false; break; }
                    tc_fence_after();
                    if (kb == sg.kb0 && i == 0) DBG(4);
                    const uint64_t da = make_smem_desc(smem_u32(sA + (size_t)stage * a_stage_bytes));
                    const uint64_t db = make_smem_desc(smem_u32(sB + (size_t)stage * b_stage_bytes));
                    for (int h = 0; h < p.tpu; ++h) {   // the unit's weight tiles, 16 KiB (1024 x 16 bytes) apart, against the same digit tile
#pragma unroll
                        for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
                            // advance 32 bytes along K inside the 128-byte swizzle atom: +2 in 16-byte units
                            umma_i8(d_tmem + (uint32_t)(h * p.NB), da + (uint64_t)(h * (A_TILE_BYTES >> 4) + 2 * k4), db + (uint64_t)(2 * k4), p.idesc,
                                    (kb > sg.kb0 || k4 > 0) ? 1u : 0u);
                        }
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
        pdl_wait();                             // x, y and the piece slots belong to earlier kernels until now
        bool ok = true;
        const int et = threadIdx.x - 64;        // 0..EPI_THREADS-1 among the epilogue threads
        const int EPI_THREADS = 32 * p.epi_warps;
        // Two warps share a lane quarter (warps 2-5 and 6-9 see the same quarters): each takes half of the activation
        // rows, in units of 8.  With 4 epilogue warps every warp takes them all.
        const int m_split = p.epi_warps == 8 ? ((p.Mpad / 8 + 1) / 2) * 8 : p.Mpad;
        const int m_lo = (warp - 2) < 4 ? 0 : m_split, m_hi = (warp - 2) < 4 ? m_split : p.Mpad;
        // per-row factors of the pre-pass: once into shared memory (a load from global memory per output costs
        // an L2 round trip each time)
        if (et < p.Mpad) s_rowf[et] = __ldcg(p.row_factor + et);
        asm volatile("bar.sync 1, %0;" ::"r"(EPI_THREADS) : "memory");
        int cut_t[2], cut_j[2], cut_n[2], cut_f[2], n_cut = 0;  // shared tiles this CTA holds a piece of
        Sched sched(p);
        Segment sg;
        for (int i = 0;; ++i) {
            const bool have = ok && sched.next(sg);
            // Shared tiles.  Every CTA that holds a piece of a tile has written it into its own slot, each 64-bit sum
            // tagged valid in its lowest bit; after its last segment a piece holder gathers an equal share of the tile's
            // rows from ALL the tile's slots (polling words that are still zero), turns it into y and leaves zeros
            // behind.  No counters, no fences: a word carries its own arrival.  The CTAs of the grid are resident
            // together (one wave) and every piece is written before its holder waits here, so a wait cannot depend
            // on a CTA that has not started.
            for (int e = 0; ok && e < n_cut && !have; ++e) {
                const int t = cut_t[e], nseg = cut_n[e], j = cut_j[e], fcta = cut_f[e];
                const int lt = t - p.dp_tiles;
                const size_t slot_items = (size_t)p.tpu * (p.Mpad / 2) * BM;   // a slot: [tile of the unit][m / 2][row] x 16 bytes
                // this CTA's share of the tile's rows, cut in units of two rows so that a (gate, up) pair stays together
                const int lo = 2 * (j * (p.bmu / 2) / nseg), rows = 2 * ((j + 1) * (p.bmu / 2) / nseg) - lo;
                const int items = rows * (p.Mpad / 2);                         // one item: a row, two activation rows
                if (rows <= 0) continue;
                // item -> (row, mp) without a division per item: start at (et % rows, et / rows), step by EPI_THREADS items
                int row = et % rows, mp = et / rows;
                const int step_row = EPI_THREADS % rows, step_mp = EPI_THREADS / rows;
                const long long t_begin = clock64();
                // the loop bounds are the same for every thread: the pair epilogue needs whole warps
                for (int base = 0; base < items; base += 4 * EPI_THREADS) {
                    const int it0 = base + et;
                    long long s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0};
                    size_t off[4];
                    int rw[4], mq[4];
                    bool in[4];
                    float wsc[4];   // the rows' weight scales: fetched with the pieces, not behind them
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        rw[u] = lo + row;
                        mq[u] = mp;
                        in[u] = it0 + u * EPI_THREADS < items;
                        off[u] = ((size_t)(rw[u] >> 7) * (p.Mpad / 2) + mp) * BM + (rw[u] & 127);
                        wsc[u] = (in[u] && t * p.bmu + rw[u] < p.N) ? __ldg(p.scales + t * p.bmu + rw[u]) : 0.0f;
                        row += step_row;
                        mp += step_mp;
                        if (row >= rows) {
                            row -= rows;
                            ++mp;
                        }
                    }
#pragma unroll 1
                    for (int q0 = 0; q0 < nseg; q0 += 4) {   // four pieces x four items: sixteen loads in flight per trip
                        ulonglong2* slot[4];
                        ulonglong2 v[4][4];
#pragma unroll
                        for (int w = 0; w < 4; ++w) {
                            // piece q of the tile sits with CTA fcta + q: its head piece (even slot) if that CTA's run
                            // of k-blocks starts inside this tile, else its tail piece (odd slot)
                            const int c = fcta + min(q0 + w, nseg - 1);
                            slot[w] = p.part + (size_t)(2 * c + (c * p.sk_per_cta >= lt * p.kb_total ? 0 : 1)) * slot_items;
#pragma unroll
                            for (int u = 0; u < 4; ++u)
                                v[w][u] = (in[u] && q0 + w < nseg) ? __ldcg(slot[w] + off[u]) : make_ulonglong2(1ull, 1ull);
                        }
                        // every word carries its own "valid" tag in bit 0: one combined test for the common case ...
                        unsigned long long allv = 1ull;
#pragma unroll
                        for (int w = 0; w < 4; ++w)
#pragma unroll
                            for (int u = 0; u < 4; ++u) allv &= v[w][u].x & v[w][u].y;
                        // ... and a rolled re-poll of the whole batch while some piece has not landed yet
                        while (!(allv & 1ull)) {
                            if (*abort_flag || clock64() - t_begin > WAIT_LIMIT_CYCLES) {
                                *abort_flag = 1;
                                if (atomicExch(&p.status->timeout_flag, 1u) == 0u) p.status->timeout_where = 8;
                                ok = false;
                                break;
                            }
                            allv = 1ull;
#pragma unroll
                            for (int w = 0; w < 4; ++w)
#pragma unroll
                                for (int u = 0; u < 4; ++u) {
                                    if (in[u] && q0 + w < nseg) v[w][u] = __ldcg(slot[w] + off[u]);
                                    allv &= v[w][u].x & v[w][u].y;
                                }
                        }
#pragma unroll
                        for (int w = 0; w < 4; ++w) {
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                if (in[u] && q0 + w < nseg) __stcg(slot[w] + off[u], make_ulonglong2(0ull, 0ull));
                                s0[u] += (long long)v[w][u].x >> 1;   // arithmetic shift: drops the tag, keeps the sign
                                s1[u] += (long long)v[w][u].y >> 1;
                            }
                        }
                    }
                    if (__any_sync(0xffffffffu, !ok)) {   // warp-uniform: the conversion below shuffles between lanes
                        ok = false;
                        break;
                    }
#pragma unroll
                    for (int u = 0; u < 4; u += 2) {  // two items = four outputs per trip
                        const bool v0 = in[u] && t * p.bmu + rw[u] < p.N, v1 = in[u + 1] && t * p.bmu + rw[u + 1] < p.N;
                        const int n0 = t * p.bmu + rw[u], n1 = t * p.bmu + rw[u + 1];
                        const int m0 = v0 ? 2 * mq[u] : 0, m1 = v1 ? 2 * mq[u + 1] : 0;
                        const long long a4[4] = {s0[u], s1[u], s0[u + 1], s1[u + 1]};
                        const int n4[4] = {n0, n0, n1, n1}, m4[4] = {m0, m0 + 1, m1, m1 + 1};
                        const float s4[4] = {wsc[u], wsc[u], wsc[u + 1], wsc[u + 1]};
                        const bool l4[4] = {v0 && m0 < p.M, v0 && m0 + 1 < p.M, v1 && m1 < p.M, v1 && m1 + 1 < p.M};
                        finalize_store4<YT>(p, y, n4, m4, a4, s4, s_rowf, po, l4);
                    }
                }
                if (threadIdx.x == 64) DBG(11);
            }
            if (__any_sync(0xffffffffu, !ok)) ok = false;
            if (!have || !ok) break;
            const int ab = i & 1;
            if (!mbar_wait(&acc_full[ab], ((uint32_t)i >> 1) & 1u, abort_flag, p.status, 4)) { ok = false; break; }
            tc_fence_after();
            if (threadIdx.x == 64) DBG(6 + 4 * (i & 1));
            {
                // Fold the digit planes into one exact 64-bit integer per output.  A whole tile is staged in shared
                // memory ([m/2][row] x 16 bytes) and converted from there in a rolled loop (unrolled register code
                // that runs once per tile costs an instruction fetch per line and was twice as slow); a piece of a
                // shared tile goes straight into this CTA's slot in global memory, every word tagged valid.
                const bool whole = sg.nseg == 1;
                for (int ht = 0; ht < p.tpu; ++ht) {   // the unit's tiles, one accumulator each
                    const int n = sg.t * p.bmu + ht * BM + r;
                    const bool row_ok = n < p.N;
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((ab * p.tpu + ht) * p.NB);
                    ulonglong2* slot = p.part + ((size_t)sg.slot * p.tpu + ht) * (p.Mpad / 2) * BM;
                    for (int m0 = m_lo; m0 < m_hi; m0 += 8) {
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
                            if (whole) {
                                int4 v;
                                v.x = (int)(a0 & 0xffffffffll);
                                v.y = (int)(a0 >> 32);
                                v.z = (int)(a1 & 0xffffffffll);
                                v.w = (int)(a1 >> 32);
                                stage_red[(size_t)(m0 / 2 + h) * BM + r] = v;
                            } else {   // |sum| < 2^46: room for the tag; two 64-bit words, each stored whole
                                __stcg(slot + (size_t)(m0 / 2 + h) * BM + r,
                                       make_ulonglong2((unsigned long long)((a0 << 1) | 1), (unsigned long long)((a1 << 1) | 1)));
                            }
                        }
                    }
                    if (ht == p.tpu - 1) {   // the accumulators of this unit have been read
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[ab]);
                        if (threadIdx.x == 64) DBG(7 + 4 * (i & 1));
                    }
                    if (whole) {
                        // every thread reads back only what it staged itself: no barrier needed
                        const float sc = row_ok ? __ldg(p.scales + n) : 0.0f;
#pragma unroll 1
                        for (int m = m_lo; m < min(m_hi, p.M); m += 4) {  // in units of 8: the staged rows m .. m+3 exist
                            const longlong2 t0 = *reinterpret_cast<const longlong2*>(&stage_red[(size_t)(m >> 1) * BM + r]);
                            const longlong2 t1 = *reinterpret_cast<const longlong2*>(&stage_red[(size_t)((m >> 1) + 1) * BM + r]);
                            const long long a4[4] = {t0.x, t0.y, t1.x, t1.y};
                            const int n4[4] = {n, n, n, n}, m4[4] = {m, m + 1, m + 2, m + 3};
                            const float s4[4] = {sc, sc, sc, sc};
                            const bool l4[4] = {row_ok, row_ok && m + 1 < p.M, row_ok && m + 2 < p.M, row_ok && m + 3 < p.M};
                            finalize_store4<YT>(p, y, n4, m4, a4, s4, s_rowf, po, l4);
                        }
                    }
                }
                if (whole) {
                    if (threadIdx.x == 64) DBG(9 + 4 * (i & 1));
                    continue;
                }
                // The conversion is shared between the CTAs that hold the tile's pieces and is done after the CTA's
                // last segment (above): remember the tile and which piece this was.
                if (n_cut < 2) {
                    cut_t[n_cut] = sg.t;
                    cut_j[n_cut] = (int)blockIdx.x - sg.first_cta;
                    cut_n[n_cut] = sg.nseg;
                    cut_f[n_cut] = sg.first_cta;
                    ++n_cut;
                } else {
                    ok = false;  // cannot happen: a run of k-blocks starts and ends inside at most two shared tiles
                    if (threadIdx.x == 64 && atomicExch(&p.status->timeout_flag, 1u) == 0u) p.status->timeout_where = 7;
                }
                if (threadIdx.x == 64) DBG(8 + 4 * (i & 1));
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
    if (threadIdx.x == 0) DBG(15);
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
constexpr size_t WS_ACC_BYTES = 48u << 20;     // pieces of K-cut tiles (two slots per CTA), zero between launches
constexpr size_t WS_CNT_BYTES = 64u << 10;     // arrival counters of the prefill kernels, kept at zero between kernels
constexpr size_t WS_OFF_XQ = 0;
constexpr size_t WS_OFF_INVS = WS_OFF_XQ + WS_XQ_BYTES + WS_GUARD;
constexpr size_t WS_OFF_ACC = WS_OFF_INVS + WS_INVS_BYTES + WS_GUARD;
constexpr size_t WS_OFF_CNT = WS_OFF_ACC + WS_ACC_BYTES + WS_GUARD;
constexpr size_t WS_TOTAL = WS_OFF_CNT + WS_CNT_BYTES + WS_GUARD;
constexpr int WS_GUARDS = 4;
constexpr size_t WS_GUARD_AT[WS_GUARDS] = {WS_OFF_INVS - WS_GUARD, WS_OFF_ACC - WS_GUARD, WS_OFF_CNT - WS_GUARD, WS_TOTAL - WS_GUARD};

// The schedule of one launch: how the row tiles are dealt to the CTAs.  One place for the regular entry points and the
// entry point with built-in scratch, so that their guards cannot drift apart.
//   whole tiles (tile = cta, cta + grid, ...) for the first dp_tiles tiles; the last sk_tiles tiles are cut along K.
// `slots_cap`: how many piece slots (two per CTA) the caller's scratch holds; a launch that would need more takes
// whole tiles only.
struct TcSchedule {
    int grid, dp_tiles, sk_tiles, sk_per_cta, sk_ctas, sk_ways;
};
void plan_tc_schedule(int tiles, int kb_total, int sm_count, int dp_percent, size_t slots_cap, TcSchedule* out) {
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
        if ((size_t)2 * s.sk_ctas > slots_cap) {
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
}

int pick_digits(int x_dtype, uint32_t rows) {
    // f32 activations: 4 planes = 28 bits below the row maximum.  Three planes (21 bits) hold the fp32 tolerance only
    // while the row's largest element stays within ~25x of its rms: with one outlier of 1000x every other element
    // keeps 11 bits and the result is ~5e-5 off.  bf16 activations carry 8 significant bits each: 3 planes.
    (void)rows;
    return x_dtype == RUSTY_CUDA_F32 ? 4 : 3;
}

template <typename XT>
cudaError_t launch_digitize(cudaStream_t stream, const void* x, int8_t* xq, float* inv_s, int M, int Mpad, int K, int D, const PeerPush& push,
                            long long* dbg, const NormArgs* norm = nullptr) {
    // Mpad is a multiple of 8 and at most 64: one row per block up to 32 rows, two beyond
    int R = 1;
    while (Mpad / R > DIG_MAX_BLOCKS || Mpad % R != 0) R <<= 1;   // R in {1, 2}: the rows' thread groups share a block evenly
    const int blocks = Mpad / R;
    if constexpr (std::is_same<XT, float>::value) {
        if (norm) {
            if (D == 4)
                return launch_pdl(digitize_x_kernel<XT, 4, true>, dim3(blocks), dim3(DIG_THREADS), 0, stream, (const XT*)x, xq, inv_s, M, Mpad, K, R, push, *norm, dbg);
            return launch_pdl(digitize_x_kernel<XT, 3, true>, dim3(blocks), dim3(DIG_THREADS), 0, stream, (const XT*)x, xq, inv_s, M, Mpad, K, R, push, *norm, dbg);
        }
    }
    if (D == 4)
        return launch_pdl(digitize_x_kernel<XT, 4, false>, dim3(blocks), dim3(DIG_THREADS), 0, stream, (const XT*)x, xq, inv_s, M, Mpad, K, R, push, NormArgs{}, dbg);
    return launch_pdl(digitize_x_kernel<XT, 3, false>, dim3(blocks), dim3(DIG_THREADS), 0, stream, (const XT*)x, xq, inv_s, M, Mpad, K, R, push, NormArgs{}, dbg);
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
    for (size_t g = 0; e == cudaSuccess && g < (size_t)WS_GUARDS; ++g) e = cudaMemsetAsync((uint8_t*)p + WS_GUARD_AT[g], WS_GUARD_BYTE, WS_GUARD, ctx->stream);
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
    for (int g = 0; g < (size_t)WS_GUARDS; ++g) {
        *err = cudaMemcpyAsync(host.data(), (uint8_t*)ctx->tc_ws + WS_GUARD_AT[g], WS_GUARD, cudaMemcpyDeviceToHost, ctx->stream);
        if (*err == cudaSuccess) *err = cudaStreamSynchronize(ctx->stream);
        if (*err != cudaSuccess) return -1;
        for (size_t i = 0; i < WS_GUARD; ++i)
            if (host[i] != WS_GUARD_BYTE) return g;
    }
    return -1;
}

// After a device-side wait gave up, pieces of K-cut tiles may be left in their slots: clear them, so that the next
// launch starts from zeros again.
void tc_workspace_clear_pieces(rusty_cuda_ctx* ctx) {
    if (!ctx->tc_ws) return;
    if (cudaMemsetAsync((uint8_t*)ctx->tc_ws + WS_OFF_ACC, 0, WS_ACC_BYTES, ctx->stream) == cudaSuccess) cudaStreamSynchronize(ctx->stream);
    cudaGetLastError();
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

// The pre-pass normalises a row held in registers: 8 x 4 activations per thread, 512 threads a row up to 32 rows and
// 256 beyond (two rows share a block).
bool tc_norm_fused(uint32_t M, uint32_t K) {
    if (M < (uint32_t)tc_min_rows()) return false;
    const uint32_t Mpad = (M + 7u) & ~7u;
    const uint32_t threads_per_row = Mpad > (uint32_t)DIG_MAX_BLOCKS ? DIG_THREADS / 2 : DIG_THREADS;
    return K % 4 == 0 && K <= (uint32_t)DIG_MAXV * 4u * threads_per_row;
}

// One launch pair (digitise + GEMM) for up to 64 activation rows.
static int launch_tc_rows(rusty_cuda_ctx* ctx, const QLinearArgs& a, const void* x, void* y, uint32_t rows, const NormArgs* norm) {
    const int M = (int)rows, Mpad = (M + 7) / 8 * 8;
    const int D = pick_digits(a.x_dtype, rows);
    const int NB = (D * Mpad + 15) / 16 * 16;
    uint8_t* ws = (uint8_t*)ctx->tc_ws;
    int8_t* xq = (int8_t*)ws;
    float* inv_s = (float*)(ws + WS_OFF_INVS);
    ulonglong2* acc = (ulonglong2*)(ws + WS_OFF_ACC);
    if ((size_t)D * Mpad * a.K > WS_XQ_BYTES)
        return fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "tensor-core path: %d digit rows x K=%u exceed the workspace", D * Mpad, a.K);

    cudaError_t le = cudaSuccess;
    int rc = RUSTY_CUDA_OK;
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
    PeerPush push_pre = push;
#ifdef RUSTY_TIMELINE
    {   // development aid: take the exchange apart (1: no meeting of the ranks, 2: no stores into the other ranks)
        static const int exp_mode = getenv("RUSTY_PEER_EXP") ? atoi(getenv("RUSTY_PEER_EXP")) : 0;
        if (exp_mode & 1) push_pre = PeerPush{};
        if (exp_mode & 2) push = PeerPush{};
    }
#endif
    {
        if (norm && (a.x_dtype != RUSTY_CUDA_F32 || !tc_norm_fused(a.M, a.K)))
            return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward: the norm cannot be applied by this call's pre-pass");
        le = a.x_dtype == RUSTY_CUDA_BF16 ? launch_digitize<__nv_bfloat16>(ctx->stream, x, xq, inv_s, M, Mpad, (int)a.K, D, push_pre, dbg ? dbg + 150 * 16 : nullptr)
                                          : launch_digitize<float>(ctx->stream, x, xq, inv_s, M, Mpad, (int)a.K, D, push_pre, dbg ? dbg + 150 * 16 : nullptr, norm);
        if (le != cudaSuccess) return check_cuda(ctx, le, "digitize_x");
        rc = after_launch(ctx, "digitize_x");
        if (rc) return rc;
    }

    TcParams p{};
    p.scales = a.scales;
    p.row_factor = inv_s;
    p.part = acc;
    p.y = y;
    p.M = M;
    p.Mpad = Mpad;
    p.D = D;
    p.NB = NB;
    p.N = (int)a.N;
    p.K = (int)a.K;
    // Two row tiles per work unit while both accumulator pairs fit tensor memory (4 * NB <= 512 columns): every
    // digit tile a CTA loads then multiplies 256 weight rows instead of 128, which takes a quarter off the bytes a
    // CTA pulls from L2 (the digits are re-read by every row tile; the weights are not).  Only where the units are
    // then taken whole: a unit's epilogue is twice a tile's, which cut units (whose pieces cross CTAs after the
    // stream) cannot afford.  Measured on batch 32: gate|up 31.9 -> 29.9 us, LM head 98.1 -> 95.9 us; with cut units
    // the whole stack loses 6 %.  RUSTY_TC_TWO_TILES = 0 / 1 / 2: never / by that rule / always (tuning aid).
    static const int two_tiles = getenv("RUSTY_TC_TWO_TILES") ? atoi(getenv("RUSTY_TC_TWO_TILES")) : 1;
    // RUSTY_TC_DP_PERCENT: least share of the SMs that whole tiles must keep streaming (default 72; 101 turns the rule off).
    static const int dp_percent = getenv("RUSTY_TC_DP_PERCENT") ? atoi(getenv("RUSTY_TC_DP_PERCENT")) : 72;
    p.kb_total = (p.K + BK - 1) / BK;
    TcSchedule sc{};
    p.tpu = 1;
    if (two_tiles > 0 && 4 * NB <= 512 && a.N > (uint32_t)BM) {
        const int units = (p.N + 2 * BM - 1) / (2 * BM);
        plan_tc_schedule(units, p.kb_total, ctx->sm_count, dp_percent, WS_ACC_BYTES / ((size_t)2 * Mpad * BM * 8), &sc);
        if (two_tiles >= 2 || sc.sk_tiles == 0) p.tpu = 2;
    }
    p.bmu = p.tpu * BM;
    p.tiles = (p.N + p.bmu - 1) / p.bmu;
    int sched_sms = ctx->sm_count;
    {   // tuning aid: schedule as if the GPU had fewer SMs
        static const int sms_env = getenv("RUSTY_TC_SMS") ? atoi(getenv("RUSTY_TC_SMS")) : 0;
        if (sms_env > 0 && sms_env < sched_sms) sched_sms = sms_env;
    }
    plan_tc_schedule(p.tiles, p.kb_total, sched_sms, dp_percent, WS_ACC_BYTES / ((size_t)p.tpu * Mpad * BM * 8), &sc);
    // A GEMM CTA and a pre-pass block do not fit one SM together (registers), and the NEXT pair's pre-pass blocks are
    // resident (two per SM, up to 16 SMs) while this GEMM's CTAs are placed.  A short launch whose every tile is cut
    // (fewer tiles than SMs) and whose grid leaves those SMs no room gets its last CTAs placed only after the pre-pass
    // has finished, 2-5 us late: plan it for 16 SMs fewer (q|k|v 6144 x 4096: 144 -> 96 CTAs, 18.2 -> 16.8 us).
    // RUSTY_TC_ROOM=0 turns the rule off (tuning aid).
    static const bool leave_room = !(getenv("RUSTY_TC_ROOM") && atoi(getenv("RUSTY_TC_ROOM")) == 0);
    if (leave_room && sc.dp_tiles == 0 && sc.grid > sched_sms - 16 && sched_sms > 32) {
        TcSchedule alt{};
        plan_tc_schedule(p.tiles, p.kb_total, sched_sms - 16, dp_percent, WS_ACC_BYTES / ((size_t)p.tpu * Mpad * BM * 8), &alt);
        if (alt.dp_tiles == 0) sc = alt;
    }
    int grid = sc.grid;
    p.dp_tiles = sc.dp_tiles;
    p.sk_tiles = sc.sk_tiles;
    p.sk_per_cta = sc.sk_per_cta;
    p.sk_ctas = sc.sk_ctas;
    p.sk_ways = sc.sk_ways;
    p.ldy = (int)a.ldy;
    p.y_col0 = (int)a.y_col0;
    p.residual = a.residual ? (const char*)a.residual + ((const char*)y - (const char*)a.y) : nullptr;   // this pass's rows
    p.act = a.act;
    {
        // narrow batches keep the small CTA (two of them fit an SM: the next kernel's CTA prefetches beside this one);
        // from 16 rows on the epilogue is what bounds the kernel and gets eight warps
        static const bool four = getenv("RUSTY_TC_EPI4") != nullptr;   // tuning aid
        p.epi_warps = (Mpad >= 16 && !four) ? 8 : 4;
    }
    p.status = ctx->status_dev;
    p.dbg = dbg;
    p.push = push;
    // int8 x int8 -> int32, both K-major: c_format=S32(2)@4, a_format=INT8(1)@7, b_format=INT8(1)@10, N>>3 @17, M>>4 @24
    p.idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    uint32_t cols = 32;
    while (cols < (uint32_t)(2 * p.tpu * NB)) cols <<= 1;   // two sets of accumulators: the epilogue of one unit overlaps the next
    p.tmem_cols = cols;
    const int a_stage = p.tpu * A_TILE_BYTES, b_stage = NB * BK;
    // Half of the SM's shared memory at most for narrow batches, so that the next kernel's CTA can move in beside this
    // one and prefetch its weights while this one drains (RUSTY_TC_FULL_SMEM=1: take it all, 8 stages).
    static const bool full_smem = getenv("RUSTY_TC_FULL_SMEM") != nullptr;
    size_t budget = ctx->smem_optin > 4096 ? ctx->smem_optin - 4096 : 0;
    if (!full_smem && NB <= 32 && 4 * (size_t)a_stage + 4096 <= budget / 2)
        budget = budget / 2 - 1024;  // narrow batches: leave room for the next kernel's CTA on the SM
    // epilogue staging of one whole 128-row tile (its folded sums); launches without whole tiles need none
    const size_t red_bytes = p.dp_tiles > 0 ? (size_t)Mpad * 8 * BM : 0;
    int stages = budget > red_bytes + 2048 ? (int)((budget - 1024 - 512 - red_bytes) / (size_t)(a_stage + b_stage)) : 0;
    if (stages > 8) stages = 8;
    if (stages < 2) return fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "tensor-core path: tile does not fit shared memory");
    p.stages = stages;
    p.red_bytes = (int)red_bytes;
    const size_t smem = 1024 + (size_t)stages * (a_stage + b_stage) + red_bytes + (size_t)(2 * stages + 4) * 8 + 256;

    CUtensorMap map_w, map_x;
    if (!make_map_u8(&map_w, a.w, a.N, a.K, (uint32_t)p.bmu) ||
        !make_map_u8(&map_x, xq, (uint64_t)D * Mpad, a.K, (uint32_t)NB))
        return fail(ctx, RUSTY_CUDA_ERR_KERNEL_EXECUTION, "tensor-core path: cuTensorMapEncodeTiled failed");

    const bool yb = a.y_dtype == RUSTY_CUDA_BF16;

    auto kern = yb ? qlinear_i8_tc_kernel<__nv_bfloat16> : qlinear_i8_tc_kernel<float>;
    {
        cudaError_t e = ensure_dynamic_smem((const void*)kern, ctx->device, smem);
        if (e != cudaSuccess) return check_cuda(ctx, e, "qlinear_i8_tc: cudaFuncSetAttribute");
    }
    le = launch_pdl(kern, dim3(grid), dim3(64 + 32 * p.epi_warps), smem, ctx->stream, map_w, map_x, p);
    if (le != cudaSuccess) return check_cuda(ctx, le, "qlinear_i8_tc");
    return after_launch(ctx, "qlinear_i8_tc");
}

int launch_tc(rusty_cuda_ctx* ctx, const QLinearArgs& a) {
    const size_t xs = a.x_dtype == RUSTY_CUDA_BF16 ? 2 : 4, ys = a.y_dtype == RUSTY_CUDA_BF16 ? 2 : 4;
    for (uint32_t m0 = 0; m0 < a.M; m0 += 64) {
        uint32_t rows = a.M - m0 < 64 ? a.M - m0 : 64;
        NormArgs nrm{};
        if (a.norm) {   // this pass's rows of the norm's operands
            nrm = *a.norm;
            const size_t off = (size_t)m0 * a.K;
            if (nrm.residual) nrm.residual += off;
            if (nrm.normed) nrm.normed += off;
            if (nrm.sum) nrm.sum += off;
        }
        int rc = launch_tc_rows(ctx, a, (const char*)a.x + (size_t)m0 * a.K * xs, (char*)a.y + (size_t)m0 * a.ldy * ys, rows, a.norm ? &nrm : nullptr);
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
// activations, per-row factors, slots for the pieces of K-cut tiles, status
// word) lives in the fixed array below, which every GPU that loads this library
// holds until the process exits.
// ----------------------------------------------------------------------------
namespace {

constexpr uint32_t STATIC_MAX_ROWS = 8;       // activation rows per call
constexpr uint32_t STATIC_MAX_K = 8192;       // input features
constexpr uint32_t STATIC_MAX_N = 262144;     // output features (a stated bound; 2048 row tiles)
constexpr int STATIC_MAX_CTAS = 160;          // CTAs launched at most (one per SM)
constexpr size_t ST_XQ_BYTES = (size_t)4 * 8 * STATIC_MAX_K;            // 4 digit planes x 8 padded rows
constexpr size_t ST_FACTOR_BYTES = 256;
constexpr size_t ST_SLOTS = 2 * STATIC_MAX_CTAS;                         // pieces of K-cut tiles: a head and a tail slot per CTA
constexpr size_t ST_SUMS_BYTES = ST_SLOTS * 8 * 8 * BM;                 // one 8-row piece (tagged int64) per slot
constexpr size_t ST_STATUS_BYTES = 256;
constexpr size_t ST_TOTAL = ST_XQ_BYTES + ST_FACTOR_BYTES + ST_SUMS_BYTES + ST_STATUS_BYTES;  // ~2.8 MiB
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
    unsigned char* zeroed = sd.base + ST_XQ_BYTES + ST_FACTOR_BYTES;  // piece slots and status: must start at zero
    ulonglong2* sums = (ulonglong2*)zeroed;
    rusty_cuda_dev_status* status = (rusty_cuda_dev_status*)(zeroed + ST_SUMS_BYTES);
    e = cudaMemsetAsync(zeroed, 0, ST_SUMS_BYTES + ST_STATUS_BYTES, st);
    if (e != cudaSuccess) return check_cuda(nullptr, e, "qlinear_i8_forward_static: clearing the scratch");

    const int Mi = (int)M, Mpad = 8, D = 4, NB = 32;
    e = launch_digitize<float>(st, x_f32, xq, factor, Mi, Mpad, (int)K, D, PeerPush{}, nullptr);
    if (e != cudaSuccess) return check_cuda(nullptr, e, "qlinear_i8_forward_static: digitize_x");

    TcParams p{};
    p.scales = scales;
    p.row_factor = factor;
    p.part = sums;
    p.y = y_f32;
    p.M = Mi;
    p.Mpad = Mpad;
    p.D = D;
    p.NB = NB;
    p.N = (int)N;
    p.K = (int)K;
    p.tpu = 1;
    p.bmu = BM;
    p.tiles = (p.N + BM - 1) / BM;
    p.kb_total = (p.K + BK - 1) / BK;
    // the same schedule rules as the regular entry points, with this scratch's capacities
    TcSchedule sc{};
    plan_tc_schedule(p.tiles, p.kb_total, sd.sm_count < STATIC_MAX_CTAS ? sd.sm_count : STATIC_MAX_CTAS, /*dp_percent=*/72, ST_SLOTS, &sc);
    const int grid = sc.grid;
    p.dp_tiles = sc.dp_tiles;
    p.sk_tiles = sc.sk_tiles;
    p.sk_per_cta = sc.sk_per_cta;
    p.sk_ctas = sc.sk_ctas;
    p.sk_ways = sc.sk_ways;
    p.ldy = (int)N;
    p.y_col0 = 0;
    p.epi_warps = 4;
    p.status = status;
    p.dbg = nullptr;
    p.idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    p.tmem_cols = 64;
    const int b_stage = NB * BK;
    const size_t red_bytes = (size_t)Mpad * 8 * BM > 12288 ? (size_t)Mpad * 8 * BM : (size_t)12288;
    const size_t budget = (sd.smem_optin > 4096 ? sd.smem_optin - 4096 : 0) / 2;
    int stages = budget > red_bytes + 4096 ? (int)((budget - 2048 - red_bytes) / (size_t)(A_TILE_BYTES + b_stage)) : 0;
    if (stages > 8) stages = 8;
    if (stages < 2) return fail(nullptr, RUSTY_CUDA_ERR_UNSUPPORTED, "qlinear_i8_forward_static: shared memory too small");
    p.stages = stages;
    p.red_bytes = (int)red_bytes;
    const size_t smem = 1024 + (size_t)stages * (A_TILE_BYTES + b_stage) + red_bytes + (size_t)(2 * stages + 4) * 8 + 256;
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
    e = launch_pdl(kern, dim3(grid), dim3(64 + 32 * p.epi_warps), smem, st, map_w, map_x, p);
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
    e = cudaMemcpyAsync(&h, base + ST_XQ_BYTES + ST_FACTOR_BYTES + ST_SUMS_BYTES, sizeof(h), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return check_cuda(nullptr, e, "qlinear_i8_static_status");
    return static_status_to_code(h.timeout_flag, h.timeout_where);
}

// Host-side decoding of the status word, exposed for tests that have no GPU.
extern "C" RUSTY_CUDA_API int rusty_cuda_qlinear_i8_static_status_decode(unsigned int timeout_flag, unsigned int timeout_where) {
    return static_status_to_code(timeout_flag, timeout_where);
}

