// Prefill GEMM over int8 weights on tcgen05 / TMEM with bf16 operands.
//
// Replaces, for many activation rows at once, the reference's "dequantise once
// at load, f32 tiled matmul per forward" (rusty-loader/src/lib.rs:155-218,
// rusty-backend/src/kernels.wgsl:16-54, :234-242):
//     y[m,n] = scale[n] * sum_k x[m,k] * q[n,k]        x bf16, q int8, fp32 accumulation
//
// The weight rows are the M side of the MMA (128 rows per tile), the activation
// rows the N side (up to 256 per tile), so the accumulator tile is y^T.
//   * int8 weight tiles (128 rows x 128 k, 16 KB) arrive by TMA with the 128-byte
//     swizzle; four converter warps (one thread per weight row) read their row
//     conflict-free, turn bytes into bf16 pairs (byte-permute into the mantissa of
//     2^23, subtract, packed convert: exact since |q| <= 128), and write them
//     straight into TENSOR MEMORY with tcgen05.st — the A operand never goes back
//     through shared memory;
//   * bf16 activation tiles (up to 256 rows x 64 k) arrive by TMA as the B operand;
//   * one elected thread issues tcgen05.mma kind::f16 (A bf16 from TMEM, B bf16
//     from shared memory, fp32 accumulators in TMEM); bf16 x bf16 products are
//     exact in the fp32 accumulate, so the only rounding is the summation;
//   * four epilogue warps read the accumulators, apply the per-row weight scale and
//     store y (bf16 or f32) while the converters already work on the next tile.
// Persistent CTAs, one per SM; every mbarrier wait is bounded.
#include <cstdlib>
#include <cstring>

#include "tc_common.cuh"

using namespace rusty_tc;

namespace {

constexpr int BM = 128;          // weight rows per tile (UMMA M)
constexpr int WK = 128;          // k per weight stage (bytes per row)
constexpr int XK = 64;           // k per activation stage (128 bytes of bf16 per row)
constexpr int W_STAGES = 3;
constexpr int A_BUFS = 3;        // converted-weight buffers in tensor memory, 64 columns each
constexpr int A_COLS = WK / 2;   // two 16-bit values per 32-bit column
constexpr int D_COLS = 256;      // accumulator columns reserved
constexpr int CONV_WARPS = 8;     // two per TMEM lane quarter, each takes half of a stage's k range
constexpr int EPI_WARPS = 8;      // two per TMEM lane quarter, each drains half of the accumulator's columns: the
                                  // accumulator is single-buffered, so the drain holds up the next tile's first MMA
constexpr int F16_THREADS = 32 * (2 + CONV_WARPS + EPI_WARPS);  // producer, MMA, converter and epilogue warps
constexpr int W_STAGE_BYTES = BM * WK;

struct F16Params {
    const float* scales;  // SYM_ROW: [N], applied to the sums; AFFINE_G64: [N*K/64], applied to the weights as they are converted
    const float* biases;  // AFFINE_G64: [N*K/64]; null selects SYM_ROW
    void* y;
    int Mx, N, K;
    int BN;               // activation rows per tile (multiple of 16, <= 256)
    int tiles_w, tiles_n, nws;  // weight-row tiles, activation-row tiles, weight stages per tile
    int x_stages;
    // Schedule: units = tiles_w * tiles_n tiles of the output.  The last `sk_units` of them are cut along K
    // (stream-K): their sk_units*nws weight stages form one linear space dealt out in contiguous runs of
    // `sk_per_cta` to the first `sk_ctas` CTAs; the other units are taken whole, unit = cta, cta + grid, ...
    int dp_units, sk_units, sk_per_cta, sk_ctas;
    float* sums;              // [sk_units][BN/4][128] x float4: f32 sums of cut tiles (zero between uses)
    unsigned int* counters;   // [sk_units] arrivals per cut tile (zero between uses)
    int ldy, y_col0;
    int act;                  // RUSTY_CUDA_ACT_*: the pair epilogue writes N/2 columns
    const void* residual;     // null, or added to every output (same layout as y)
    PeerPush push;            // nranks > 1: every output is also stored into the other ranks' arenas (peer.cu)
    uint32_t idesc;
    rusty_cuda_dev_status* status;
};

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

// One output of activation row m and weight row n (this lane's), already scaled.  Every lane of the warp calls this
// together.  With the pair activation rows 2j / 2j+1 of the weight are gate_j / up_j (MLP::forward,
// rusty-graph/src/lib.rs:317-323): the even lane takes its neighbour's value and writes silu(gate) * up into column
// (y_col0 + n) / 2; silu as kernels.wgsl:104-113.
// The same element of every other rank's y, over NVLink (plain stores to peer addresses; the byte offsets of the other
// arenas sit in shared memory: indexing the kernel parameter with a run-time index would copy it to local memory).
struct PeerOut {
    int n;
    const long long* delta;
};
template <typename YT>
__device__ __forceinline__ void store_everywhere(YT* dst, float v, const PeerOut& po) {
    store_y<YT>(dst, v);
    for (int g = 0; g < po.n; ++g) store_y<YT>(reinterpret_cast<YT*>(reinterpret_cast<char*>(dst) + po.delta[g]), v);
}

template <typename YT>
__device__ __forceinline__ void store_out(const F16Params& p, YT* y, int m, int n, float v, bool row_ok, const PeerOut& po) {
    if (p.act) {
        const float up = __shfl_down_sync(0xffffffffu, v, 1);
        v = __fdividef(v, 1.0f + __expf(-v)) * up;
        if (row_ok && m < p.Mx && !(n & 1)) store_everywhere<YT>(y + (size_t)m * p.ldy + ((p.y_col0 + n) >> 1), v, po);
    } else if (row_ok && m < p.Mx) {
        const size_t at = (size_t)m * p.ldy + p.y_col0 + n;
        if (p.residual) v += load_y<YT>(reinterpret_cast<const YT*>(p.residual) + at);
        store_everywhere<YT>(y + at, v, po);
    }
}

// 16 int8 (one 128-bit word) -> 8 registers of packed bf16 pairs (low half = even k).
// u = q ^ 0x80 is q + 128; dropping u into the low mantissa byte of 2^23 and subtracting 2^23 + 128 leaves q
// exactly as an f32, and |q| <= 128 fits bf16's 8 significant bits, so the packed conversion is exact too.
__device__ __forceinline__ void int8x16_to_bf16x2(const uint4& w, uint32_t* out) {
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t u = words[i] ^ 0x80808080u;
        const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f;
        const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f;
        const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f;
        const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f;
        __nv_bfloat162 a = __floats2bfloat162_rn(f0, f1);
        __nv_bfloat162 b = __floats2bfloat162_rn(f2, f3);
        out[2 * i] = *reinterpret_cast<uint32_t*>(&a);
        out[2 * i + 1] = *reinterpret_cast<uint32_t*>(&b);
    }
}

// The reference's affine layout (WGSL `affine_dequantize`, rusty-backend/src/kernels.wgsl:385-400): w = f32(u8) * scale +
// bias, one (scale, bias) per 64 consecutive elements.  The product is rounded to bf16 for the tensor core (2^-9
// relative per weight: inside the 1e-2 tolerance of the bf16 path, not the 1e-5 of the f32 paths).
__device__ __forceinline__ void u8x16_affine_to_bf16x2(const uint4& w, float sc, float bi, uint32_t* out) {
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t u = words[i];
        const float f0 = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388608.0f, sc, bi);
        const float f1 = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388608.0f, sc, bi);
        const float f2 = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388608.0f, sc, bi);
        const float f3 = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388608.0f, sc, bi);
        __nv_bfloat162 a = __floats2bfloat162_rn(f0, f1);
        __nv_bfloat162 b = __floats2bfloat162_rn(f2, f3);
        out[2 * i] = *reinterpret_cast<uint32_t*>(&a);
        out[2 * i + 1] = *reinterpret_cast<uint32_t*>(&b);
    }
}

// The same with one (scale, bias) per element: 16 consecutive k of one row whose scales and biases are 16 consecutive
// floats each (an [in,out] affine weight after its re-layout: groups run along the output dimension).
__device__ __forceinline__ void u8x16_affine_vec_to_bf16x2(const uint4& w, const float* sc, const float* bi, uint32_t* out) {
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t u = words[i];
        const float4 s4 = reinterpret_cast<const float4*>(sc)[i], b4 = reinterpret_cast<const float4*>(bi)[i];   // shared memory, broadcast
        const float f0 = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388608.0f, s4.x, b4.x);
        const float f1 = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388608.0f, s4.y, b4.y);
        const float f2 = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388608.0f, s4.z, b4.z);
        const float f3 = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388608.0f, s4.w, b4.w);
        __nv_bfloat162 a = __floats2bfloat162_rn(f0, f1);
        __nv_bfloat162 b = __floats2bfloat162_rn(f2, f3);
        out[2 * i] = *reinterpret_cast<uint32_t*>(&a);
        out[2 * i + 1] = *reinterpret_cast<uint32_t*>(&b);
    }
}

// One piece of work: weight stages [s0, s1) of output tile `u`.  nseg > 1: the tile is shared with other CTAs.
struct Piece {
    int u, s0, s1, nseg, lu;
};

// Every role of the CTA walks the same list of pieces: the stream-K share first, whole tiles after it.
struct PieceSched {
    const F16Params& p;
    int g, g_end, dp_next;
    __device__ PieceSched(const F16Params& pp) : p(pp) {
        const int c = blockIdx.x;
        g = c < p.sk_ctas ? c * p.sk_per_cta : 0;
        g_end = c < p.sk_ctas ? min(p.sk_units * p.nws, g + p.sk_per_cta) : 0;
        dp_next = c;
    }
    __device__ bool next(Piece& q) {
        if (g < g_end) {
            q.lu = g / p.nws;
            q.u = p.dp_units + q.lu;
            q.s0 = g % p.nws;
            q.s1 = min(p.nws, q.s0 + (g_end - g));
            const int first = (q.lu * p.nws) / p.sk_per_cta;
            const int last = ((q.lu + 1) * p.nws - 1) / p.sk_per_cta;
            q.nseg = last - first + 1;
            g += q.s1 - q.s0;
            return true;
        }
        if (dp_next < p.dp_units) {
            q.u = dp_next;
            q.lu = 0;
            q.s0 = 0;
            q.s1 = p.nws;
            q.nseg = 1;
            dp_next += gridDim.x;
            return true;
        }
        return false;
    }
};

__device__ __forceinline__ void red_add_f32x4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// QM: 0 = one scale per output row (applied to the sums); 1 = AFFINE_G64 with groups along K ([N][K/64] scales and biases);
// 2 = AFFINE_G64 of an [in,out] weight after its re-layout: one (scale, bias) per 64 consecutive OUTPUT rows and k,
// stored [N/64][K] (internal mode QMODE_AFFINE_GC)
template <typename YT, int QM>
__global__ void __launch_bounds__(F16_THREADS, 1)
qlinear_f16_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const F16Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int x_stage_bytes = p.BN * XK * 2;
    uint8_t* sW = smem;
    uint8_t* sX = smem + (size_t)W_STAGES * W_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sX + (size_t)p.x_stages * x_stage_bytes);
    uint64_t* w_full = bars;                   // [W_STAGES]
    uint64_t* w_empty = w_full + W_STAGES;     // [W_STAGES]
    uint64_t* a_full = w_empty + W_STAGES;     // [A_BUFS]
    uint64_t* a_empty = a_full + A_BUFS;       // [A_BUFS]
    uint64_t* d_full = a_empty + A_BUFS;       // [1]
    uint64_t* d_empty = d_full + 1;            // [1]
    uint64_t* x_full = d_empty + 1;            // [x_stages]
    uint64_t* x_empty = x_full + p.x_stages;   // [x_stages]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(x_empty + p.x_stages);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    __shared__ long long s_peer_delta[PEER_MAX_RANKS];
    // QM == 2: per converter warp two buffers of (64 scales, 64 biases): those of the stage being converted and of the next
    __shared__ __align__(16) float s_gc[QM == 2 ? CONV_WARPS * 256 : 4];
    if (threadIdx.x == 0) {
        int k = 0;  // the other ranks, compacted (own rank left out); static indices into the parameter
#pragma unroll
        for (int g = 0; g < PEER_MAX_RANKS; ++g)
            if (g < p.push.nranks && g != p.push.rank) s_peer_delta[k++] = p.push.delta[g];
    }
    const PeerOut po = {p.push.nranks > 1 ? p.push.nranks - 1 : 0, s_peer_delta};   // visible after the set-up barrier below

    if (threadIdx.x == 0) {
        for (int s = 0; s < W_STAGES; ++s) {
            mbar_init(&w_full[s], 1);
            mbar_init(&w_empty[s], CONV_WARPS);
        }
        for (int s = 0; s < A_BUFS; ++s) {
            mbar_init(&a_full[s], CONV_WARPS);
            mbar_init(&a_empty[s], 1);
        }
        mbar_init(d_full, 1);
        mbar_init(d_empty, EPI_WARPS);
        for (int s = 0; s < p.x_stages; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&x_empty[s], 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a0 = tmem_base + D_COLS;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
            int ws = 0, xs = 0;
            uint32_t wph = 0, xph = 0;
            bool ok = true, waited = false;
            PieceSched sched(p);
            Piece pc;
            while (ok && sched.next(pc)) {
                const int t = pc.u % p.tiles_w, j = pc.u / p.tiles_w;
                for (int s = pc.s0; s < pc.s1 && ok; ++s) {
                    if (!mbar_wait(&w_empty[ws], wph ^ 1u, abort_flag, p.status, 11)) { ok = false; break; }
                    mbar_expect_tx(&w_full[ws], (uint32_t)W_STAGE_BYTES);
                    tma_load_2d(sW + (size_t)ws * W_STAGE_BYTES, &map_w, s * WK, t * BM, &w_full[ws], pol_w);
                    if (++ws == W_STAGES) { ws = 0; wph ^= 1u; }
                    if (!waited) {  // the weights never depend on earlier kernels; the activations may
                        pdl_wait();
                        waited = true;
                    }
                    for (int h = 0; h < WK / XK; ++h) {
                        if (!mbar_wait(&x_empty[xs], xph ^ 1u, abort_flag, p.status, 12)) { ok = false; break; }
                        mbar_expect_tx(&x_full[xs], (uint32_t)x_stage_bytes);
                        tma_load_2d(sX + (size_t)xs * x_stage_bytes, &map_x, s * WK + h * XK, j * p.BN, &x_full[xs], pol_x);
                        if (++xs == p.x_stages) { xs = 0; xph ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            int ab = 0, xs = 0;
            uint32_t aph = 0, xph = 0;
            bool ok = true;
            int i = 0;
            PieceSched sched(p);
            Piece pc;
            for (; ok && sched.next(pc); ++i) {
                if (!mbar_wait(d_empty, ((uint32_t)i & 1u) ^ 1u, abort_flag, p.status, 13)) { ok = false; break; }
                tc_fence_after();
                for (int s = pc.s0; s < pc.s1 && ok; ++s) {
                    if (!mbar_wait(&a_full[ab], aph, abort_flag, p.status, 14)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_tmem = tmem_a0 + (uint32_t)(ab * A_COLS);
                    for (int h = 0; h < WK / XK; ++h) {
                        if (!mbar_wait(&x_full[xs], xph, abort_flag, p.status, 15)) { ok = false; break; }
                        tc_fence_after();
                        const uint64_t db = make_smem_desc(smem_u32(sX + (size_t)xs * x_stage_bytes));
#pragma unroll
                        for (int k16 = 0; k16 < XK / 16; ++k16)
                            umma_f16_ts(tmem_base, a_tmem + (uint32_t)((h * (XK / 16) + k16) * 8), db + (uint64_t)(2 * k16), p.idesc,
                                        (s > pc.s0 || h > 0 || k16 > 0) ? 1u : 0u);
                        umma_commit(&x_empty[xs]);
                        if (++xs == p.x_stages) { xs = 0; xph ^= 1u; }
                    }
                    umma_commit(&a_empty[ab]);
                    if (++ab == A_BUFS) { ab = 0; aph ^= 1u; }
                }
                if (ok) umma_commit(d_full);
            }
        }
    } else if (warp < 2 + CONV_WARPS) {
        // ------------------------------ converters --------------------------------
        // Warp pair (w, w+4) shares TMEM lane quarter q = w & 3; `half` picks k 0..63 or 64..127 of the stage.
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        const int r = q * 32 + lane;  // weight row inside the tile = TMEM lane
        int ws = 0, ab = 0;
        uint32_t wph = 0, aph = 0;
        bool ok = true;
        PieceSched sched(p);
        Piece pc;
        while (ok && sched.next(pc)) {
            const int n_row = (pc.u % p.tiles_w) * BM + r;   // this thread's weight row
            for (int s = pc.s0; s < pc.s1 && ok; ++s) {
                // affine: this thread's 64 k-elements of the stage are exactly one group of its row (K % 64 == 0)
                float g_sc = 0.0f, g_bi = 0.0f;
                // QM == 2: the warp's 32 rows lie in one 64-row group, so the stage's 64 scales and 64 biases are the same
                // for every lane: lane l copies four of them (cp.async, 16 bytes) into the warp's own corner of shared
                // memory, one stage ahead of the conversion that reads them back as broadcasts
                [[maybe_unused]] const float* gc = nullptr;
                if constexpr (QM == 2) {
                    float* mine = s_gc + (size_t)(warp - 2) * 256;
                    const bool rows_ok = n_row - lane < p.N;   // (N % 64 == 0: the group is inside the matrix or outside)
                    auto issue = [&](int st, int buf) {
                        const int k0 = st * WK + half * 64;
                        if (rows_ok && k0 < p.K) {
                            const float* src = (lane < 16 ? p.scales : p.biases) + (size_t)(n_row >> 6) * p.K + k0 + (lane & 15) * 4;
                            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(mine + buf * 128 + lane * 4)), "l"(src) : "memory");
                        }
                        asm volatile("cp.async.commit_group;" ::: "memory");
                    };
                    const int buf = (s - pc.s0) & 1;
                    if (s == pc.s0) issue(s, buf);
                    if (s + 1 < pc.s1) {
                        issue(s + 1, buf ^ 1);
                        asm volatile("cp.async.wait_group 1;" ::: "memory");
                    } else {
                        asm volatile("cp.async.wait_group 0;" ::: "memory");
                    }
                    __syncwarp();
                    if (rows_ok && s * WK + half * 64 < p.K) gc = mine + buf * 128;
                }
                if constexpr (QM == 1) {
                    const int k0 = s * WK + half * 64;
                    if (n_row < p.N && k0 < p.K) {
                        const size_t g = ((size_t)n_row * p.K + k0) >> 6;
                        g_sc = __ldg(p.scales + g);
                        g_bi = __ldg(p.biases + g);
                    }
                }
                if (!mbar_wait(&w_full[ws], wph, abort_flag, p.status, 16)) { ok = false; break; }
                // row r of the swizzled tile: logical 16-byte chunk c sits at physical chunk c ^ (r & 7)
                const uint32_t row = smem_u32(sW + (size_t)ws * W_STAGE_BYTES + (size_t)r * WK);
                uint4 raw[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) raw[c] = lds128(row + (uint32_t)(((half * 4 + c) ^ (r & 7)) << 4));   // (kept in front of the hand-back)
                __syncwarp();
                if (lane == 0) mbar_arrive(&w_empty[ws]);  // this warp's share is in registers
                if (++ws == W_STAGES) { ws = 0; wph ^= 1u; }
                uint32_t cv[32];
                if constexpr (QM == 2) {
                    if (gc) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) u8x16_affine_vec_to_bf16x2(raw[c], gc + 16 * c, gc + 64 + 16 * c, cv + 8 * c);
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e) cv[e] = 0u;
                    }
                } else if constexpr (QM == 1) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) u8x16_affine_to_bf16x2(raw[c], g_sc, g_bi, cv + 8 * c);
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c) int8x16_to_bf16x2(raw[c], cv + 8 * c);
                }
                if (!mbar_wait(&a_empty[ab], aph ^ 1u, abort_flag, p.status, 17)) { ok = false; break; }
                tc_fence_after();
                tmem_st32(tmem_a0 + ((uint32_t)(q * 32) << 16) + (uint32_t)(ab * A_COLS + half * 32), cv);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[ab]);
                if (++ab == A_BUFS) { ab = 0; aph ^= 1u; }
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int q = warp & 3;
        const int r = q * 32 + lane;
        // this warp's share of the accumulator's columns (activation rows of the tile), in chunks of 16
        const int c_split = ((p.BN / 2 + 15) / 16) * 16;
        const int c_lo = (warp - (2 + CONV_WARPS)) >= 4 ? c_split : 0;
        const int c_hi = (warp - (2 + CONV_WARPS)) >= 4 ? p.BN : c_split;
        YT* y = reinterpret_cast<YT*>(p.y);
        const bool plain = !p.act && !p.residual && po.n == 0;
        pdl_wait();
        bool ok = true;
        int i = 0;
        PieceSched sched(p);
        Piece pc;
        for (; ok && sched.next(pc); ++i) {
            const int t = pc.u % p.tiles_w, j = pc.u / p.tiles_w;
            const int n = t * BM + r;
            const bool row_ok = n < p.N;
            const float sc = !row_ok ? 0.0f : QM != 0 ? 1.0f : __ldg(p.scales + n);
            if (!mbar_wait(d_full, (uint32_t)i & 1u, abort_flag, p.status, 18)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
            if (pc.nseg == 1) {
                for (int c0 = c_lo; c0 < c_hi; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(taddr + (uint32_t)c0, v);
                    tmem_ld_wait();
                    if (plain) {   // the common case keeps the shortest code: this loop holds up the next tile's MMAs
                        if (row_ok) {
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                const int m = j * p.BN + c0 + e;
                                if (m < p.Mx) store_y<YT>(y + (size_t)m * p.ldy + p.y_col0 + n, __uint_as_float(v[e]) * sc);
                            }
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 16; ++e) store_out<YT>(p, y, j * p.BN + c0 + e, n, __uint_as_float(v[e]) * sc, row_ok, po);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(d_empty);
            } else {
                // a K-slice of a shared tile: add it into the tile's f32 sums ([col/4][row] x float4, so a warp's
                // vector reductions cover 512 contiguous bytes); the last CTA to arrive writes y.
                float* tile = p.sums + (size_t)pc.lu * p.BN * BM;
                for (int c0 = c_lo; c0 < c_hi; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(taddr + (uint32_t)c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 16; e += 4)
                        red_add_f32x4(tile + ((size_t)((c0 + e) / 4) * BM + r) * 4, __uint_as_float(v[e]), __uint_as_float(v[e + 1]),
                                      __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(d_empty);
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");
                if (threadIdx.x == 32 * (2 + CONV_WARPS)) {
                    const unsigned prev = atomicAdd(p.counters + pc.lu, 1u);
                    *last_flag = (prev == (unsigned)(pc.nseg - 1)) ? 1 : 0;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");
                if (*last_flag) {
                    __threadfence();
                    for (int c0 = c_lo; c0 < c_hi; c0 += 16) {
                        float4 f[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) f[e] = __ldcg(reinterpret_cast<const float4*>(tile) + (size_t)(c0 / 4 + e) * BM + r);
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            __stcg(reinterpret_cast<float4*>(tile) + (size_t)(c0 / 4 + e) * BM + r, make_float4(0.f, 0.f, 0.f, 0.f));
                        if (plain) {
                            if (row_ok) {
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float vals[4] = {f[e].x, f[e].y, f[e].z, f[e].w};
#pragma unroll
                                    for (int k = 0; k < 4; ++k) {
                                        const int m = j * p.BN + c0 + e * 4 + k;
                                        if (m < p.Mx) store_y<YT>(y + (size_t)m * p.ldy + p.y_col0 + n, vals[k] * sc);
                                    }
                                }
                            }
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float vals[4] = {f[e].x, f[e].y, f[e].z, f[e].w};
#pragma unroll
                                for (int k = 0; k < 4; ++k) store_out<YT>(p, y, j * p.BN + c0 + e * 4 + k, n, vals[k] * sc, row_ok, po);
                            }
                        }
                    }
                    if (threadIdx.x == 32 * (2 + CONV_WARPS)) p.counters[pc.lu] = 0u;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace

namespace rusty {

bool f16tc_supported(const rusty_cuda_ctx*, const QLinearArgs& a) {
    if (!encode_tiled_fn()) return false;
    if (a.layout != RUSTY_CUDA_LAYOUT_NK) return false;
    if (a.qmode == RUSTY_CUDA_QMODE_AFFINE_G64 ? (a.K % 64 != 0 || a.act)
        : a.qmode == QMODE_AFFINE_GC          ? (a.K % 128 != 0 || a.N % 64 != 0 || a.act)
                                              : a.qmode != RUSTY_CUDA_QMODE_SYM_ROW)
        return false;
    if (a.x_dtype != RUSTY_CUDA_BF16) return false;
    if (a.K % 16 != 0) return false;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.x) & 15) != 0) return false;
    return true;
}

int launch_f16tc(rusty_cuda_ctx* ctx, const QLinearArgs& a) {
    F16Params p{};
    p.scales = a.scales;
    p.biases = (a.qmode == RUSTY_CUDA_QMODE_AFFINE_G64 || a.qmode == QMODE_AFFINE_GC) ? a.biases : nullptr;
    p.y = a.y;
    p.Mx = (int)a.M;
    p.N = (int)a.N;
    p.K = (int)a.K;
    p.BN = a.M >= 256 ? 256 : (int)((a.M + 15) / 16 * 16);
    p.tiles_w = (p.N + BM - 1) / BM;
    p.tiles_n = (p.Mx + p.BN - 1) / p.BN;
    p.nws = (p.K + WK - 1) / WK;
    p.ldy = (int)a.ldy;
    p.y_col0 = (int)a.y_col0;
    p.act = a.act;
    p.residual = a.residual;
    if (a.push && a.push->nranks > 1) p.push = *a.push;
    p.status = ctx->status_dev;
    // bf16 A x bf16 B -> f32: c_format=F32(1)@4, a_format=BF16(1)@7, b_format=BF16(1)@10, N>>3 @17, M>>4 @24
    p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    // (the group-column affine variant keeps 8 KB of static shared memory for its scales and biases)
    const size_t reserve = a.qmode == QMODE_AFFINE_GC ? 4096 + 8192 : 4096;
    const size_t budget = ctx->smem_optin > reserve ? ctx->smem_optin - reserve : 0;
    const size_t x_stage = (size_t)p.BN * XK * 2;
    int xs = (int)((budget - 1024 - 512 - (size_t)W_STAGES * W_STAGE_BYTES) / x_stage);
    if (xs > 8) xs = 8;
    if (xs < 2) return fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "f16 tensor-core path: tile does not fit shared memory");
    p.x_stages = xs;
    const size_t smem = 1024 + (size_t)W_STAGES * W_STAGE_BYTES + (size_t)xs * x_stage + (size_t)(2 * W_STAGES + 2 * A_BUFS + 2 + 2 * xs) * 8 + 64;

    CUtensorMap map_w, map_x;
    if (!make_map_u8(&map_w, a.w, a.N, a.K, BM) || !make_map_bf16(&map_x, a.x, a.M, a.K, (uint32_t)p.BN))
        return fail(ctx, RUSTY_CUDA_ERR_KERNEL_EXECUTION, "f16 tensor-core path: cuTensorMapEncodeTiled failed");
    const int units = p.tiles_w * p.tiles_n;
    int grid = units < ctx->sm_count ? units : ctx->sm_count;
    // whole waves of tiles are taken tile-per-CTA; the remainder is cut along K over all CTAs (>= 4 stages each)
    p.sk_units = units >= grid ? units % grid : 0;
    p.dp_units = units - p.sk_units;
    p.sk_per_cta = p.sk_ctas = 0;
    p.sums = nullptr;
    p.counters = nullptr;
    if (p.sk_units > 0) {
        float* sums = nullptr;
        unsigned int* counters = nullptr;
        size_t sums_bytes = 0, cnt_bytes = 0;
        tc_workspace_sums(ctx, &sums, &sums_bytes, &counters, &cnt_bytes);
        const size_t need = (size_t)p.sk_units * p.BN * BM * 4;
        static const bool no_sk = getenv("RUSTY_F16_NO_STREAMK") != nullptr;
        if (sums && need <= sums_bytes && (size_t)p.sk_units * 4 <= cnt_bytes && !no_sk) {
            const int work = p.sk_units * p.nws;
            p.sk_per_cta = (work + grid - 1) / grid;
            if (p.sk_per_cta < 4) p.sk_per_cta = 4;
            p.sk_ctas = (work + p.sk_per_cta - 1) / p.sk_per_cta;
            p.sums = sums;
            p.counters = counters;
        } else {
            p.dp_units = units;
            p.sk_units = 0;
        }
    }
    const bool yb = a.y_dtype == RUSTY_CUDA_BF16;
    const int qm = a.qmode == QMODE_AFFINE_GC ? 2 : p.biases != nullptr ? 1 : 0;
    auto kern = qm == 2   ? (yb ? qlinear_f16_tc_kernel<__nv_bfloat16, 2> : qlinear_f16_tc_kernel<float, 2>)
                : qm == 1 ? (yb ? qlinear_f16_tc_kernel<__nv_bfloat16, 1> : qlinear_f16_tc_kernel<float, 1>)
                          : (yb ? qlinear_f16_tc_kernel<__nv_bfloat16, 0> : qlinear_f16_tc_kernel<float, 0>);
    {
        cudaError_t e = ensure_dynamic_smem((const void*)kern, ctx->device, smem);
        if (e != cudaSuccess) return check_cuda(ctx, e, "qlinear_f16_tc: cudaFuncSetAttribute");
    }
#ifdef RUSTY_TIMELINE
    {   // development aid: what the launch would take if the epilogue stored nothing (results are then invalid)
        static const bool nostore = getenv("RUSTY_F16_NOSTORE") != nullptr;
        if (nostore) p.Mx = 0;
    }
#endif
    cudaError_t le = launch_pdl(kern, dim3(grid), dim3(F16_THREADS), smem, ctx->stream, map_w, map_x, p);
    if (le != cudaSuccess) return check_cuda(ctx, le, "qlinear_f16_tc");
    return after_launch(ctx, "qlinear_f16_tc");
}

}  // namespace rusty
