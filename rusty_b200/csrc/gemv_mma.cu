// Fused int8-weight GEMV for one or two activation rows on the warp-level integer tensor-core path.
//
// Same arithmetic contract as the other fused kernels (mode SYM_ROW, [out,in] storage):
//     y[m,n] = scale[n] * sum_k x[m,k] * f32(q[n,k])
// standing in for the reference's dequantise-at-load + f32 matmul per forward
// (rusty-loader/src/lib.rs:155-218, rusty-backend/src/kernels.wgsl:234-242).
//
// Why not CUDA cores: a byte of weight costs three lane-instructions there (permute, subtract, FMA), and a
// 16 MB matrix is only ~2.6 us of HBM time, so the conversion sits on the critical path behind the activations.
// Here the weights are never converted: mma.sync.m16n8k32 (s8 x s8 -> s32) takes 16 weight rows x 32 k straight
// from shared memory as its A operand, one instruction per 512 weight bytes.  The activations become the B operand:
// each activation is split EXACTLY into signed 7-bit digits against a power-of-two scale,
//     x[m,k] * s = d0 + d1/128 + d2/128^2 + d3/128^3        (f32: four digits, 28 bits; bf16: three, the fourth is 0),
// digit i of row m is column 4m + i of B (8 columns: one or two activation rows), the integer dot products are exact
// and the digits are recombined in 64-bit integers.
//
// Data movement.  One CTA per SM, each owning a contiguous range of weight rows (an even share of N, in units of two
// rows so that a (gate, up) pair never straddles CTAs): no K split across CTAs, no sum across CTAs.
//   * one producer thread streams the CTA's rows as (16 rows x 1024 k) stages of 16 KB: ONE TMA copy each (the
//     matrix seen as [k-block][row][128 bytes], 128-byte swizzle, so that the fragment loads below are bank-conflict
//     free) into a ring of shared-memory stages, mbarrier complete_tx.  The copies start BEFORE
//     griddepcontrol.wait: weights never depend on the previous kernel, and a short kernel's CTA takes at most half
//     of an SM, so the next kernel's CTA lands its weights while this one computes.  What the ring cannot hold yet
//     is asked into L2 at once (TMA prefetch).  The last group of 16 rows of a share is shifted back so that it ends
//     with the share: a CTA never loads another CTA's rows.
//   * warp w of the 8 compute warps owns k-bytes [128 w, 128 w + 128) of every stage, i.e. a fixed slice of K.  After
//     the wait it works on ITS slice of the activations only: slice maximum -> its own power-of-two scale -> digits
//     into a warp-private corner of shared memory.  No block-wide barrier, no block-wide maximum: the warps run free
//     of each other from the first instruction to the last, and a slice's digits hang below the slice's own maximum
//     (never worse, usually better, than below the row's).
//   * it then walks the stages, software-pipelined: the four 16-byte weight loads of stage i+1 are issued before the
//     four MMAs of stage i, which go into four independent accumulators.
//   * after the last stage of a group of 16 rows each warp folds its digit columns (exact int64, one shuffle), scales
//     by its own 1/s (a power of two: exact) and parks the result as doubles; a reducer warp adds the 8 slices in a
//     fixed order, applies scale[n] (held in shared memory; and silu(gate)*up for pairs), rounds to f32 and stores y,
//     while the compute warps are already on the next group.
// Every mbarrier wait is bounded.
//
// A second instantiation (GC, further down) runs the reference's own quantised format -- u8 [in,out] with one scale and
// bias per 64 consecutive OUTPUT features of an input row -- after its one-time re-layout to [out,in]: there the scales
// ride on the activations, one CTA owns part of one 64-row group and one pair of activation rows.
#include <cstdlib>

#include "tc_common.cuh"

using namespace rusty_tc;

namespace {

constexpr int GW = 8;                        // compute warps
constexpr int GM_THREADS = 32 * (GW + 2);    // + reducer warp + producer warp
constexpr int KB = 128;                      // k-bytes one warp covers per stage
constexpr int KC = GW * KB;                  // k-bytes per stage (1024)
constexpr int STAGE_ROWS = 16;               // = MMA m
constexpr int STAGE_BYTES = STAGE_ROWS * KC; // [8 k-blocks][16 rows][128 bytes]
constexpr int MAX_M = 2;                     // activation rows: 4 digit columns each, 8 columns of B

struct GmParams {
    const uint8_t* W;
    const float* scales;
    const float* gscale;   // group-column affine weights (GC kernel): scale and bias of row group n / 64 at every k,
    const float* gbias;    //   [N/64][K] each; the weight bytes are then unsigned
    const void* x;
    void* y;
    int M, N, K;
    int D;          // digits per activation: 4 (f32 x) or 3 (bf16 x; the fourth column stays zero)
    int R;          // 4 * M digit columns (<= 8)
    int nch;        // stages along K: ceil(K / KC)
    int dstride;    // bytes between digit columns of a warp's corner of shared memory: nch*KB + 16
    int stages;
    int units;      // ceil(N / 2): row pairs dealt evenly to the CTAs
    int sc_cap;     // row scales kept in shared memory per CTA (>= the largest row share when it fits)
    int ldy, y_col0;
    int gc_rows;    // GC kernel: weight rows per CTA (16, 32 or 64: a CTA stays inside one 64-row group)
    int act;        // RUSTY_CUDA_ACT_SWIGLU_PAIRS: rows 2j, 2j+1 -> column (y_col0 + 2j) / 2
    int x_bf16, y_bf16;
    rusty_cuda_dev_status* status;
    long long* dbg;   // per-CTA timeline (16 slots each); null outside development builds
    int n_peers;                          // other ranks whose copy of y also receives every output (peer.cu); 0: none
    long long peer_delta[PEER_MAX_RANKS]; // byte offsets of their arenas, compacted (used with static indices only)
};

// Kernel timeline (%globaltimer stamps per CTA), compiled in only with -DRUSTY_TIMELINE (a development build).
#ifdef RUSTY_TIMELINE
#define GDBG(slot) do { if (p.dbg) p.dbg[(size_t)blockIdx.x * 16 + (slot)] = (long long)globaltimer_ns(); } while (0)
#else
#define GDBG(slot) do { } while (0)
#endif

// D[16x8] += A[16x32] * B[32x8], int8 operands, int32 accumulators.
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The same with unsigned weight bytes (affine weights are u8).
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float4 load_x4(const GmParams& p, int m, int k) {
    if (p.x_bf16) {
        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.x) + (size_t)m * p.K + k);
        return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                           __uint_as_float(raw.y & 0xffff0000u));
    }
    return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x) + (size_t)m * p.K + k);
}

// The CTA's share of the weight rows: units (row pairs) [u0, u1) -> rows [2 u0, min(N, 2 u1)).
__device__ __forceinline__ void cta_rows(const GmParams& p, int& row0, int& rows) {
    const long long u0 = (long long)blockIdx.x * p.units / gridDim.x, u1 = (long long)(blockIdx.x + 1) * p.units / gridDim.x;
    row0 = (int)(2 * u0);
    const int row1 = min(p.N, (int)(2 * u1));
    rows = row1 - row0;
}

// Four activations (already times their scale) -> their digits -> four 4-byte words, one per digit column, written
// `dstride` bytes apart starting at `at` (column 0 = most significant).  Deliberately NOT inlined: a CTA runs this a
// handful of times, and code that a CTA executes once costs an instruction-cache miss per line.
template <int D>
__device__ __noinline__ void emit_digits(float v0, float v1, float v2, float v3, uint8_t* at, int dstride) {
    const uint32_t w0 = digits_of<D>(v0), w1 = digits_of<D>(v1), w2 = digits_of<D>(v2), w3 = digits_of<D>(v3);
    // 4 elements x 4 digit bytes -> 4 digit columns x 4 element bytes
    const uint32_t t0 = __byte_perm(w0, w1, 0x5140), t1 = __byte_perm(w2, w3, 0x5140);   // bytes 0 and 1
    const uint32_t t2 = __byte_perm(w0, w1, 0x7362), t3 = __byte_perm(w2, w3, 0x7362);   // bytes 2 and 3
    // byte b holds digit b counted from the least significant, byte D-1 the top digit = column 0; with three
    // digits the fourth column is zero
    if (D == 4) {
        *reinterpret_cast<uint32_t*>(at + 3 * (size_t)dstride) = __byte_perm(t0, t1, 0x5410);
        *reinterpret_cast<uint32_t*>(at + 2 * (size_t)dstride) = __byte_perm(t0, t1, 0x7632);
        *reinterpret_cast<uint32_t*>(at + 1 * (size_t)dstride) = __byte_perm(t2, t3, 0x5410);
        *reinterpret_cast<uint32_t*>(at) = __byte_perm(t2, t3, 0x7632);
    } else {
        *reinterpret_cast<uint32_t*>(at + 3 * (size_t)dstride) = 0u;
        *reinterpret_cast<uint32_t*>(at + 2 * (size_t)dstride) = __byte_perm(t0, t1, 0x5410);
        *reinterpret_cast<uint32_t*>(at + 1 * (size_t)dstride) = __byte_perm(t0, t1, 0x7632);
        *reinterpret_cast<uint32_t*>(at) = __byte_perm(t2, t3, 0x5410);
    }
}

// GC ("group columns"): the reference's own layout, [in,out] storage with one (scale, bias) per 64 consecutive
// OUTPUT features of an input row, after its one-time re-layout to [out,in]:
//     y[m,n] = sum_k x[m,k] * (u[n,k] * s[g,k] + b[g,k]),   g = n / 64
//            = sum_k (x[m,k] * s[g,k]) * u[n,k]  +  sum_k x[m,k] * b[g,k]
// so for the 64 rows of a group the scales move over to the activations: a' = x (.) s_g is digitised instead of x, the
// unsigned weight bytes go into the tensor core as they are, and the bias term is one number per group and
// activation row.  A CTA takes 16, 32 or 64 rows of one group, so everything it needs of s and b is two K-long vectors.
// Weight rows per CTA of the GC kernel: the largest of 64, 32, 16 that still gives every SM a CTA (a CTA's fixed cost,
// the digits of its activations, is paid per CTA; too few CTAs leave SMs idle).
int gc_rows_per_cta(const rusty_cuda_ctx* ctx, uint32_t N, uint32_t M) {
    const uint32_t pairs = (M + MAX_M - 1) / MAX_M, sms = ctx->sm_count > 0 ? (uint32_t)ctx->sm_count : 1u;
    for (uint32_t rows = 64; rows > 16; rows /= 2)
        if ((N / rows) * pairs >= sms) return (int)rows;
    return 16;
}

template <bool GC>
__global__ void __launch_bounds__(GM_THREADS, 2) gemv_mma_kernel(const __grid_constant__ CUtensorMap map_w, const GmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // carve: [weight stages][digits, one corner per warp][partials 2 x GW x 32 doubles][barriers][flag][row scales]
    uint8_t* sW = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));   // swizzle atoms are 1 KiB
    uint8_t* sDig = sW + (size_t)p.stages * STAGE_BYTES;
    const int dig_warp_bytes = p.R * p.dstride;          // one warp's corner: R columns of nch*128 + 16 bytes
    double* sPart = reinterpret_cast<double*>(sDig + (size_t)GW * dig_warp_bytes);   // [2][GW][m][16 rows]: sums of a K slice
    uint64_t* full = reinterpret_cast<uint64_t*>(sPart + 2 * GW * 32);
    uint64_t* empty = full + p.stages;        // compute warps are done with a stage (count GW)
    uint64_t* done = empty + p.stages;        // [2] partials of a row group are parked (count GW)
    uint64_t* freeb = done + 2;               // [2] the reducer has read them (count 1)
    volatile int* abort_flag = reinterpret_cast<volatile int*>(freeb + 2);
    float* s_wscale = reinterpret_cast<float*>(freeb + 2) + 4;   // [sc_cap] scale[n] of this CTA's rows

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) GDBG(0);
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], GW);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&done[b], GW);
            mbar_init(&freeb[b], 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    // GC: blockIdx.y picks the pair of activation rows this CTA works on (batches of more than two rows)
    const int m_base = GC ? (int)blockIdx.y * MAX_M : 0;
    const int Mrows = GC ? min(MAX_M, p.M - m_base) : p.M;
    int row0, rows;
    if constexpr (GC) {
        row0 = (int)blockIdx.x * p.gc_rows;
        rows = min(p.gc_rows, p.N - row0);
    } else {
        cta_rows(p, row0, rows);
    }
    const int groups = (rows + STAGE_ROWS - 1) / STAGE_ROWS;
    const int total = groups * p.nch;          // stages this CTA walks: index = group * nch + chunk

    // first row (relative to row0) of group g: the last group is shifted back to end with the share
    auto group_start = [&](int g) { return min(g * STAGE_ROWS, max(rows - STAGE_ROWS, 0)); };

    if (warp == GW + 1) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            // one pass over the weights: nothing to keep in L2; several row pairs: the other pairs' CTAs read them again
            const uint64_t pol = (GC && gridDim.y > 1) ? policy_evict_last() : policy_evict_first();
            // What the ring will not hold at first: into L2 now, so that it is a short trip later.  Long streams
            // are left alone (the ring runs far ahead of the consumers there anyway).
            if (total <= 3 * p.stages)
                for (int i = p.stages + 2; i < total; ++i) tma_prefetch_3d(&map_w, 0, row0 + group_start(i / p.nch), (i % p.nch) * (KC / 128));
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int g = 0; ok && g < groups; ++g) {
                const int r0 = row0 + group_start(g);
                for (int c = 0; c < p.nch; ++c) {
                    if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, 31)) { ok = false; break; }
                    mbar_expect_tx(&full[stage], (uint32_t)STAGE_BYTES);   // the whole box, zero-filled where it leaves the matrix
                    tma_load_3d(sW + (size_t)stage * STAGE_BYTES, &map_w, 0, r0, c * (KC / 128), &full[stage], pol);
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
            }
            GDBG(7);
        }
    } else if (warp == GW) {
        // ------------------------------ reducer -------------------------------
        // The row scales are a property of the weight: fetch this CTA's share before waiting for the previous kernel,
        // so that no trip to memory is left in the per-group chain below.
        if constexpr (!GC)
            for (int i = lane; i < min(rows, p.sc_cap); i += 32) s_wscale[i] = __ldg(p.scales + row0 + i);
        __syncwarp();
        pdl_wait();  // y belongs to earlier kernels until now
        // lane = m * 16 + r: activation row m, weight row r of the group
        const int m = lane >> 4, r = lane & 15;
        for (int g = 0; g < groups; ++g) {
            const int b = g & 1;
            if (!mbar_wait(&done[b], ((uint32_t)g >> 1) & 1u, abort_flag, p.status, 32)) break;
            if (g == 0 && lane == 0) GDBG(8);
            double a = 0.0;
            const volatile double* src = sPart + (size_t)b * GW * 32 + lane;   // volatile: read BEFORE the buffer is handed back below
#pragma unroll
            for (int w = 0; w < GW; ++w) a += src[w * 32];   // the K slices in a fixed order: the same bits on every run
            __syncwarp();
            if (lane == 0) mbar_arrive(&freeb[b]);
            const int i0 = group_start(g) + r, n = row0 + i0;
            const bool in = m < Mrows && i0 < rows && i0 >= g * STAGE_ROWS;   // rows a shifted last group repeats are skipped
            const float sc = !in ? 0.0f : GC ? 1.0f : (i0 < p.sc_cap ? s_wscale[i0] : __ldg(p.scales + n));
            // the sum of the slices is exact in double (integers times powers of two); one rounding to f32, then the
            // weight's scale (one more rounding), as in the other fused kernels
            float v = __double2float_rn(a) * sc;
            size_t col = (size_t)p.y_col0 + n;
            bool live = in;
            if (p.act) {
                // rows n, n + 1 (n even: row0 and the group size are even) are one (gate, up) pair: silu(gate) * up
                // (rusty-graph/src/lib.rs:317-323; silu as kernels.wgsl:104-113)
                const float up = __shfl_down_sync(0xffffffffu, v, 1);
                live = in && !(r & 1) && i0 + 1 < rows;
                v = __fdividef(v, 1.0f + __expf(-v)) * up;
                col >>= 1;
            }
            if (live) {
                const size_t at = (size_t)(m_base + m) * p.ldy + col;
                if (p.y_bf16) {
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.y) + at;
                    const __nv_bfloat16 b = __float2bfloat16_rn(v);
                    *dst = b;
#pragma unroll
                    for (int g = 0; g < PEER_MAX_RANKS - 1; ++g)   // the same element of every other rank's y, over NVLink
                        if (g < p.n_peers) *reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(dst) + p.peer_delta[g]) = b;
                } else {
                    float* dst = reinterpret_cast<float*>(p.y) + at;
                    *dst = v;
#pragma unroll
                    for (int g = 0; g < PEER_MAX_RANKS - 1; ++g)
                        if (g < p.n_peers) *reinterpret_cast<float*>(reinterpret_cast<char*>(dst) + p.peer_delta[g]) = v;
                }
            }
        }
        if (lane == 0) GDBG(6);
    } else {
        // ------------------------------ compute -------------------------------
        const int g8 = lane >> 2, j = lane & 3;      // fragment coordinates: weight row (and row + 8) / digit column, k quarter
        uint8_t* dig = sDig + (size_t)warp * dig_warp_bytes;   // this warp's corner: column r at r * dstride, chunk c at c * KB
        // stage layout [k-block = warp][row][128 bytes], 16-byte chunk c of row r at c ^ (r & 7): this lane's chunks 2j, 2j+1
        const uint32_t frag0 = (uint32_t)(warp * (STAGE_ROWS * 128) + g8 * 128 + (((2 * j) ^ g8) << 4));
        const uint32_t frag1 = (uint32_t)(warp * (STAGE_ROWS * 128) + g8 * 128 + (((2 * j + 1) ^ g8) << 4));
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        // this lane's 2 x 32 weight bytes (rows g8 and g8 + 8) of the next stage: ring -> registers, slot handed back
        auto fetch = [&](uint4 (&w)[4]) {
            if (!mbar_wait(&full[stage], phase, abort_flag, p.status, 33)) { ok = false; return; }
            const uint8_t* st = sW + (size_t)stage * STAGE_BYTES;
            const uint32_t sa = smem_u32(st);
            w[0] = lds128(sa + frag0);
            w[1] = lds128(sa + frag1);
            w[2] = lds128(sa + frag0 + 8 * 128);   // row g8 + 8: the same swizzle
            w[3] = lds128(sa + frag1 + 8 * 128);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[stage]);   // this warp's share of the stage is in registers
            if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        };
        // The first two stages go into the pipeline registers BEFORE the activations exist: their ring slots are
        // handed back at once, so the producer can run two stages further ahead of the wait.
        uint4 wA[4], wB[4];
        if (total > 0) fetch(wA);
        if (ok && total > 1) fetch(wB);

        // GC: the group's scale and bias vectors belong to the weight; this lane's share of the items held in
        // registers is asked into L2 before the wait as well
        constexpr int XV = 4;
        auto item_k = [&](int c) { return c * KC + warp * KB + lane * 4; };
        const float* gs = nullptr;
        const float* gb = nullptr;
        double cb_row[MAX_M] = {0.0, 0.0};   // this lane's, later this warp's, part of sum_k x[m,k] * b[g,k]
        if constexpr (GC) {
            gs = p.gscale + (size_t)(row0 / 64) * p.K;
            gb = p.gbias + (size_t)(row0 / 64) * p.K;
            int c = 0;
#pragma unroll
            for (int i = 0; i < XV; ++i) {
                const int k = item_k(c);
                const bool live = i < Mrows * p.nch && k < p.K;
                if (live) {   // read beside x after the wait: a short trip then
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(gs + k));
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(gb + k));
                }
                if (++c == p.nch) c = 0;
            }
        }
        // GC: v <- v (.) s, and the bias sum when `with_bias` (the first of the two reads of an item)
        auto fold_group = [&](int mrow, float4& v, const float4& s4, const float4& b4, bool with_bias) {
            if (with_bias) {
                const double d = (double)v.x * b4.x + (double)v.y * b4.y + (double)v.z * b4.z + (double)v.w * b4.w;
                if (mrow == 0) cb_row[0] += d;
                else cb_row[1] += d;
            }
            v.x *= s4.x; v.y *= s4.y; v.z *= s4.z; v.w *= s4.w;
        };

        pdl_wait();  // x may come from the previous kernel
        if (threadIdx.x == 0) GDBG(1);

        // ---- this warp's slice of the activations: item i = (row m = i / nch, chunk c = i % nch) is the four
        // activations at k = c*KC + warp*KB + 4*lane.  The first XV items stay in registers between the maximum
        // and the digits (K <= 4096 with one row, 2048 with two); further items are read twice.
        const int items = Mrows * p.nch;
        float4 xv[XV];
        float mx_row[MAX_M] = {0.f, 0.f};
        auto fold_max = [&](int mrow, const float4& v) {
            const float a4[4] = {fabsf(v.x), fabsf(v.y), fabsf(v.z), fabsf(v.w)};
            float mx = 0.0f;
#pragma unroll
            for (int e = 0; e < 4; ++e) mx = (a4[e] <= 3.0e38f) ? fmaxf(mx, a4[e]) : __int_as_float(0x7f800000);  // NaN or inf poisons the slice
            if (mrow == 0) mx_row[0] = fmaxf(mx_row[0], mx);
            else mx_row[1] = fmaxf(mx_row[1], mx);
        };
        {
            int mrow = 0, c = 0;   // item i = (mrow, c), advanced without divisions
#pragma unroll
            for (int i = 0; i < XV; ++i) {
                const int k = item_k(c);
                xv[i] = (i < items && k < p.K) ? load_x4(p, m_base + mrow, k) : make_float4(0.f, 0.f, 0.f, 0.f);
                if constexpr (GC) {
                    const bool live = i < items && k < p.K;
                    const float4 s4 = live ? __ldg(reinterpret_cast<const float4*>(gs + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    const float4 b4 = live ? __ldg(reinterpret_cast<const float4*>(gb + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    fold_group(mrow, xv[i], s4, b4, true);
                }
                if (++c == p.nch) { c = 0; ++mrow; }
            }
            mrow = 0; c = 0;
#pragma unroll
            for (int i = 0; i < XV; ++i) {
                if (i < items) fold_max(mrow, xv[i]);
                if (++c == p.nch) { c = 0; ++mrow; }
            }
            for (int i0 = XV; i0 < items; i0 += 4) {   // four loads in flight per trip
                float4 v[4];
                int mr[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int k = item_k(c);
                    mr[u] = mrow;
                    const bool live = i0 + u < items && k < p.K;
                    v[u] = live ? load_x4(p, m_base + mrow, k) : make_float4(0.f, 0.f, 0.f, 0.f);
                    if constexpr (GC)
                        if (live) fold_group(mrow, v[u], __ldg(reinterpret_cast<const float4*>(gs + k)), __ldg(reinterpret_cast<const float4*>(gb + k)), true);
                    if (++c == p.nch) { c = 0; ++mrow; }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (i0 + u < items) fold_max(mr[u], v[u]);
            }
        }
        if (threadIdx.x == 0) GDBG(2);
        float sc_row[MAX_M] = {1.f, 1.f};    // s: |x| * s <= 127 over the slice
        double fac_row[MAX_M] = {0.0, 0.0};   // 1/s * 128^-3: powers of two, the product is exact
#pragma unroll
        for (int mm = 0; mm < MAX_M; ++mm) {
            if (mm < Mrows) {
                float v = mx_row[mm];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
                int e2 = 0;   // s = 2^e2
                if (v >= 1.0e-30f && v <= 3.0e38f) {
                    const int e = (int)((__float_as_uint(v) >> 23) & 0xffu) - 126;   // v = f * 2^e, f in [0.5, 1)
                    e2 = 7 - e;                                                       // v * 2^e2 in [64, 128)
                    if (v * __uint_as_float((uint32_t)(127 + e2) << 23) > 127.0f) --e2;
                } else if (v > 0.0f && v <= 3.0e38f) {
                    int e;
                    frexpf(v, &e);
                    e2 = 7 - e > 120 ? 120 : 7 - e;   // tiny slices: any power of two that keeps |x * s| <= 127 will do
                }
                const bool finite = v <= 3.0e38f;
                sc_row[mm] = finite ? __uint_as_float((uint32_t)(127 + e2) << 23) : 0.0f;   // a poisoned slice: zero digits ...
                // ... and NaN outputs.  2^(-e2 - 21) as a double, built from its exponent field
                fac_row[mm] = finite ? __longlong_as_double((long long)(1023 - e2 - 21) << 52) : (double)__int_as_float(0x7fc00000);
            }
        }
        if constexpr (GC) {
#pragma unroll
            for (int mm = 0; mm < MAX_M; ++mm)
                if (mm < Mrows)
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) cb_row[mm] += __shfl_xor_sync(0xffffffffu, cb_row[mm], off);
        }
        if (threadIdx.x == 0) GDBG(9);
        // digits of one item -> the warp's corner: column 4*m + i holds digit i (0 = most significant)
        auto emit = [&](int mrow, int c, const float4& v) {
            const float sm = mrow == 0 ? sc_row[0] : sc_row[1];
            uint8_t* at = dig + (size_t)(4 * mrow) * p.dstride + (size_t)c * KB + lane * 4;
            if (p.D == 4) emit_digits<4>(v.x * sm, v.y * sm, v.z * sm, v.w * sm, at, p.dstride);
            else emit_digits<3>(v.x * sm, v.y * sm, v.z * sm, v.w * sm, at, p.dstride);
        };
        {
            int mrow = 0, c = 0;   // item i = (mrow, c), advanced without divisions
#pragma unroll
            for (int i = 0; i < XV; ++i) {
                if (i < items) emit(mrow, c, xv[i]);   // beyond K the held value is zero: zero digits
                if (++c == p.nch) { c = 0; ++mrow; }
            }
            for (int i0 = XV; i0 < items; i0 += 4) {   // four loads in flight per trip
                float4 v[4];
                int mr[4], cc[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int k = item_k(c);
                    mr[u] = mrow;
                    cc[u] = c;
                    const bool live = i0 + u < items && k < p.K;
                    v[u] = live ? load_x4(p, m_base + mrow, k) : make_float4(0.f, 0.f, 0.f, 0.f);
                    if constexpr (GC)
                        if (live) fold_group(mrow, v[u], __ldg(reinterpret_cast<const float4*>(gs + k)), make_float4(0.f, 0.f, 0.f, 0.f), false);
                    if (++c == p.nch) { c = 0; ++mrow; }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (i0 + u < items) emit(mr[u], cc[u], v[u]);
            }
        }
        __syncwarp();
        if (threadIdx.x == 0) GDBG(3);
        const double fac = (j >> 1) == 0 ? fac_row[0] : fac_row[1];   // of the activation row this lane folds (m = j / 2)
        [[maybe_unused]] const double cbw = (j >> 1) == 0 ? cb_row[0] : cb_row[1];   // GC: this K slice's bias term of that row

        // ---- main loop, software-pipelined over the stages ----
        const bool b_live = g8 < p.R;
        const uint8_t* dig_b = dig + (size_t)g8 * p.dstride + 32 * j;
        int acc[4][4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[q][e] = 0;
        int g = 0, c = 0;
        // four MMAs of one stage (eight consecutive k-bytes per MMA and lane, the same bytes of A and of B, so the
        // products line up), four independent accumulators; then the end of a row group if it is one
        auto consume = [&](const uint4 (&w)[4]) {
            uint4 d0 = make_uint4(0, 0, 0, 0), d1 = d0;   // the matching 32 digit bytes of chunk c, digit column g8
            if (b_live) {
                d0 = *reinterpret_cast<const uint4*>(dig_b + (size_t)c * KB);
                d1 = *reinterpret_cast<const uint4*>(dig_b + (size_t)c * KB + 16);
            }
            if constexpr (GC) {
                mma_u8s8(acc[0], w[0].x, w[2].x, w[0].y, w[2].y, d0.x, d0.y);
                mma_u8s8(acc[1], w[0].z, w[2].z, w[0].w, w[2].w, d0.z, d0.w);
                mma_u8s8(acc[2], w[1].x, w[3].x, w[1].y, w[3].y, d1.x, d1.y);
                mma_u8s8(acc[3], w[1].z, w[3].z, w[1].w, w[3].w, d1.z, d1.w);
            } else {
                mma_s8(acc[0], w[0].x, w[2].x, w[0].y, w[2].y, d0.x, d0.y);
                mma_s8(acc[1], w[0].z, w[2].z, w[0].w, w[2].w, d0.z, d0.w);
                mma_s8(acc[2], w[1].x, w[3].x, w[1].y, w[3].y, d1.x, d1.y);
                mma_s8(acc[3], w[1].z, w[3].z, w[1].w, w[3].w, d1.z, d1.w);
            }
            if (++c == p.nch) {
                // accumulator element e: weight row g8 (e = 0, 1) or g8 + 8 (e = 2, 3), digit column 2j + (e & 1).
                // Columns 4m .. 4m+3 are the digits of activation row m, most significant first: lane pair (2m, 2m+1).
                long long v[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int hi = acc[0][2 * h] + acc[1][2 * h] + acc[2][2 * h] + acc[3][2 * h];
                    const int lo = acc[0][2 * h + 1] + acc[1][2 * h + 1] + acc[2][2 * h + 1] + acc[3][2 * h + 1];
                    v[h] = (long long)hi * 128 + lo;
                }
#pragma unroll
                for (int q = 0; q < 4; ++q)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[q][e] = 0;
                const long long p0 = __shfl_xor_sync(0xffffffffu, v[0], 1), p1 = __shfl_xor_sync(0xffffffffu, v[1], 1);
                // park this slice's sums of the group for the reducer: [buf][warp][m][16 rows]
                const int b = g & 1;
                if (g >= 2 && !mbar_wait(&freeb[b], (((uint32_t)g >> 1) - 1u) & 1u, abort_flag, p.status, 34)) ok = false;
                if (ok) {
                    if (!(j & 1) && (j >> 1) < Mrows) {
                        double* dst = sPart + (size_t)(b * GW + warp) * 32 + (j >> 1) * 16 + g8;
                        double o0 = (double)(v[0] * 16384 + p0) * fac, o1 = (double)(v[1] * 16384 + p1) * fac;
                        if constexpr (GC) { o0 += cbw; o1 += cbw; }
                        dst[0] = o0;
                        dst[8] = o1;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&done[b]);
                }
                c = 0;
                ++g;
            }
        };
        if (threadIdx.x == 0) GDBG(4);
        for (int i = 0; ok && i < total; i += 2) {   // wA holds stage i, wB stage i + 1
            consume(wA);
            if (threadIdx.x == 0 && i < 12) GDBG(10 + (i >> 1));
            if (!ok) break;
            if (i + 2 < total) {
                fetch(wA);
                if (!ok) break;
            }
            if (i + 1 >= total) break;
            consume(wB);
            if (!ok) break;
            if (i + 3 < total) fetch(wB);
        }
        if (threadIdx.x == 0) GDBG(5);
    }
}

template <bool GC>
int launch_gm(rusty_cuda_ctx* ctx, const CUtensorMap& map_w, const GmParams& p, dim3 grid, size_t smem) {
    auto kern = gemv_mma_kernel<GC>;
    cudaError_t e = rusty::ensure_dynamic_smem((const void*)kern, ctx->device, smem);
    if (e != cudaSuccess) return rusty::check_cuda(ctx, e, "gemv_mma: cudaFuncSetAttribute");
    cudaError_t le = launch_pdl(kern, grid, dim3(GM_THREADS), smem, ctx->stream, map_w, p);
    if (le != cudaSuccess) return rusty::check_cuda(ctx, le, "gemv_mma");
    return rusty::after_launch(ctx, "gemv_mma");
}

// Shared-memory plan: digit planes + partials + scale cache + barriers are fixed by the shape; the rest of the budget
// is the ring of weight stages.
bool plan_smem(const rusty_cuda_ctx* ctx, const rusty::QLinearArgs& a, int* stages, size_t* smem, int* D, int* R, int* nch, int* sc_cap) {
    const bool gc = a.qmode == rusty::QMODE_AFFINE_GC;
    const int M = a.M > (uint32_t)MAX_M ? MAX_M : (int)a.M;   // (GC: more rows go as passes of two)
    *D = (a.x_dtype == RUSTY_CUDA_F32 || gc) ? 4 : 3;   // (GC: x times a group scale is a full f32 whatever x was)
    *R = 4 * M;
    *nch = (int)((a.K + KC - 1) / KC);
    const int sms = ctx->sm_count > 0 ? ctx->sm_count : 1;
    const int units = (int)((a.N + 1) / 2);
    const int grid = units < sms ? units : sms;
    const int rows_max = gc ? gc_rows_per_cta(ctx, a.N, a.M) : 2 * ((units + grid - 1) / grid);
    *sc_cap = gc ? 0 : rows_max < 4096 ? rows_max : 4096;
    const size_t dig = (size_t)GW * *R * ((size_t)*nch * KB + 16);   // one corner per warp
    const size_t part = (size_t)2 * GW * 32 * 8;
    const size_t fixed = dig + part + (size_t)*sc_cap * 4 + 1024;
    // Half of the SM at most while the kernel is short (the next kernel's CTA then sits beside this one and lands its
    // weights while this one computes); a CTA that streams many times the ring takes the whole SM: depth matters more.
    const size_t optin = ctx->smem_optin > 2048 ? ctx->smem_optin - 2048 : 0;
    const bool longrun = (size_t)rows_max * a.K > 6 * (optin / 2) || fixed + 1024 + 2 * (size_t)STAGE_BYTES > optin / 2;
    const size_t budget = longrun ? optin : optin / 2;
    if (budget < fixed + 1024 + 2 * (size_t)STAGE_BYTES) return false;
    int s = (int)((budget - fixed - 1024) / STAGE_BYTES);
    if (s > 12) s = 12;
    *stages = s;
    *smem = 1024 + (size_t)s * STAGE_BYTES + fixed + (size_t)(2 * s + 4) * 8;   // + slack to align the ring to 1 KiB
    return true;
}

}  // namespace

namespace rusty {

bool gemv_mma_supported(const rusty_cuda_ctx* ctx, const QLinearArgs& a) {
    const bool gc = a.qmode == QMODE_AFFINE_GC;
    if (a.layout != RUSTY_CUDA_LAYOUT_NK || (a.qmode != RUSTY_CUDA_QMODE_SYM_ROW && !gc)) return false;
    if (gc ? (a.N % 64 != 0 || a.act || a.M < 1) : (a.M < 1 || a.M > (uint32_t)MAX_M)) return false;
    if (a.K % 128 != 0 || !encode_tiled_fn()) return false;   // the weight is read as [K/128][rows][128 bytes] by TMA
    static const bool off = getenv("RUSTY_NO_GEMV_MMA") != nullptr;
    if (off) return false;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.x) & 15) != 0) return false;
    int stages, D, R, nch, sc_cap;
    size_t smem;
    return plan_smem(ctx, a, &stages, &smem, &D, &R, &nch, &sc_cap);
}

int launch_gemv_mma(rusty_cuda_ctx* ctx, const QLinearArgs& a) {
    GmParams p{};
    size_t smem = 0;
    if (!plan_smem(ctx, a, &p.stages, &smem, &p.D, &p.R, &p.nch, &p.sc_cap))
        return fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "gemv_mma: the digit planes of K=%u do not fit shared memory", a.K);
    const bool gc = a.qmode == QMODE_AFFINE_GC;
    p.W = a.w;
    p.scales = a.scales;
    p.gscale = gc ? a.scales : nullptr;
    p.gbias = gc ? a.biases : nullptr;
    p.x = a.x;
    p.y = a.y;
    p.M = (int)a.M;
    p.N = (int)a.N;
    p.K = (int)a.K;
    p.dstride = p.nch * KB + 16;
    p.units = (p.N + 1) / 2;
    p.ldy = (int)a.ldy;
    p.y_col0 = (int)a.y_col0;
    if (a.push && a.push->nranks > 1)
        for (int g = 0; g < a.push->nranks && g < PEER_MAX_RANKS; ++g)
            if (g != a.push->rank) p.peer_delta[p.n_peers++] = a.push->delta[g];
    p.act = a.act;
    p.x_bf16 = a.x_dtype == RUSTY_CUDA_BF16;
    p.y_bf16 = a.y_dtype == RUSTY_CUDA_BF16;
    p.status = ctx->status_dev;
    p.dbg = nullptr;
    if (ctx->tc_dbg) {  // development builds: one timeline region (152 CTAs x 16 slots) per launch, round robin
        p.dbg = (long long*)ctx->tc_dbg + (size_t)(ctx->tc_dbg_slots > 0 ? ctx->tc_dbg_seq % ctx->tc_dbg_slots : 0) * 152 * 16;
        ctx->tc_dbg_seq++;
    }
    int grid = ctx->sm_count;
    if (grid > p.units) grid = p.units;
    CUtensorMap map_w;
    if (!make_map_u8_rows_by_kblocks(&map_w, a.w, a.N, a.K, STAGE_ROWS, KC / 128))
        return fail(ctx, RUSTY_CUDA_ERR_KERNEL_EXECUTION, "gemv_mma: cuTensorMapEncodeTiled failed");
    if (!gc) return launch_gm<false>(ctx, map_w, p, dim3(grid), smem);
    // group-column affine weights: one CTA per 32 rows and pair of activation rows (at most 65535 pairs per launch)
    const uint32_t pairs = (a.M + MAX_M - 1) / MAX_M;
    const size_t xs = p.x_bf16 ? 2 : 4, ys = p.y_bf16 ? 2 : 4;
    for (uint32_t p0 = 0; p0 < pairs; p0 += 65535u) {
        GmParams q = p;
        q.gc_rows = gc_rows_per_cta(ctx, a.N, a.M);
        const uint32_t np = pairs - p0 < 65535u ? pairs - p0 : 65535u, m0 = p0 * MAX_M;
        q.M = (int)(a.M - m0 < np * MAX_M ? a.M - m0 : np * MAX_M);
        q.x = reinterpret_cast<const char*>(a.x) + (size_t)m0 * a.K * xs;
        q.y = reinterpret_cast<char*>(a.y) + (size_t)m0 * a.ldy * ys;
        if (a.N / q.gc_rows > 148 || pairs > 1) q.dbg = nullptr;   // (development builds: a timeline region holds 148 CTAs of one launch)
        int rc = launch_gm<true>(ctx, map_w, q, dim3(a.N / q.gc_rows, np), smem);
        if (rc) return rc;
    }
    return RUSTY_CUDA_OK;
}

}  // namespace rusty
