// PTX wrappers shared by the tensor-core kernels: mbarrier, TMA, tcgen05 / TMEM,
// programmatic dependent launch, bounded waits.
#pragma once

#include <cuda.h>
#include <cstdlib>

#include "internal.h"

namespace rusty_tc {
using rusty::PeerPush;
using rusty::PEER_SYNC_SLOTS;
using rusty::NormArgs;
using rusty::PEER_MAX_RANKS;

constexpr long long WAIT_LIMIT_CYCLES = 8000000000ll;  // ~4 s of SM clock

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// 16 bytes of shared memory as a volatile asm statement, so that the load stays in front of the mbarrier arrive that
// hands a ring slot back.  Written as plain C++ loads, the fragment loads of the GEMV were moved behind the arrive, down to
// the first use of the values: the registers then held what the slot had been refilled with in the meantime.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// Bounded wait.  Returns false (after raising the status word) when the limit
// expires or another role of this CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          rusty_cuda_dev_status* status, unsigned site) {
    long long t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 255u) {
            if (*abort_flag) return false;
            if (t0 == 0) t0 = clock64();
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                if (atomicExch(&status->timeout_flag, 1u) == 0u) status->timeout_where = site;
                return false;
            }
        }
    }
}
// ---- activations -> signed 7-bit digits --------------------------------------
// One activation times its row scale (|v| <= 127, exact: the scale is a power of two) -> the integer
// T = round(v * 128^(D-1)) -> D balanced digits, T = ((d_top * 128 + ...) * 128 + d_0) with d_top in [-127, 127] and
// the others in [-64, 63].  Returned as bytes: byte i = digit i for i < D-1 (least significant first), byte D-1 = top.
template <int D>
__device__ __forceinline__ uint32_t digits_of(float v) {
    const int t = __float2int_rn(v * (D == 4 ? 2097152.0f : 16384.0f));
    // bias: every low 7-bit field becomes digit + 64; digit = field - 64 as a byte is the field with bit 6 flipped and
    // copied into bit 7 (three bit operations for all fields at once)
    if (D == 4) {
        const uint32_t u = (uint32_t)(t + (64 + 64 * 128 + 64 * 128 * 128));
        const uint32_t w = (u & 0x7Fu) | ((u << 1) & 0x7F00u) | ((u << 2) & 0x7F0000u) | ((u << 3) & 0xFF000000u);
        const uint32_t f = w ^ 0x00404040u;
        return f | ((f & 0x00404040u) << 1);
    }
    const uint32_t u = (uint32_t)(t + (64 + 64 * 128));
    const uint32_t w = (u & 0x7Fu) | ((u << 1) & 0x7F00u) | ((u << 2) & 0xFF0000u);
    const uint32_t f = w ^ 0x00004040u;
    return f | ((f & 0x00004040u) << 1);
}

// ---- exchange by peer stores ------------------------------------------------
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Called by the 32 lanes of ONE warp of block b (b < PEER_SYNC_SLOTS) after griddepcontrol.wait: tells the other ranks
// that this rank has finished everything before this kernel (its pushed stores included) and waits until the same block
// of every other rank has said so.  Lane g talks to rank g: one add into its arena, one polled cell of ours, all
// ranks in parallel.  Gives up after pp.wait_ns, records `site` in the status word and returns false; the caller
// carries on.  The caller follows it with a block-wide barrier.
__device__ __forceinline__ bool peer_sync_block(const PeerPush& pp, int b, unsigned site, long long* tl = nullptr) {
    if (pp.nranks <= 1) return true;
    const int lane = threadIdx.x & 31;
    unsigned int* mine = pp.ctl + PEER_MAX_RANKS * PEER_SYNC_SLOTS + b;
    unsigned int c = 0;
    if (lane == 0) {
        c = *reinterpret_cast<volatile unsigned int*>(mine) + 1u;   // only this block ever touches its cell
        *reinterpret_cast<volatile unsigned int*>(mine) = c;
    }
    c = __shfl_sync(0xffffffffu, c, 0);
#ifdef RUSTY_TIMELINE
    if (tl && lane == 0) tl[4] = (long long)globaltimer_ns();
#endif
    bool ok = true;
    if (lane < pp.nranks && lane != pp.rank) {
        // What this rank stored before (its pushes included) was performed when the kernels that stored it completed,
        // which is what let this kernel pass griddepcontrol.wait, so a relaxed add is enough.  (A release here is a
        // system-scope fence: measured at 3-4 us per operation while the next kernel's weight prefetch is in flight.)
        asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(pp.peer_ctl[lane] + pp.rank * PEER_SYNC_SLOTS + b) : "memory");
        const unsigned long long t0 = globaltimer_ns();
#ifdef RUSTY_TIMELINE
        if (tl) tl[5] = (long long)t0;
        int polls = 0;
#endif
        while ((int)(ld_acquire_sys_u32(pp.ctl + lane * PEER_SYNC_SLOTS + b) - c) < 0) {
#ifdef RUSTY_TIMELINE
            if (tl) tl[6] = ++polls;
#endif
            if (globaltimer_ns() - t0 > pp.wait_ns) {
                if (atomicExch(&pp.status->timeout_flag, 1u) == 0u) pp.status->timeout_where = site;
                ok = false;
                break;
            }
            __nanosleep(64);
        }
    }
    return __all_sync(0xffffffffu, ok);
}

// Programmatic dependent launch: let the next kernel in the stream start its
// prologue now / wait until everything earlier in the stream has finished and
// its writes are visible.  Both are no-ops for a kernel launched the plain way.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int32_t c0, int32_t c1, uint64_t* bar,
                                            uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int32_t c0, int32_t c1, int32_t c2, uint64_t* bar,
                                            uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4, %5}], [%2], %6;"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* map, int32_t c0, int32_t c1, int32_t c2) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0),
                 "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, int8 x int8 -> int32
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// mbarrier arrives once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t addr, int32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(addr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, rows of 128 bytes,
// 8-row groups 1024 bytes apart (descriptor version 1 = Blackwell).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address
    d |= (uint64_t)1 << 16;                         // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                         // version
    d |= (uint64_t)2 << 61;                         // SWIZZLE_128B
    return d;
}


// D[tmem] (+)= A[tmem] * B[smem]^T, 16-bit floats -> f32 (A: M x 16 elements packed two per 32-bit column)
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 consecutive 32-bit columns of this thread's TMEM lane <- registers
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        :
        : "r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
          "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
          "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(addr));
}

// Shared-memory matrix descriptor helpers are above; tensor-map encoding (host):
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();
// [rows, K] uint8 row-major, boxes of box_rows x 128 bytes, 128-byte swizzle, zero fill outside.
bool make_map_u8(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows);
// The same matrix seen as [K/128 k-blocks][rows][128 bytes] (K % 128 == 0): one box = box_kblocks x box_rows lines of
// 128 bytes, laid out in shared memory k-block by k-block, 128-byte swizzle (16-byte chunk c of row r sits at
// c ^ (r & 7)); coordinates are (0, row, k-block); zero fill outside.
bool make_map_u8_rows_by_kblocks(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows, uint32_t box_kblocks);
// [rows, K] bf16 row-major, boxes of box_rows x 64 elements (128 bytes), 128-byte swizzle, zero fill outside.
bool make_map_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows);

// Launch with programmatic stream serialisation: the kernel may begin while its
// predecessor in the stream is still draining; it orders itself with
// griddepcontrol.wait.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool no_pdl = getenv("RUSTY_NO_PDL") != nullptr;  // tuning aid: plain stream order
    cfg.numAttrs = no_pdl ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace rusty_tc
