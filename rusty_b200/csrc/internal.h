// Internal definitions shared by the translation units of librusty_cuda.
// Nothing here is part of the C ABI (see include/rusty_cuda.h).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "rusty_cuda.h"

// Device-side status word shared by every kernel that can give up on a bounded
// wait.  Lives in pinned, mapped host memory so the host can read it without a
// copy and a kernel can set it with a plain store.
struct rusty_cuda_dev_status {
    unsigned int timeout_flag;   // != 0: some bounded wait ran out
    unsigned int timeout_where;  // kernel-defined site id of the first give-up
    unsigned int bad_index_flag; // != 0: a gather met an index outside its table (the row was written as zeros)
    unsigned int bad_index_value;  // the first such index
};

struct rusty_cuda_ctx {
    int device = -1;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    size_t smem_optin = 0;
    cudaStream_t stream = nullptr;
    std::string name;
    std::string last_error;
    std::atomic<uint64_t> launches{0};
    // exact-byte-size bins, like rusty-backend/src/pool.rs
    std::mutex pool_mu;
    std::unordered_map<size_t, std::vector<void*>> pool_bins;
    // device-visible status word (pinned + mapped)
    rusty_cuda_dev_status* status_host = nullptr;
    rusty_cuda_dev_status* status_dev = nullptr;
    // workspace of the tensor-core path (digit planes, split-K sums); reserved when
    // the first fused linear is created, never inside a forward call
    void* tc_ws = nullptr;
    size_t tc_ws_bytes = 0;
    void* tc_dbg = nullptr;  // optional kernel timeline buffer (development aid)
    int tc_dbg_seq = 0, tc_dbg_slots = 0;
    // stream capture in progress (rusty_cuda_graph_begin .. _end)
    bool capturing = false;
    // Releases that arrive while a capture is open (a host-language destructor may run at any time) are parked here:
    // freeing or synchronising would invalidate the capture.  rusty_cuda_graph_end performs them.
    std::vector<void*> deferred_free;
    std::vector<struct rusty_cuda_graph*> deferred_graphs;
    uint64_t launches_at_capture = 0;
};

struct rusty_cuda_buf {
    rusty_cuda_ctx* ctx = nullptr;
    void* ptr = nullptr;
    size_t bytes = 0;
    bool pooled = false;
    bool borrowed = false;  // storage owned by someone else (IPC import / wrap)
    std::atomic<int> refs{1};
};

struct rusty_cuda_graph {
    rusty_cuda_ctx* ctx = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t kernels = 0;  // kernel launches recorded in the graph
};

struct rusty_cuda_event {
    rusty_cuda_ctx* ctx = nullptr;
    cudaEvent_t ev = nullptr;
};

struct rusty_cuda_qlinear {
    rusty_cuda_ctx* ctx = nullptr;
    rusty_cuda_buf* weight = nullptr;
    rusty_cuda_buf* scales = nullptr;
    rusty_cuda_buf* biases = nullptr;
    uint32_t N = 0, K = 0;
    int layout = 0, qmode = 0;   // layout of `weight` as the kernels read it
    int given_layout = 0;        // layout the caller handed over ([in,out] weights with one scale per output are
                                 // re-laid-out to [out,in] once, at create: `weight` is then the library's own copy)
    int act = 0;  // RUSTY_CUDA_ACT_*: applied to pairs of output features in the kernel's epilogue
};

namespace rusty {

int fail(rusty_cuda_ctx* ctx, int code, const char* fmt, ...);
int check_cuda(rusty_cuda_ctx* ctx, cudaError_t e, const char* what);

// RAII: make the context's device current for the duration of a call.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = (cudaSetDevice(dev) == cudaSuccess);
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

inline void count_launch(rusty_cuda_ctx* ctx, uint64_t n = 1) { ctx->launches.fetch_add(n, std::memory_order_relaxed); }

// Checks the launch error of the kernel just enqueued.
int after_launch(rusty_cuda_ctx* ctx, const char* kernel);

// Raise a kernel's dynamic shared-memory limit on `device` (current) to at least `bytes`.  The per-(kernel, device)
// high-water mark sits in one mutex-guarded table keyed by the full device ordinal: contexts on different host
// threads may launch the same kernel at once.
cudaError_t ensure_dynamic_smem(const void* kernel, int device, size_t bytes);

// Kernel launchers implemented in the .cu files -----------------------------
int launch_matmul_f32(rusty_cuda_ctx* ctx, const float* a, const float* b, float* out, uint32_t M, uint32_t K,
                      uint32_t N);
int launch_matmul_bt_f32(rusty_cuda_ctx* ctx, const float* a, const float* b, float* out, uint32_t M, uint32_t K,
                         uint32_t N);
int launch_dequantize_u8(rusty_cuda_ctx* ctx, const uint32_t* in, size_t in_words, size_t n_in, float* out,
                         size_t n_out);
int launch_affine_dequantize_g64(rusty_cuda_ctx* ctx, const uint8_t* w, const float* scales, const float* biases,
                                 float* out, size_t n);

// Exchange by peer stores (peer.cu): what a kernel needs to write its outputs into the other ranks' copies of y and
// to keep step with them.  Every rank owns an arena with the same layout; rank g's arena is mapped here at peer_base[g].
// All ranks enqueue the same sequence of operations on an arena, and every operation BEGINS with a kernel whose blocks
// (at most PEER_SYNC_SLOTS of them, the same number on every rank) meet their namesakes on the other ranks: block b adds
// one to cell [rank][b] of every other arena, then waits until cells [g][b] of its own arena have all reached its own
// count.  A block gets there only after griddepcontrol.wait, i.e. after everything this rank enqueued before has
// finished and its stores have been performed, so "rank g's block b has arrived" means "what rank g pushed in earlier
// operations has landed here, and rank g no longer reads what this operation overwrites".
//   ctl[g * PEER_SYNC_SLOTS + b]               arrivals of rank g's block b (written by rank g)
//   ctl[PEER_MAX_RANKS * PEER_SYNC_SLOTS + b]  this rank's own count for block b (local)
constexpr int PEER_MAX_RANKS = 8;
constexpr int PEER_SYNC_SLOTS = 64;
struct PeerPush {
    int nranks, rank;                            // nranks <= 1: nothing to push, nothing to wait for
    unsigned int* ctl;                           // this rank's control block (PEER_MAX_RANKS + 1) * PEER_SYNC_SLOTS words
    unsigned int* peer_ctl[PEER_MAX_RANKS];      // every rank's control block as mapped in this process (own included)
    long long delta[PEER_MAX_RANKS];             // bytes from an address in this arena to the same place in rank g's
    unsigned long long wait_ns;                  // limit of a wait for the other ranks
    rusty_cuda_dev_status* status;
};

struct QLinearArgs {
    const uint8_t* w;
    const float* scales;
    const float* biases;
    uint32_t N, K;  // N: output features computed by this call (rows of w it reads)
    int layout, qmode;
    const void* x;
    int x_dtype;
    uint32_t M;
    void* y;
    int y_dtype;
    uint32_t ldy;    // row stride of y in elements (>= N)
    uint32_t y_col0; // first output column written (for shards writing into a wider y)
    // RUSTY_CUDA_ACT_SWIGLU_PAIRS: rows 2j / 2j+1 of w are gate_j / up_j; the kernel writes silu(gate)*up into column
    // (y_col0 + 2j) / 2, so y has N/2 columns per call, ldy counts those, and y_col0 (even) still counts rows of w
    int act;
    // Non-null: y lies in a peer arena; the kernel also stores every output into the other ranks' arenas and
    // signals them (honoured by the kernels for which qlinear_pushes_fused() is true).
    const PeerPush* push = nullptr;
    // Non-null: the activations are RMSNorm(x [+ residual]) * weight, computed by the kernel that prepares them for
    // the tensor cores (honoured where qlinear_norm_fused() is true; x, residual and the outputs are f32 [M, K]).
    const struct NormArgs* norm = nullptr;
    // Non-null: y = residual + Linear(x); same element type, row stride and column window as y (may be y itself).
    // Honoured by the tensor-core kernels (qlinear_residual_fused()); never together with the pair activation.
    const void* residual = nullptr;
};

// RMSNorm in front of a Linear (norm_embed.cu has the formula and its reference lines).
struct NormArgs {
    const float* residual;  // null: plain RMSNorm of x
    const float* weight;    // [K]
    float eps;
    float* normed;          // null, or where the normalised activations are also written
    float* sum;             // null, or where x + residual is also written (needs residual)
};
int launch_rms_norm(rusty_cuda_ctx* ctx, const float* x, const float* residual, const float* weight, float* out, float* sum_out,
                    uint32_t M, uint32_t K, float eps);
// whether the Linear's own activation pre-pass can apply the norm for this call
bool qlinear_norm_fused(const rusty_cuda_ctx* ctx, const rusty_cuda_qlinear* ql, int x_dtype, uint32_t M, int y_dtype);
bool tc_norm_fused(uint32_t M, uint32_t K);
// out[n][k] = in[k][n], bytes (the one-time re-layout of an [in,out] weight)
int launch_transpose_u8(rusty_cuda_ctx* ctx, const uint8_t* in, uint8_t* out, uint32_t K, uint32_t N);
int launch_transpose_f32(rusty_cuda_ctx* ctx, const float* in, float* out, uint32_t K, uint32_t N);
// Internal quantisation mode of a re-laid-out AFFINE_G64 [in,out] weight: bytes stored [out,in], scales and biases
// stored [N/64][K] (one pair per 64 consecutive OUTPUT features and input k).  Never crosses the C ABI.
constexpr int QMODE_AFFINE_GC = 64;
int launch_residual_add(rusty_cuda_ctx* ctx, const void* a, const void* b, void* out, size_t n, int y_dtype);
bool qlinear_residual_fused(const rusty_cuda_qlinear* ql, int x_dtype, uint32_t M, int y_dtype);

bool gemv_supported(const rusty_cuda_ctx* ctx, const QLinearArgs& a);
int launch_gemv(rusty_cuda_ctx* ctx, const QLinearArgs& a);

// One or two activation rows on the warp-level integer tensor-core path, weights staged by TMA (gemv_mma.cu).
bool gemv_mma_supported(const rusty_cuda_ctx* ctx, const QLinearArgs& a);
int launch_gemv_mma(rusty_cuda_ctx* ctx, const QLinearArgs& a);

// Tensor-core (tcgen05 / TMEM) path.
bool tc_supported(const rusty_cuda_ctx* ctx, const QLinearArgs& a);
uint32_t tc_min_rows();
int tc_workspace_reserve(rusty_cuda_ctx* ctx);
void tc_workspace_release(rusty_cuda_ctx* ctx);
void tc_workspace_clear_pieces(rusty_cuda_ctx* ctx);
int tc_workspace_check_guards(rusty_cuda_ctx* ctx, cudaError_t* err);
void tc_workspace_sums(rusty_cuda_ctx* ctx, float** sums, size_t* sums_bytes, unsigned int** counters, size_t* cnt_bytes);
int launch_tc(rusty_cuda_ctx* ctx, const QLinearArgs& a);
bool tc_pushes_fused(uint32_t M);

// Prefill path: int8 -> fp16 into tensor memory, bf16 activations (tcgen05 kind::f16).
bool f16tc_supported(const rusty_cuda_ctx* ctx, const QLinearArgs& a);
int launch_f16tc(rusty_cuda_ctx* ctx, const QLinearArgs& a);
uint32_t f16tc_min_rows();

// True when the kernel chosen for this shape stores into the peers' arenas itself.
bool qlinear_pushes_fused(const rusty_cuda_qlinear* ql, int x_dtype, uint32_t M, int y_dtype);
// True when that kernel also meets the other ranks itself (else rusty_cuda_qlinear_forward_pushed puts the wait kernel in front).
bool qlinear_meets_in_kernel(const rusty_cuda_qlinear* ql, int x_dtype, uint32_t M, int y_dtype);
const char* qlinear_plan(const rusty_cuda_qlinear* ql, int x_dtype, uint32_t M, int y_dtype);
// Forward into columns [y_col0, y_col0 + N) of a y whose rows are ldy elements apart.
int qlinear_forward_cols(rusty_cuda_ctx* ctx, const rusty_cuda_qlinear* ql, const rusty_cuda_buf* x, int x_dtype,
                         uint32_t M, rusty_cuda_buf* y, int y_dtype, uint32_t ldy, uint32_t y_col0,
                         const PeerPush* push = nullptr, const NormArgs* norm = nullptr, const rusty_cuda_buf* residual = nullptr);

}  // namespace rusty

#define RUSTY_REQUIRE_CTX(ctx)                                                                            \
    do {                                                                                                  \
        if (!(ctx)) return rusty::fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "%s: null context", __func__); \
    } while (0)
