/*
 * rusty_cuda.h — C ABI of the B200 (sm_100a) backend for rusty's
 * quantized-linear path.
 *
 * Every entry point is what a Rust `extern "C"` block inside rusty-backend
 * would bind to replace the wgpu implementation of the same operation; the
 * reference interface each one stands in for is cited as file:line (paths
 * inside the rusty repository).
 *
 * Conventions
 *   - every function returns an int status (RUSTY_CUDA_OK == 0); nothing
 *     throws, aborts or exits.  `rusty_cuda_last_error` gives the text.
 *   - all operations enqueue on the context's single stream and return at
 *     once (rusty: one wgpu::Queue, one submit per op, order = call order).
 *     `rusty_cuda_buf_download` and `rusty_cuda_sync` are the only blocking
 *     calls, like `UnifiedTensor::to_vec`'s `device.poll(Wait)`.
 *   - the caller allocates every output buffer; no op allocates device memory
 *     (the reference's ops only allocate a 16-byte uniform).
 *   - one context per host thread per GPU.
 *   - there is no CPU fallback: without a CUDA device every call fails with
 *     RUSTY_CUDA_ERR_GPU_INITIALIZATION.
 */
#ifndef RUSTY_CUDA_H
#define RUSTY_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define RUSTY_CUDA_API __attribute__((visibility("default")))
#else
#define RUSTY_CUDA_API
#endif

/* Status codes, named after the variants of rusty-backend's BackendError
 * (rusty-backend/src/error.rs:13-61). */
enum {
    RUSTY_CUDA_OK = 0,
    RUSTY_CUDA_ERR_GPU_INITIALIZATION = 1, /* GpuInitialization / DeviceCreation */
    RUSTY_CUDA_ERR_MEMORY_ALLOCATION = 2,  /* MemoryAllocation / OutOfMemory */
    RUSTY_CUDA_ERR_INVALID_DIMENSIONS = 3, /* InvalidDimensions */
    RUSTY_CUDA_ERR_INVALID_DATA_TYPE = 4,  /* InvalidDataType */
    RUSTY_CUDA_ERR_BUFFER_OPERATION = 5,   /* BufferOperation (size/offset out of range) */
    RUSTY_CUDA_ERR_KERNEL_EXECUTION = 6,   /* KernelExecution (launch or async error) */
    RUSTY_CUDA_ERR_UNSUPPORTED = 7,        /* UnsupportedOperation */
    RUSTY_CUDA_ERR_DATA_TRANSFER = 8,      /* DataTransfer */
    RUSTY_CUDA_ERR_INVALID_OPERATION = 9,  /* InvalidOperation (null handle, wrong state) */
    RUSTY_CUDA_ERR_TIMEOUT = 10,           /* Timeout (a bounded device-side wait gave up) */
    RUSTY_CUDA_ERR_OTHER = 11
};

/* Element types.  rusty's DType has FP32 and FP16 only
 * (rusty-backend/src/lib.rs:56-76) and moves quantised bytes as untyped
 * buffers; the fused path needs to name them. */
enum {
    RUSTY_CUDA_F32 = 0,
    RUSTY_CUDA_F16 = 1,
    RUSTY_CUDA_BF16 = 2,
    RUSTY_CUDA_I8 = 3,
    RUSTY_CUDA_U8 = 4
};

/* Quantisation modes of a fused linear. */
enum {
    /* u8 weights, f32 scale and bias per group of 64 consecutive elements of
     * the flat row-major weight: the layout `affine_dequantize` consumes
     * (rusty-backend/src/kernels.wgsl:385-400, rusty-loader/src/lib.rs:155-218). */
    RUSTY_CUDA_QMODE_AFFINE_G64 = 0,
    /* signed int8 weights, one f32 scale per output feature, no bias. */
    RUSTY_CUDA_QMODE_SYM_ROW = 1
};

/* Storage order of a fused linear's weight. */
enum {
    RUSTY_CUDA_LAYOUT_NK = 0, /* [out, in]: the matmul_bt contraction (kernels.wgsl:234-242) */
    RUSTY_CUDA_LAYOUT_KN = 1  /* [in, out]: the matmul_tiled contraction (kernels.wgsl:16-54), rusty's Linear */
};

typedef struct rusty_cuda_ctx rusty_cuda_ctx;
typedef struct rusty_cuda_buf rusty_cuda_buf;
typedef struct rusty_cuda_qlinear rusty_cuda_qlinear;
typedef struct rusty_cuda_comm rusty_cuda_comm;
typedef struct rusty_cuda_graph rusty_cuda_graph;

/* ---- context: WgpuContext::new + ComputeEngine::new -----------------------
 * (rusty-backend/src/lib.rs:20-47, :343).  Owns the device, one stream, the
 * exact-size-bin buffer pool and the last-error text. */
RUSTY_CUDA_API int rusty_cuda_device_count(int* count);
RUSTY_CUDA_API int rusty_cuda_ctx_create(int device, rusty_cuda_ctx** out);
RUSTY_CUDA_API int rusty_cuda_ctx_destroy(rusty_cuda_ctx* ctx);
/* WgpuContext::adapter_info (lib.rs:49-52): "<name> (CUDA sm_XY)". */
RUSTY_CUDA_API int rusty_cuda_ctx_adapter_info(rusty_cuda_ctx* ctx, char* dst, size_t dst_len);
/* Text of the most recent failure on this context (or of the most recent
 * failure with no context when ctx is NULL).  Never NULL. */
RUSTY_CUDA_API const char* rusty_cuda_last_error(rusty_cuda_ctx* ctx);
/* device.poll(Maintain::Wait) (lib.rs:233): drain the stream; reports any
 * asynchronous kernel error and any device-side timeout flag. */
RUSTY_CUDA_API int rusty_cuda_sync(rusty_cuda_ctx* ctx);
/* The kernels' internal scratch regions are separated by guard zones that nothing may write.  Drains the stream,
 * reads the guards back and returns RUSTY_CUDA_ERR_KERNEL_EXECUTION if one was damaged (an out-of-bounds write by a
 * kernel of this library).  No counterpart in the reference (wgpu validates buffer bounds itself). */
RUSTY_CUDA_API int rusty_cuda_ctx_self_check(rusty_cuda_ctx* ctx);
/* Number of kernels this context has launched so far (host-side counter). */
RUSTY_CUDA_API int rusty_cuda_ctx_launch_count(rusty_cuda_ctx* ctx, uint64_t* count);
/* The context's CUDA stream as an opaque pointer (cudaStream_t), for callers
 * that record their own events on it. */
RUSTY_CUDA_API int rusty_cuda_ctx_stream(rusty_cuda_ctx* ctx, void** stream);

/* ---- buffers: UnifiedTensor's storage --------------------------------------
 * pooled != 0  : UnifiedTensor::empty (lib.rs:141-153) — taken from, and on the
 *                last release returned to, the exact-byte-size bin of the pool
 *                (rusty-backend/src/pool.rs:30-50); contents uninitialised.
 * pooled == 0  : UnifiedTensor::new / from_bytes (lib.rs:115-135, :165-190) —
 *                a fresh allocation freed on the last release.
 * Buffers are reference counted like the Arc<TensorData> they replace
 * (`reshaped` views share storage, lib.rs:198-213). */
RUSTY_CUDA_API int rusty_cuda_buf_alloc(rusty_cuda_ctx* ctx, size_t bytes, int pooled, rusty_cuda_buf** out);
RUSTY_CUDA_API int rusty_cuda_buf_retain(rusty_cuda_buf* buf);
RUSTY_CUDA_API int rusty_cuda_buf_release(rusty_cuda_buf* buf);
RUSTY_CUDA_API int rusty_cuda_buf_size(const rusty_cuda_buf* buf, size_t* bytes);
RUSTY_CUDA_API int rusty_cuda_buf_device_ptr(const rusty_cuda_buf* buf, void** ptr);
/* queue.write_buffer / create_buffer_init (lib.rs:110-112, :117-126). */
RUSTY_CUDA_API int rusty_cuda_buf_upload(rusty_cuda_ctx* ctx, rusty_cuda_buf* dst, size_t dst_offset,
                                         const void* src, size_t bytes);
/* UnifiedTensor::to_vec (lib.rs:215-240): copy back and wait. */
RUSTY_CUDA_API int rusty_cuda_buf_download(rusty_cuda_ctx* ctx, const rusty_cuda_buf* src, size_t src_offset,
                                           void* dst, size_t bytes);
/* ComputeEngine::copy_tensor (lib.rs:4019-4037): all of src to dst at a byte offset. */
RUSTY_CUDA_API int rusty_cuda_buf_copy(rusty_cuda_ctx* ctx, const rusty_cuda_buf* src, rusty_cuda_buf* dst,
                                       size_t dst_offset);
/* BufferPool::clear (pool.rs:52-55) and a count of idle pooled buffers. */
RUSTY_CUDA_API int rusty_cuda_pool_clear(rusty_cuda_ctx* ctx);
RUSTY_CUDA_API int rusty_cuda_pool_idle_count(rusty_cuda_ctx* ctx, size_t bytes, size_t* count);
/* Pinned host staging memory for callers that want asynchronous transfers. */
RUSTY_CUDA_API int rusty_cuda_host_alloc(size_t bytes, void** out);
RUSTY_CUDA_API int rusty_cuda_host_free(void* p);
/* Asynchronous variants of upload/download: `src`/`dst` should be pinned; the
 * call returns once the copy is enqueued. */
RUSTY_CUDA_API int rusty_cuda_buf_upload_async(rusty_cuda_ctx* ctx, rusty_cuda_buf* dst, size_t dst_offset,
                                               const void* src, size_t bytes);
RUSTY_CUDA_API int rusty_cuda_buf_download_async(rusty_cuda_ctx* ctx, const rusty_cuda_buf* src,
                                                 size_t src_offset, void* dst, size_t bytes);

/* ---- unfused operators: ComputeEngine methods ------------------------------
 * Dimensions are explicit because the C ABI carries no shape vector; the Rust
 * side passes the values the reference reads from the tensors' shapes. */
/* ComputeEngine::matmul -> WGSL matmul_tiled (lib.rs:4403-4453, kernels.wgsl:16-54):
 * out[M,N] = a[M,K] * b[K,N], f32. */
RUSTY_CUDA_API int rusty_cuda_matmul_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* a, const rusty_cuda_buf* b,
                                         rusty_cuda_buf* out, uint32_t M, uint32_t K, uint32_t N);
/* ComputeEngine::matmul_bt -> WGSL matmul_bt (lib.rs:4299-4349, kernels.wgsl:234-242):
 * out[M,N] = a[M,K] * b[N,K]^T, f32. */
RUSTY_CUDA_API int rusty_cuda_matmul_bt_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* a, const rusty_cuda_buf* b,
                                            rusty_cuda_buf* out, uint32_t M, uint32_t K, uint32_t N);
/* ComputeEngine::dequantize -> WGSL dequantize (lib.rs:4872-4899, kernels.wgsl:156-166):
 * `n_in` = product of the input tensor's shape (bytes to unpack); the input and
 * output array lengths that guard the shader's loads and stores are taken from
 * the buffers' sizes (in/4 words, out/4 floats). */
RUSTY_CUDA_API int rusty_cuda_dequantize_u8(rusty_cuda_ctx* ctx, const rusty_cuda_buf* in, rusty_cuda_buf* out,
                                            size_t n_in);
/* ComputeEngine::affine_dequantize -> WGSL affine_dequantize (lib.rs:4939-4990,
 * kernels.wgsl:385-400): out[i] = f32(u8[i]) * scales[i/64] + biases[i/64] for
 * every i < n (the reference's dispatch drops i >= 4 194 240; this does not). */
RUSTY_CUDA_API int rusty_cuda_affine_dequantize_g64(rusty_cuda_ctx* ctx, const rusty_cuda_buf* weight,
                                                    const rusty_cuda_buf* scales, const rusty_cuda_buf* biases,
                                                    rusty_cuda_buf* out, size_t n);

/* ComputeEngine::add -> WGSL add (lib.rs:4039-4083, kernels.wgsl:139-144): out[i] = a[i] + b[i],
 * f32, i < n.  On the path only as the sum that closes Linear's LoRA branch
 * (rusty-graph/src/lib.rs:78). */
RUSTY_CUDA_API int rusty_cuda_add_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* a, const rusty_cuda_buf* b,
                                      rusty_cuda_buf* out, size_t n);

/* ---- fused quantised linear ------------------------------------------------
 * Replaces the composition "upload_quantized -> affine_dequantize once -> f32
 * matmul per forward" (rusty-loader/src/lib.rs:155-218 followed by
 * rusty-graph/src/lib.rs:69-70 -> rusty-autograd/src/lib.rs:468-477) with
 * kernels that read the 1-byte weights and their scales once per forward.
 * The object borrows (retains) the buffers it is given, with one exception: a
 * SYM_ROW weight in LAYOUT_KN (rusty's own [in,out] Linear storage) with
 * K % 16 == 0 is re-laid-out ONCE, inside this call, into an [out,in] buffer
 * that the object owns (N*K more bytes of device memory), so that every
 * forward runs on the TMA / tensor-core kernels; the caller's weight buffer
 * is then not kept and may be released.  An AFFINE_G64 weight in LAYOUT_KN
 * (the reference's own quantised format: one scale and bias per 64
 * consecutive OUTPUT features of an input row) with K % 128 == 0 is re-laid-out
 * the same way, bytes to [out,in] and scales / biases to [N/64][K] (N*K*9/8
 * more bytes; none of the caller's three buffers is kept): its forwards run on
 * the int8 tensor-core GEMV with the group's scales folded into the
 * activations (f32 activations: 1e-5 of the reference's arithmetic) and, with
 * bf16 activations and M >= 65, on the bf16 tensor-core kernel (1e-2).  (RUSTY_KN_RELAYOUT=0 in the environment keeps the [in,out]
 * CUDA-core kernel for both.)
 *   AFFINE_G64: weight u8 [N*K], scales/biases f32 [N*K/64]; K % 64 == 0 for
 *               LAYOUT_NK (N % 64 == 0 for LAYOUT_KN) so a group never
 *               straddles two rows.
 *   SYM_ROW   : weight i8 [N*K], scales f32 [N], biases NULL. */
RUSTY_CUDA_API int rusty_cuda_qlinear_create(rusty_cuda_ctx* ctx, rusty_cuda_buf* weight, rusty_cuda_buf* scales,
                                             rusty_cuda_buf* biases, uint32_t N, uint32_t K, int layout, int qmode,
                                             rusty_cuda_qlinear** out);
RUSTY_CUDA_API int rusty_cuda_qlinear_destroy(rusty_cuda_qlinear* ql);
/* Linear::forward for a quantised weight (rusty-graph/src/lib.rs:69-70):
 * y[M,N] = x[M,K] * W^T-or-W with fp32 accumulation.  x_dtype / y_dtype are
 * RUSTY_CUDA_F32 or RUSTY_CUDA_BF16. */
RUSTY_CUDA_API int rusty_cuda_qlinear_forward(rusty_cuda_ctx* ctx, const rusty_cuda_qlinear* ql,
                                              const rusty_cuda_buf* x, int x_dtype, uint32_t M,
                                              rusty_cuda_buf* y, int y_dtype);
/* Name of the kernel `rusty_cuda_qlinear_forward` would launch for this shape
 * ("gemv_f32", "tcgen05", ...); for tests and logs. */
RUSTY_CUDA_API int rusty_cuda_qlinear_plan(const rusty_cuda_qlinear* ql, int x_dtype, uint32_t M, int y_dtype,
                                           char* dst, size_t dst_len);

/* The loop of Linear::forward calls a model forward makes
 * (rusty-graph/src/lib.rs:199-201, :270, :318-322, :435) in one host call:
 * forward i uses qls[i], xs[i], ys[i]; all share M and the dtypes.  Same
 * kernels, same order, as n separate rusty_cuda_qlinear_forward calls. */
RUSTY_CUDA_API int rusty_cuda_qlinear_forward_batch(rusty_cuda_ctx* ctx, size_t n,
                                                    const rusty_cuda_qlinear* const* qls,
                                                    const rusty_cuda_buf* const* xs, int x_dtype, uint32_t M,
                                                    rusty_cuda_buf* const* ys, int y_dtype);

/* Fused int8 linear for callers that must not allocate device memory (no counterpart in the reference,
 * whose ops lean on wgpu's allocator).  Meant for hosts where cudaMalloc is off limits once serving has begun:
 * a real-time loop whose device memory was carved up front, or a process whose own allocator owns the whole
 * device.  Raw device pointers in, nothing allocated or freed, no context needed:
 *     y[M,N] (f32) = x[M,K] (f32) . (w[N,K] (int8, row-major) * scales[N])^T      on `stream` (a cudaStream_t).
 * The kernel's scratch is a fixed ~2.8 MiB array that lives inside the library on every GPU that loads it,
 * which caps the shapes: M <= 8 rows, K <= 8192 (K % 16 == 0, w 16-byte aligned) and N <= 262144;
 * larger calls are rejected with RUSTY_CUDA_ERR_INVALID_DIMENSIONS before anything is
 * launched.  The current device must be the one the pointers belong to.  The first call on each device looks the
 * array's address up; make that call before any stream capture.
 * All calls share the one array: it is cleared where the kernel needs zeros, it otherwise keeps the previous
 * call's contents, and two calls that overlap on the GPU (different streams) race on it.
 * The call only enqueues.  A bounded device-side wait that gives up (it cannot, unless two calls raced) leaves y
 * incomplete and raises a flag in the array, which rusty_cuda_qlinear_i8_static_status reports. */
RUSTY_CUDA_API int rusty_cuda_qlinear_i8_forward_static(const void* w_i8, const float* scales, const float* x_f32,
                                                        float* y_f32, uint32_t M, uint32_t N, uint32_t K,
                                                        void* stream);
/* Drains `stream` and returns RUSTY_CUDA_ERR_TIMEOUT when the most recent static forward on the current device gave
 * up on a wait, RUSTY_CUDA_OK otherwise (the next static forward clears the flag).  Allocates nothing.  No
 * counterpart in the reference.  The _decode form maps a raw status word to the same codes on the host alone. */
RUSTY_CUDA_API int rusty_cuda_qlinear_i8_static_status(void* stream);
RUSTY_CUDA_API int rusty_cuda_qlinear_i8_static_status_decode(unsigned int timeout_flag, unsigned int timeout_where);

/* ---- output-feature sharding across the GPUs of one node -------------------
 * No counterpart in the reference (single device, no collective anywhere); this
 * is Linear::forward (rusty-graph/src/lib.rs:69-70) for a weight whose rows
 * [r*N/G, (r+1)*N/G) live on rank r.  x is replicated; every rank receives the
 * whole y[M,N].  One process per GPU; the 128-byte id comes from rank 0
 * (rusty_cuda_comm_unique_id) and reaches the others by the launcher's own means. */
RUSTY_CUDA_API int rusty_cuda_comm_unique_id(void* out128);
RUSTY_CUDA_API int rusty_cuda_comm_create(rusty_cuda_ctx* ctx, int nranks, int rank, const void* id128,
                                          rusty_cuda_comm** out);
RUSTY_CUDA_API int rusty_cuda_comm_destroy(rusty_cuda_comm* comm);
/* Host-side watchdog hook: reports an asynchronous NCCL error without blocking. */
RUSTY_CUDA_API int rusty_cuda_comm_check(rusty_cuda_comm* comm);
/* y_full[M, G*Nl] = all-gather over ranks of x[M,K] . shard^T.  `gather_ws` is a
 * caller-owned buffer of G*M*Nl elements of y_dtype used for the exchange. */
RUSTY_CUDA_API int rusty_cuda_qlinear_forward_sharded(rusty_cuda_ctx* ctx, rusty_cuda_comm* comm,
                                                      const rusty_cuda_qlinear* ql_shard, const rusty_cuda_buf* x,
                                                      int x_dtype, uint32_t M, rusty_cuda_buf* gather_ws,
                                                      rusty_cuda_buf* y_full, int y_dtype);
RUSTY_CUDA_API int rusty_cuda_qlinear_forward_sharded_batch(rusty_cuda_ctx* ctx, rusty_cuda_comm* comm, size_t n,
                                                            const rusty_cuda_qlinear* const* ql_shards,
                                                            const rusty_cuda_buf* const* xs, int x_dtype, uint32_t M,
                                                            rusty_cuda_buf* gather_ws, rusty_cuda_buf* const* ys,
                                                            int y_dtype);

/* ---- SwiGLU glue of the MLP (rusty-graph/src/lib.rs:317-323) ------------------
 * MLP::forward is gate = Linear, silu(gate), up = Linear, mul, down = Linear.  The two unfused shaders: */
/* WGSL `silu` (kernels.wgsl:104-113): out[i] = x[i] * (1 / (1 + exp(-x[i]))), f32. */
RUSTY_CUDA_API int rusty_cuda_silu_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* x, rusty_cuda_buf* out, size_t n);
/* WGSL `mul` (kernels.wgsl:146-151): out[i] = a[i] * b[i], f32. */
RUSTY_CUDA_API int rusty_cuda_mul_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* a, const rusty_cuda_buf* b,
                                      rusty_cuda_buf* out, size_t n);
/* And the fused form (no counterpart in the reference): a gate|up weight stored pair-interleaved, row 2j = gate_j,
 * row 2j+1 = up_j (RUSTY_CUDA_LAYOUT_NK, RUSTY_CUDA_QMODE_SYM_ROW, N even).  After
 * rusty_cuda_qlinear_set_activation(ql, RUSTY_CUDA_ACT_SWIGLU_PAIRS) every forward of `ql` (plain, batch, sharded,
 * pushed) writes y[M, N/2] with y[m,j] = silu(x.gate_j) * (x.up_j): the activation runs in the kernel's epilogue and
 * the [M, N] intermediate never exists.  Row shards must hold whole pairs.  Kernels without the fused epilogue
 * answer RUSTY_CUDA_ERR_UNSUPPORTED. */
#define RUSTY_CUDA_ACT_NONE 0
#define RUSTY_CUDA_ACT_SWIGLU_PAIRS 1
RUSTY_CUDA_API int rusty_cuda_qlinear_set_activation(rusty_cuda_qlinear* ql, int act);

/* ---- exchange by peer stores over NVLink (no counterpart in the reference) ----
 * The second multi-GPU form of Linear::forward (rusty-graph/src/lib.rs:69-70):
 * instead of an all-gather after the kernel, each rank's kernel stores its
 * output columns straight into every rank's copy of y.  An arena is one device
 * allocation with the same layout on every rank (one process per GPU, one node);
 * ranks swap the 64-byte handles over any host channel and attach.
 *
 * Protocol: every rank enqueues the same sequence of pushed operations on an
 * arena (pushed forwards, rusty_cuda_arena_wait, the sharded arg-max / top-k);
 * the ranks meet at the START of each one: its first kernel tells the other
 * ranks that everything this rank enqueued before has completed and waits for
 * the same word from them.  y_full of a pushed forward is therefore complete on
 * this rank once the next pushed operation on the arena has run; it may be
 * read until the following pushed forward is enqueued and may be the output of
 * a pushed forward again from the second-next on.  Waits for other ranks are
 * bounded (environment RUSTY_PEER_WAIT_MS, default 5000): when one runs out,
 * the next rusty_cuda_sync returns RUSTY_CUDA_ERR_TIMEOUT and the context stays
 * usable; the arena's ranks are then out of step, so destroy it on every rank
 * and build a new one before pushing again.  Keep an arena alive until every
 * rank has stopped pushing to it. */
#define RUSTY_CUDA_IPC_HANDLE_BYTES 64
typedef struct rusty_cuda_arena rusty_cuda_arena;
RUSTY_CUDA_API int rusty_cuda_arena_create(rusty_cuda_ctx* ctx, size_t bytes, int nranks, int rank, rusty_cuda_arena** out);
/* Writes this arena's IPC handle (RUSTY_CUDA_IPC_HANDLE_BYTES bytes). */
RUSTY_CUDA_API int rusty_cuda_arena_export(const rusty_cuda_arena* arena, void* handle64);
/* `handles`: nranks handles back to back, in rank order (the own slot is ignored). */
RUSTY_CUDA_API int rusty_cuda_arena_attach(rusty_cuda_arena* arena, const void* handles);
/* A buffer object over [offset, offset+bytes) of the arena's data region (offset % 256 == 0);
 * use the same offsets on every rank.  Released with rusty_cuda_buf_release. */
RUSTY_CUDA_API int rusty_cuda_arena_buf(rusty_cuda_arena* arena, size_t offset, size_t bytes, rusty_cuda_buf** out);
/* Enqueues a wait until the pushes of all ranks enqueued so far have landed in this rank's arena. */
RUSTY_CUDA_API int rusty_cuda_arena_wait(rusty_cuda_ctx* ctx, rusty_cuda_arena* arena);
RUSTY_CUDA_API int rusty_cuda_arena_destroy(rusty_cuda_arena* arena);
/* y_full[M, G*Nl] (a buffer of the arena): columns [rank*Nl, (rank+1)*Nl) = x[M,K] . shard^T, written here
 * and into every other rank's arena at the same offset. */
RUSTY_CUDA_API int rusty_cuda_qlinear_forward_pushed(rusty_cuda_ctx* ctx, rusty_cuda_arena* arena,
                                                     const rusty_cuda_qlinear* ql_shard, const rusty_cuda_buf* x, int x_dtype,
                                                     uint32_t M, rusty_cuda_buf* y_full, int y_dtype);
RUSTY_CUDA_API int rusty_cuda_qlinear_forward_pushed_batch(rusty_cuda_ctx* ctx, rusty_cuda_arena* arena, size_t n,
                                                           const rusty_cuda_qlinear* const* ql_shards,
                                                           const rusty_cuda_buf* const* xs, int x_dtype, uint32_t M,
                                                           rusty_cuda_buf* const* ys, int y_dtype);

/* ---- the steps in front of a layer's Linears: Embedding gather and RMSNorm --------
 * Embedding::forward (rusty-graph/src/lib.rs:121-135): out[t, :] = table[ids[t], :], table f32 [vocab, dim], ids
 * u32[n_ids] in a DEVICE buffer (the reference copies the whole table to the host on every call and slices it there),
 * dim % 4 == 0.  An id >= vocab panics in the reference; here its row is written as zeros and the next
 * rusty_cuda_sync returns RUSTY_CUDA_ERR_INVALID_OPERATION naming the id. */
RUSTY_CUDA_API int rusty_cuda_embedding_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* table, const rusty_cuda_buf* ids,
                                            rusty_cuda_buf* out, size_t n_ids, uint32_t vocab, uint32_t dim);
/* WGSL `rms_norm` (kernels.wgsl:81-102) and `rms_norm_residual` (:570-597), as RMSNorm::forward calls them
 * (rusty-graph/src/lib.rs:148-170), for EVERY row of x[M, K] (the shader stops after row 0; its residual form treats the
 * whole tensor as one row):  v = x (+ residual);  out = v * (1 / sqrt(mean(v^2) + eps)) * weight,  f32, K % 4 == 0; the
 * reference uses eps = 1e-5.  residual may be NULL.  sum_out (may be NULL; needs residual) receives v, the new residual
 * stream.  The sum of squares is a tree sum in f32 (the shader adds sequentially): a few ulp apart, not bit-identical. */
RUSTY_CUDA_API int rusty_cuda_rms_norm_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* x, const rusty_cuda_buf* residual,
                                           const rusty_cuda_buf* weight, rusty_cuda_buf* out, rusty_cuda_buf* sum_out,
                                           uint32_t M, uint32_t K, float eps);
/* y = Linear(RMSNorm(x (+ residual)) * norm_weight) in one call: norm1 -> q|k|v and norm2 -> gate|up of
 * TransformerBlock::forward (rusty-graph/src/lib.rs:365-377).  Where the Linear's kernel prepares its activations in
 * a pass of its own (3 <= M, K <= 8192, or <= 16384 up to 32 rows) that pass applies the norm to the row it already
 * holds in registers, so the norm costs no launch and no trip through memory; other shapes run the norm kernel above
 * first.  x, residual, normed_out, sum_out: f32 [M, K] (K = the Linear's in_features).  normed_out (may be NULL)
 * receives the normalised activations; sum_out as above.  While a stream capture is open pass normed_out for shapes
 * that are not fused (no scratch can be allocated then). */
RUSTY_CUDA_API int rusty_cuda_qlinear_forward_normed(rusty_cuda_ctx* ctx, const rusty_cuda_qlinear* ql, const rusty_cuda_buf* x,
                                                     const rusty_cuda_buf* residual, const rusty_cuda_buf* norm_weight, float eps,
                                                     uint32_t M, rusty_cuda_buf* normed_out, rusty_cuda_buf* sum_out,
                                                     rusty_cuda_buf* y, int y_dtype);

/* y = residual + Linear(x): `x = x + attn_out` and `x = x + mlp_out` of TransformerBlock::forward
 * (rusty-graph/src/lib.rs:365-377, ComputeEngine::add after o_proj / down_proj) applied where the Linear's outputs are
 * rounded (the tensor-core kernels, M >= 3: for f32 outputs fl(residual + fl(out)), bit-identical to Linear followed by
 * `add`; bf16 outputs are rounded once, after the add); other
 * shapes run the Linear and one add kernel.  residual: [M, N] of y's type; it may be y itself (the residual stream
 * updated in place).  Not for a weight that carries the pair activation. */
RUSTY_CUDA_API int rusty_cuda_qlinear_forward_residual(rusty_cuda_ctx* ctx, const rusty_cuda_qlinear* ql, const rusty_cuda_buf* x,
                                                       int x_dtype, uint32_t M, const rusty_cuda_buf* residual,
                                                       rusty_cuda_buf* y, int y_dtype);

/* ---- the step after the LM head: greedy token choice on the device -------------
 * Sampler::sample with temperature <= 0 (rusty-loader/src/tokenizer.rs:151-158): per activation row the index of
 * the largest logit, the LAST one among equals, 0 for a row without candidates; NaN never wins (the reference panics
 * on it).  out_idx: u32[M]; out_val (may be NULL): f32[M], the maxima.  The WGSL `top_k` kernel
 * (kernels.wgsl:168-188) with k = 1 differs only in taking the FIRST of equal maxima. */
RUSTY_CUDA_API int rusty_cuda_argmax_rows_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* logits, uint32_t M, uint32_t N,
                                              rusty_cuda_buf* out_idx, rusty_cuda_buf* out_val);
/* With output-feature shards (no counterpart in the reference): logits_shard is this rank's [M, Nl] block of
 * columns [rank*Nl, (rank+1)*Nl); each rank stores its per-row candidate into `table` — a buffer of the arena at the
 * same offset on every rank, nranks * M * 8 bytes — of every rank, and every rank ends with the global indices.
 * Counts as two pushed operations of the arena's protocol. */
RUSTY_CUDA_API int rusty_cuda_argmax_rows_sharded(rusty_cuda_ctx* ctx, rusty_cuda_arena* arena,
                                                  const rusty_cuda_buf* logits_shard, uint32_t M, uint32_t Nl,
                                                  rusty_cuda_buf* table, rusty_cuda_buf* out_idx, rusty_cuda_buf* out_val);
/* The k largest logits of every row: WGSL `top_k` (kernels.wgsl:168-188) for each row of logits[M, N] — descending
 * values, equal values in ascending index order, values that are not > -1e9 (NaN included) never taken, and slots for
 * which nothing is left report index 0 (value -inf) as the shader's exhausted rounds do.  1 <= k <= 1024.
 * out_idx: u32 [M, k]; out_val (may be NULL): f32 [M, k]. */
RUSTY_CUDA_API int rusty_cuda_top_k_rows_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* logits, uint32_t M, uint32_t N, uint32_t k,
                                             rusty_cuda_buf* out_idx, rusty_cuda_buf* out_val);
/* Soft-max statistics of every row at a temperature (> 0): out_max[m] = the largest logit, out_sum[m] = sum_j
 * exp((x[m,j] - max) / temperature): what Sampler::sample computes before sorting (rusty-loader/src/tokenizer.rs:161-170),
 * NaN skipped, f32 tree sum.  With the row's top-k pairs the host walks the nucleus without reading the logits back
 * (probability of a candidate = exp((value - max) / temperature) / sum). */
RUSTY_CUDA_API int rusty_cuda_softmax_stats_rows_f32(rusty_cuda_ctx* ctx, const rusty_cuda_buf* logits, uint32_t M, uint32_t N,
                                                     float temperature, rusty_cuda_buf* out_max, rusty_cuda_buf* out_sum);
/* The same over output-feature shards: every rank passes its own columns [M, Nl] (global index = rank * Nl + column);
 * only k (value, index) pairs per row and rank cross NVLink, every rank ends with the k global winners.
 * table: a buffer of the arena, nranks * M * k * 8 bytes, at the same offset on every rank.  k * nranks <= 2048. */
RUSTY_CUDA_API int rusty_cuda_top_k_rows_sharded(rusty_cuda_ctx* ctx, rusty_cuda_arena* arena, const rusty_cuda_buf* logits_shard,
                                                 uint32_t M, uint32_t Nl, uint32_t k, rusty_cuda_buf* table,
                                                 rusty_cuda_buf* out_idx, rusty_cuda_buf* out_val);

/* ---- stream capture and timing ---------------------------------------------
 * rusty submits one command buffer per op (lib.rs:4452); a decode step here is
 * hundreds of short kernels, so the sequence can be recorded once into a CUDA
 * graph and replayed with one launch.  Between begin and end, operator calls
 * on this context are captured instead of executed; uploads, downloads and
 * sync are not allowed. */
RUSTY_CUDA_API int rusty_cuda_graph_begin(rusty_cuda_ctx* ctx);
RUSTY_CUDA_API int rusty_cuda_graph_end(rusty_cuda_ctx* ctx, rusty_cuda_graph** out);
RUSTY_CUDA_API int rusty_cuda_graph_launch(rusty_cuda_ctx* ctx, rusty_cuda_graph* graph);
RUSTY_CUDA_API int rusty_cuda_graph_destroy(rusty_cuda_graph* graph);
/* Device timestamps on the context's stream (the reference's benchmarks use
 * host wall-clock around submit + poll, benchmarks/src/main.rs:99-106). */
typedef struct rusty_cuda_event rusty_cuda_event;
RUSTY_CUDA_API int rusty_cuda_event_create(rusty_cuda_ctx* ctx, rusty_cuda_event** out);
RUSTY_CUDA_API int rusty_cuda_event_record(rusty_cuda_ctx* ctx, rusty_cuda_event* ev);
/* Waits for `stop`, then returns the device time from `start` to `stop`. */
RUSTY_CUDA_API int rusty_cuda_event_elapsed_ms(rusty_cuda_ctx* ctx, rusty_cuda_event* start, rusty_cuda_event* stop,
                                               float* ms);
RUSTY_CUDA_API int rusty_cuda_event_destroy(rusty_cuda_event* ev);

/* ---- harness helper (no counterpart in the reference) ------------------------------
 */
/* Overwrite `bytes` bytes at `offset` with `value` (cudaMemsetAsync); used by
 * harnesses to flush L2 between timed iterations and to clear outputs. */
RUSTY_CUDA_API int rusty_cuda_buf_fill_u8(rusty_cuda_ctx* ctx, rusty_cuda_buf* buf, size_t offset, int value,
                                          size_t bytes);

#ifdef __cplusplus
}
#endif
#endif /* RUSTY_CUDA_H */
