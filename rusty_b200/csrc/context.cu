// Context, buffer pool and buffer transfer entry points of librusty_cuda.
//
// Stands in for rusty-backend's WgpuContext (lib.rs:11-53), BufferPool
// (pool.rs:5-56) and the storage half of UnifiedTensor (lib.rs:78-241):
// one device, one in-order stream, exact-size bins for pooled buffers,
// reference-counted storage.
#include <cstring>

#include "internal.h"

namespace {
std::mutex g_err_mu;
std::string g_last_error = "";  // failures that have no context to hang on
thread_local std::string t_scratch;
}  // namespace

namespace rusty {

int fail(rusty_cuda_ctx* ctx, int code, const char* fmt, ...) {
    char msg[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof msg, fmt, ap);
    va_end(ap);
    if (ctx) {
        ctx->last_error = msg;
    } else {
        std::lock_guard<std::mutex> g(g_err_mu);
        g_last_error = msg;
    }
    return code;
}

int check_cuda(rusty_cuda_ctx* ctx, cudaError_t e, const char* what) {
    if (e == cudaSuccess) return RUSTY_CUDA_OK;
    int code = RUSTY_CUDA_ERR_OTHER;
    switch (e) {
        case cudaErrorMemoryAllocation: code = RUSTY_CUDA_ERR_MEMORY_ALLOCATION; break;
        case cudaErrorNoDevice:
        case cudaErrorInsufficientDriver:
        case cudaErrorInvalidDevice:
        case cudaErrorInitializationError: code = RUSTY_CUDA_ERR_GPU_INITIALIZATION; break;
        case cudaErrorInvalidValue: code = RUSTY_CUDA_ERR_INVALID_OPERATION; break;
        default: code = RUSTY_CUDA_ERR_KERNEL_EXECUTION; break;
    }
    return fail(ctx, code, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

int after_launch(rusty_cuda_ctx* ctx, const char* kernel) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, kernel);
    count_launch(ctx);
    return RUSTY_CUDA_OK;
}

}  // namespace rusty

using namespace rusty;

namespace rusty {
cudaError_t ensure_dynamic_smem(const void* kernel, int device, size_t bytes) {
    static std::mutex mu;
    static std::unordered_map<uint64_t, size_t> high;  // (kernel address mixed with the device ordinal) -> bytes opted in
    const uint64_t key = (uint64_t)reinterpret_cast<uintptr_t>(kernel) * 1315423911ull + (uint64_t)(uint32_t)device;
    std::lock_guard<std::mutex> lk(mu);
    auto it = high.find(key);
    if (it != high.end() && it->second >= bytes) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) high[key] = bytes;
    return e;
}
}  // namespace rusty

extern "C" {

int rusty_cuda_device_count(int* count) {
    if (!count) return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "device_count: null out pointer");
    *count = 0;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return check_cuda(nullptr, e, "cudaGetDeviceCount");
    }
    *count = n;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_ctx_create(int device, rusty_cuda_ctx** out) {
    if (!out) return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "ctx_create: null out pointer");
    *out = nullptr;
    int n = 0;
    int rc = rusty_cuda_device_count(&n);
    if (rc != RUSTY_CUDA_OK) return RUSTY_CUDA_ERR_GPU_INITIALIZATION;
    if (n == 0) return fail(nullptr, RUSTY_CUDA_ERR_GPU_INITIALIZATION, "ctx_create: no CUDA device (there is no CPU fallback)");
    if (device < 0 || device >= n)
        return fail(nullptr, RUSTY_CUDA_ERR_GPU_INITIALIZATION, "ctx_create: device %d out of range (0..%d)", device, n - 1);
    DeviceGuard g(device);
    if (!g.ok) return fail(nullptr, RUSTY_CUDA_ERR_GPU_INITIALIZATION, "ctx_create: cudaSetDevice(%d) failed", device);
    cudaDeviceProp p;
    rc = check_cuda(nullptr, cudaGetDeviceProperties(&p, device), "cudaGetDeviceProperties");
    if (rc) return rc;
    if (p.major != 10)
        return fail(nullptr, RUSTY_CUDA_ERR_UNSUPPORTED,
                    "ctx_create: device %d is sm_%d%d; this library holds sm_100a code only", device, p.major, p.minor);
    rusty_cuda_ctx* c = new (std::nothrow) rusty_cuda_ctx();
    if (!c) return fail(nullptr, RUSTY_CUDA_ERR_MEMORY_ALLOCATION, "ctx_create: host allocation failed");
    c->device = device;
    c->sm_count = p.multiProcessorCount;
    c->cc_major = p.major;
    c->cc_minor = p.minor;
    c->smem_optin = p.sharedMemPerBlockOptin;
    c->name = p.name;
    rc = check_cuda(nullptr, cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking), "cudaStreamCreate");
    if (rc) {
        delete c;
        return rc;
    }
    rc = check_cuda(nullptr, cudaHostAlloc((void**)&c->status_host, sizeof(rusty_cuda_dev_status), cudaHostAllocMapped),
                    "cudaHostAlloc(status)");
    if (!rc) {
        memset(c->status_host, 0, sizeof(rusty_cuda_dev_status));
        rc = check_cuda(nullptr, cudaHostGetDevicePointer((void**)&c->status_dev, c->status_host, 0),
                        "cudaHostGetDevicePointer(status)");
    }
    if (rc) {
        if (c->status_host) cudaFreeHost(c->status_host);
        cudaStreamDestroy(c->stream);
        delete c;
        return rc;
    }
    *out = c;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_ctx_destroy(rusty_cuda_ctx* ctx) {
    if (!ctx) return RUSTY_CUDA_OK;
    DeviceGuard g(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (void* p : ctx->deferred_free) cudaFree(p);   // releases parked by a capture that was never ended
    ctx->deferred_free.clear();
    rusty_cuda_pool_clear(ctx);
    tc_workspace_release(ctx);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_ctx_adapter_info(rusty_cuda_ctx* ctx, char* dst, size_t dst_len) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!dst || dst_len == 0) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "adapter_info: empty destination");
    snprintf(dst, dst_len, "%s (CUDA sm_%d%d, %d SMs)", ctx->name.c_str(), ctx->cc_major, ctx->cc_minor, ctx->sm_count);
    return RUSTY_CUDA_OK;
}

const char* rusty_cuda_last_error(rusty_cuda_ctx* ctx) {
    if (ctx) return ctx->last_error.c_str();
    std::lock_guard<std::mutex> g(g_err_mu);
    t_scratch = g_last_error;
    return t_scratch.c_str();
}

#define RUSTY_NOT_CAPTURING(ctx, what)                                                                        \
    do {                                                                                                      \
        if ((ctx)->capturing)                                                                                 \
            return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, what ": not allowed while a graph capture is open"); \
    } while (0)

int rusty_cuda_ctx_self_check(rusty_cuda_ctx* ctx) {
    RUSTY_REQUIRE_CTX(ctx);
    RUSTY_NOT_CAPTURING(ctx, "self_check");
    DeviceGuard g(ctx->device);
    cudaError_t e = cudaSuccess;
    const int bad = tc_workspace_check_guards(ctx, &e);
    if (e != cudaSuccess) return check_cuda(ctx, e, "self_check: reading the guard zones");
    if (bad >= 0)
        return fail(ctx, RUSTY_CUDA_ERR_KERNEL_EXECUTION, "self_check: guard zone %d of the kernel workspace was overwritten", bad);
    return RUSTY_CUDA_OK;
}

int rusty_cuda_sync(rusty_cuda_ctx* ctx) {
    RUSTY_REQUIRE_CTX(ctx);
    RUSTY_NOT_CAPTURING(ctx, "sync");
    DeviceGuard g(ctx->device);
    int rc = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
    if (rc) return rc;
    if (ctx->status_host->timeout_flag) {
        unsigned where = ctx->status_host->timeout_where;
        ctx->status_host->timeout_flag = 0;
        ctx->status_host->timeout_where = 0;
        tc_workspace_clear_pieces(ctx);   // a kernel that gave up may have left pieces of K-cut tiles behind
        return fail(ctx, RUSTY_CUDA_ERR_TIMEOUT, "a bounded device-side wait gave up (site %u)", where);
    }
    if (ctx->status_host->bad_index_flag) {
        unsigned id = ctx->status_host->bad_index_value;
        ctx->status_host->bad_index_flag = 0;
        ctx->status_host->bad_index_value = 0;
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "embedding: token id %u lies outside the table (its row was written as zeros)", id);
    }
    return RUSTY_CUDA_OK;
}

int rusty_cuda_ctx_launch_count(rusty_cuda_ctx* ctx, uint64_t* count) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!count) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "launch_count: null out pointer");
    *count = ctx->launches.load();
    return RUSTY_CUDA_OK;
}

int rusty_cuda_ctx_stream(rusty_cuda_ctx* ctx, void** stream) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!stream) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "ctx_stream: null out pointer");
    *stream = (void*)ctx->stream;
    return RUSTY_CUDA_OK;
}

// ---- buffers ---------------------------------------------------------------

int rusty_cuda_buf_alloc(rusty_cuda_ctx* ctx, size_t bytes, int pooled, rusty_cuda_buf** out) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!out) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "buf_alloc: null out pointer");
    *out = nullptr;
    DeviceGuard g(ctx->device);
    void* p = nullptr;
    if (pooled) {
        std::lock_guard<std::mutex> lk(ctx->pool_mu);
        auto it = ctx->pool_bins.find(bytes);
        if (it != ctx->pool_bins.end() && !it->second.empty()) {
            p = it->second.back();
            it->second.pop_back();
        }
    }
    if (!p && ctx->capturing)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "buf_alloc: no idle pool buffer of %zu bytes, and device memory cannot be allocated while a capture is open", bytes);
    if (!p) {
        // A zero-byte tensor still gets a distinct, valid allocation.
        cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
        if (e != cudaSuccess) {
            cudaGetLastError();
            size_t fr = 0, tot = 0;
            cudaMemGetInfo(&fr, &tot);
            return fail(ctx, RUSTY_CUDA_ERR_MEMORY_ALLOCATION, "buf_alloc: out of memory (requested %zu bytes, %zu available)",
                        bytes, fr);
        }
    }
    rusty_cuda_buf* b = new (std::nothrow) rusty_cuda_buf();
    if (!b) {
        cudaFree(p);
        return fail(ctx, RUSTY_CUDA_ERR_MEMORY_ALLOCATION, "buf_alloc: host allocation failed");
    }
    b->ctx = ctx;
    b->ptr = p;
    b->bytes = bytes;
    b->pooled = pooled != 0;
    *out = b;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_buf_retain(rusty_cuda_buf* buf) {
    if (!buf) return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "buf_retain: null buffer");
    buf->refs.fetch_add(1);
    return RUSTY_CUDA_OK;
}

int rusty_cuda_buf_release(rusty_cuda_buf* buf) {
    if (!buf) return RUSTY_CUDA_OK;
    if (buf->refs.fetch_sub(1) != 1) return RUSTY_CUDA_OK;
    rusty_cuda_ctx* ctx = buf->ctx;
    if (buf->borrowed) {
        delete buf;
        return RUSTY_CUDA_OK;
    }
    if (buf->pooled) {
        // TensorData::drop (lib.rs:92-98): back to the bin of its exact size.
        // Work already enqueued on the single in-order stream finishes before
        // any later user of the buffer runs, so no synchronisation is needed.
        std::lock_guard<std::mutex> lk(ctx->pool_mu);
        ctx->pool_bins[buf->bytes].push_back(buf->ptr);
    } else if (ctx->capturing) {
        std::lock_guard<std::mutex> lk(ctx->pool_mu);
        ctx->deferred_free.push_back(buf->ptr);   // freed when the capture ends
    } else {
        DeviceGuard g(ctx->device);
        cudaStreamSynchronize(ctx->stream);
        cudaFree(buf->ptr);
    }
    delete buf;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_buf_size(const rusty_cuda_buf* buf, size_t* bytes) {
    if (!buf || !bytes) return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "buf_size: null argument");
    *bytes = buf->bytes;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_buf_device_ptr(const rusty_cuda_buf* buf, void** ptr) {
    if (!buf || !ptr) return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "buf_device_ptr: null argument");
    *ptr = buf->ptr;
    return RUSTY_CUDA_OK;
}

static int range_check(rusty_cuda_ctx* ctx, const char* what, const rusty_cuda_buf* b, size_t off, size_t bytes) {
    if (!b) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "%s: null buffer", what);
    if (off > b->bytes || bytes > b->bytes - off)
        return fail(ctx, RUSTY_CUDA_ERR_BUFFER_OPERATION, "%s: range [%zu, %zu) exceeds the buffer's %zu bytes", what, off,
                    off + bytes, b->bytes);
    return RUSTY_CUDA_OK;
}

int rusty_cuda_buf_upload_async(rusty_cuda_ctx* ctx, rusty_cuda_buf* dst, size_t dst_offset, const void* src,
                                size_t bytes) {
    RUSTY_REQUIRE_CTX(ctx);
    RUSTY_NOT_CAPTURING(ctx, "buf_upload");
    int rc = range_check(ctx, "buf_upload", dst, dst_offset, bytes);
    if (rc) return rc;
    if (bytes == 0) return RUSTY_CUDA_OK;
    if (!src) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "buf_upload: null source");
    DeviceGuard g(ctx->device);
    cudaError_t e = cudaMemcpyAsync((char*)dst->ptr + dst_offset, src, bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) return fail(ctx, RUSTY_CUDA_ERR_DATA_TRANSFER, "buf_upload: %s", cudaGetErrorString(e));
    return RUSTY_CUDA_OK;
}

int rusty_cuda_buf_upload(rusty_cuda_ctx* ctx, rusty_cuda_buf* dst, size_t dst_offset, const void* src, size_t bytes) {
    int rc = rusty_cuda_buf_upload_async(ctx, dst, dst_offset, src, bytes);
    if (rc) return rc;
    // queue.write_buffer copies the caller's bytes before returning; pageable
    // host memory may still be read after cudaMemcpyAsync returns, so wait.
    DeviceGuard g(ctx->device);
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return fail(ctx, RUSTY_CUDA_ERR_DATA_TRANSFER, "buf_upload: %s", cudaGetErrorString(e));
    return RUSTY_CUDA_OK;
}

int rusty_cuda_buf_download_async(rusty_cuda_ctx* ctx, const rusty_cuda_buf* src, size_t src_offset, void* dst,
                                  size_t bytes) {
    RUSTY_REQUIRE_CTX(ctx);
    RUSTY_NOT_CAPTURING(ctx, "buf_download");
    int rc = range_check(ctx, "buf_download", src, src_offset, bytes);
    if (rc) return rc;
    if (bytes == 0) return RUSTY_CUDA_OK;
    if (!dst) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "buf_download: null destination");
    DeviceGuard g(ctx->device);
    cudaError_t e = cudaMemcpyAsync(dst, (const char*)src->ptr + src_offset, bytes, cudaMemcpyDeviceToHost, ctx->stream);
    if (e != cudaSuccess) return fail(ctx, RUSTY_CUDA_ERR_DATA_TRANSFER, "buf_download: %s", cudaGetErrorString(e));
    return RUSTY_CUDA_OK;
}

int rusty_cuda_buf_download(rusty_cuda_ctx* ctx, const rusty_cuda_buf* src, size_t src_offset, void* dst, size_t bytes) {
    int rc = rusty_cuda_buf_download_async(ctx, src, src_offset, dst, bytes);
    if (rc) return rc;
    return rusty_cuda_sync(ctx);
}

int rusty_cuda_buf_copy(rusty_cuda_ctx* ctx, const rusty_cuda_buf* src, rusty_cuda_buf* dst, size_t dst_offset) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!src) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "buf_copy: null source");
    int rc = range_check(ctx, "buf_copy", dst, dst_offset, src->bytes);
    if (rc) return rc;
    if (src->bytes == 0) return RUSTY_CUDA_OK;
    DeviceGuard g(ctx->device);
    cudaError_t e =
        cudaMemcpyAsync((char*)dst->ptr + dst_offset, src->ptr, src->bytes, cudaMemcpyDeviceToDevice, ctx->stream);
    if (e != cudaSuccess) return fail(ctx, RUSTY_CUDA_ERR_DATA_TRANSFER, "buf_copy: %s", cudaGetErrorString(e));
    return RUSTY_CUDA_OK;
}

int rusty_cuda_pool_clear(rusty_cuda_ctx* ctx) {
    RUSTY_REQUIRE_CTX(ctx);
    DeviceGuard g(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    std::lock_guard<std::mutex> lk(ctx->pool_mu);
    for (auto& kv : ctx->pool_bins)
        for (void* p : kv.second) cudaFree(p);
    ctx->pool_bins.clear();
    return RUSTY_CUDA_OK;
}

int rusty_cuda_pool_idle_count(rusty_cuda_ctx* ctx, size_t bytes, size_t* count) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!count) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "pool_idle_count: null out pointer");
    std::lock_guard<std::mutex> lk(ctx->pool_mu);
    auto it = ctx->pool_bins.find(bytes);
    *count = it == ctx->pool_bins.end() ? 0 : it->second.size();
    return RUSTY_CUDA_OK;
}

int rusty_cuda_host_alloc(size_t bytes, void** out) {
    if (!out) return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "host_alloc: null out pointer");
    *out = nullptr;
    cudaError_t e = cudaHostAlloc(out, bytes ? bytes : 16, cudaHostAllocDefault);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return check_cuda(nullptr, e, "cudaHostAlloc");
    }
    return RUSTY_CUDA_OK;
}

int rusty_cuda_host_free(void* p) {
    if (!p) return RUSTY_CUDA_OK;
    cudaError_t e = cudaFreeHost(p);
    if (e != cudaSuccess) return check_cuda(nullptr, e, "cudaFreeHost");
    return RUSTY_CUDA_OK;
}

}  // extern "C"
