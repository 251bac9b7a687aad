// Output-feature sharding of a fused linear across the GPUs of one node.
//
// The reference is single-device (no collective anywhere in its tree); this is
// the multi-GPU form of Linear::forward (rusty-graph/src/lib.rs:69-70) for
// weights split by rows of W[out,in]: rank r holds rows [r*N/G, (r+1)*N/G) and
// their scales, x is replicated, and every rank ends with the whole y[M,N].
// Each dot product is computed by exactly one rank with the single-GPU kernel,
// so the sharded result equals the unsharded one bit for bit.
//
// Exchange: NCCL all-gather over NVLink on the context's stream.  NCCL is bound
// at run time with dlopen (the copy PyTorch already loaded, or the system one),
// so the library has no link-time dependency on it.
#include <dlfcn.h>

#include <cstring>

#include "internal.h"

using namespace rusty;

namespace {

// The few NCCL entry points used, by their C signatures (nccl.h).
typedef struct ncclComm* ncclComm_t;
struct Id128 {
    char b[128];  // ncclUniqueId, passed by value
};
struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, Id128, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*CommAbort)(ncclComm_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*CommGetAsyncError)(ncclComm_t, int*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};

NcclApi& nccl() {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        const char* names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (api.handle) {
            *(void**)&api.GetUniqueId = dlsym(api.handle, "ncclGetUniqueId");
            *(void**)&api.CommInitRank = dlsym(api.handle, "ncclCommInitRank");
            *(void**)&api.CommDestroy = dlsym(api.handle, "ncclCommDestroy");
            *(void**)&api.CommAbort = dlsym(api.handle, "ncclCommAbort");
            *(void**)&api.AllGather = dlsym(api.handle, "ncclAllGather");
            *(void**)&api.CommGetAsyncError = dlsym(api.handle, "ncclCommGetAsyncError");
            *(void**)&api.GetErrorString = dlsym(api.handle, "ncclGetErrorString");
            api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.GetErrorString;
        }
    }
    return api;
}

constexpr int NCCL_UINT8 = 1;  // ncclUint8

// gathered [G][M][Nl] (rank-major) -> y [M][G*Nl]; 16-byte vectors when Nl*esize allows.
__global__ void __launch_bounds__(256) interleave_shards_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                               int G, int M, size_t row_bytes /* Nl * esize */) {
    const size_t vec = row_bytes / 16;
    const size_t total = (size_t)G * M * vec;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t v = i % vec;
        const size_t m = (i / vec) % M;
        const size_t g = i / (vec * M);
        const uint4 val = reinterpret_cast<const uint4*>(src + (g * M + m) * row_bytes)[v];
        reinterpret_cast<uint4*>(dst + (m * G + g) * row_bytes)[v] = val;
    }
}

}  // namespace

struct rusty_cuda_comm {
    rusty_cuda_ctx* ctx = nullptr;
    ncclComm_t comm = nullptr;
    int nranks = 1, rank = 0;
};

extern "C" {

int rusty_cuda_comm_unique_id(void* out128) {
    if (!out128) return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "comm_unique_id: null out pointer");
    NcclApi& n = nccl();
    if (!n.ok) return fail(nullptr, RUSTY_CUDA_ERR_UNSUPPORTED, "comm_unique_id: libnccl.so.2 could not be loaded");
    int rc = n.GetUniqueId(out128);
    if (rc != 0) return fail(nullptr, RUSTY_CUDA_ERR_OTHER, "ncclGetUniqueId: %s", n.GetErrorString(rc));
    return RUSTY_CUDA_OK;
}

int rusty_cuda_comm_create(rusty_cuda_ctx* ctx, int nranks, int rank, const void* id128, rusty_cuda_comm** out) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!out || !id128) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "comm_create: null argument");
    *out = nullptr;
    if (nranks < 1 || rank < 0 || rank >= nranks)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "comm_create: rank %d of %d", rank, nranks);
    NcclApi& n = nccl();
    if (!n.ok) return fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "comm_create: libnccl.so.2 could not be loaded");
    DeviceGuard g(ctx->device);
    Id128 id;
    memcpy(id.b, id128, 128);
    ncclComm_t c = nullptr;
    int rc = n.CommInitRank(&c, nranks, id, rank);
    if (rc != 0) return fail(ctx, RUSTY_CUDA_ERR_OTHER, "ncclCommInitRank: %s", n.GetErrorString(rc));
    rusty_cuda_comm* cm = new (std::nothrow) rusty_cuda_comm();
    if (!cm) {
        n.CommDestroy(c);
        return fail(ctx, RUSTY_CUDA_ERR_MEMORY_ALLOCATION, "comm_create: host allocation failed");
    }
    cm->ctx = ctx;
    cm->comm = c;
    cm->nranks = nranks;
    cm->rank = rank;
    *out = cm;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_comm_destroy(rusty_cuda_comm* comm) {
    if (!comm) return RUSTY_CUDA_OK;
    DeviceGuard g(comm->ctx->device);
    cudaStreamSynchronize(comm->ctx->stream);
    nccl().CommDestroy(comm->comm);
    delete comm;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_comm_check(rusty_cuda_comm* comm) {
    if (!comm) return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "comm_check: null communicator");
    NcclApi& n = nccl();
    if (!n.CommGetAsyncError) return RUSTY_CUDA_OK;
    int async_err = 0;
    int rc = n.CommGetAsyncError(comm->comm, &async_err);
    if (rc != 0) return fail(comm->ctx, RUSTY_CUDA_ERR_OTHER, "ncclCommGetAsyncError: %s", n.GetErrorString(rc));
    if (async_err != 0) return fail(comm->ctx, RUSTY_CUDA_ERR_KERNEL_EXECUTION, "NCCL asynchronous error: %s", n.GetErrorString(async_err));
    return RUSTY_CUDA_OK;
}

int rusty_cuda_qlinear_forward_sharded(rusty_cuda_ctx* ctx, rusty_cuda_comm* comm, const rusty_cuda_qlinear* ql_shard,
                                       const rusty_cuda_buf* x, int x_dtype, uint32_t M, rusty_cuda_buf* gather_ws,
                                       rusty_cuda_buf* y_full, int y_dtype) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!comm || !ql_shard || !x || !gather_ws || !y_full)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_sharded: null argument");
    if (comm->ctx != ctx) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_sharded: communicator of another context");
    const size_t ys = y_dtype == RUSTY_CUDA_BF16 ? 2 : y_dtype == RUSTY_CUDA_F32 ? 4 : 0;
    if (!ys) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DATA_TYPE, "qlinear_forward_sharded: y must be f32 or bf16");
    const int G = comm->nranks;
    const uint32_t Nl = ql_shard->act ? ql_shard->N / 2 : ql_shard->N;  // output columns of this rank
    const size_t shard_bytes = (size_t)M * Nl * ys;
    if (gather_ws->bytes < shard_bytes * G || y_full->bytes < shard_bytes * G)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_forward_sharded: gather workspace and y need %zu bytes each",
                    shard_bytes * G);
    if (((size_t)Nl * ys) % 16 != 0)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_forward_sharded: a shard row (%zu bytes) must be a multiple of 16",
                    (size_t)Nl * ys);
    if (M == 0 || Nl == 0) return RUSTY_CUDA_OK;
    // 1. this rank's shard, contiguous, into its slot of the gather workspace
    rusty_cuda_buf slot = {};
    slot.ctx = ctx;
    slot.ptr = (char*)gather_ws->ptr + shard_bytes * comm->rank;
    slot.bytes = shard_bytes;
    int rc = qlinear_forward_cols(ctx, ql_shard, x, x_dtype, M, &slot, y_dtype, Nl, 0);
    if (rc) return rc;
    DeviceGuard g(ctx->device);
    if (G == 1) {
        return check_cuda(ctx, cudaMemcpyAsync(y_full->ptr, slot.ptr, shard_bytes, cudaMemcpyDeviceToDevice, ctx->stream),
                          "qlinear_forward_sharded: copy");
    }
    // 2. all-gather in place: slot r of every rank -> [G][M][Nl] everywhere
    NcclApi& n = nccl();
    int nrc = n.AllGather(slot.ptr, gather_ws->ptr, shard_bytes, NCCL_UINT8, comm->comm, ctx->stream);
    if (nrc != 0) return fail(ctx, RUSTY_CUDA_ERR_OTHER, "ncclAllGather: %s", n.GetErrorString(nrc));
    // 3. rank-major -> row-major y[M, G*Nl]
    const size_t vecs = (size_t)G * M * ((size_t)Nl * ys / 16);
    size_t blocks = (vecs + 255) / 256, cap = (size_t)ctx->sm_count * 8;
    if (blocks > cap) blocks = cap;
    interleave_shards_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>((const uint8_t*)gather_ws->ptr, (uint8_t*)y_full->ptr, G,
                                                                        (int)M, (size_t)Nl * ys);
    return after_launch(ctx, "interleave_shards");
}

int rusty_cuda_qlinear_forward_sharded_batch(rusty_cuda_ctx* ctx, rusty_cuda_comm* comm, size_t n,
                                             const rusty_cuda_qlinear* const* ql_shards, const rusty_cuda_buf* const* xs,
                                             int x_dtype, uint32_t M, rusty_cuda_buf* gather_ws, rusty_cuda_buf* const* ys,
                                             int y_dtype) {
    RUSTY_REQUIRE_CTX(ctx);
    if (n && (!ql_shards || !xs || !ys)) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_sharded_batch: null array");
    for (size_t i = 0; i < n; ++i) {
        int rc = rusty_cuda_qlinear_forward_sharded(ctx, comm, ql_shards[i], xs[i], x_dtype, M, gather_ws, ys[i], y_dtype);
        if (rc) return rc;
    }
    return RUSTY_CUDA_OK;
}

}  // extern "C"
