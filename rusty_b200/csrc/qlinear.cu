// Fused quantised Linear: object, shape checks and kernel selection.
//
// Stands in for the reference's Linear::forward over a quantised weight
// (rusty-graph/src/lib.rs:69-70), which there is "dequantise once at load
// (rusty-loader/src/lib.rs:155-218), then an f32 matmul per call".
#include <cstdlib>
#include <cstring>

#include "internal.h"

using namespace rusty;

namespace rusty {

static size_t dtype_size(int dt) {
    switch (dt) {
        case RUSTY_CUDA_F32: return 4;
        case RUSTY_CUDA_BF16: return 2;
        default: return 0;
    }
}

// whether the group-column affine GEMV can run a weight of this shape at all (checked before the re-layout)
static bool gc_kernel_available(const rusty_cuda_ctx* ctx, uint32_t N, uint32_t K) {
    QLinearArgs a{};
    a.N = N;
    a.K = K;
    a.layout = RUSTY_CUDA_LAYOUT_NK;
    a.qmode = QMODE_AFFINE_GC;
    a.x_dtype = RUSTY_CUDA_F32;
    a.y_dtype = RUSTY_CUDA_F32;
    a.M = 2;
    return gemv_mma_supported(ctx, a);
}

uint32_t f16tc_min_rows() {
    // RUSTY_F16_MIN_ROWS overrides the batch size from which bf16 activations take the fp16/bf16 MMA kernel (tuning aid).
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("RUSTY_F16_MIN_ROWS");
        v = e ? atoi(e) : 65;
        if (v < 1) v = 1;
    }
    return (uint32_t)v;
}

// Which kernel a forward of this shape runs.
const char* qlinear_plan(const rusty_cuda_qlinear* ql, int x_dtype, uint32_t M, int y_dtype) {
    QLinearArgs a{};
    a.N = ql->N;
    a.K = ql->K;
    a.layout = ql->layout;
    a.qmode = ql->qmode;
    a.x_dtype = x_dtype;
    a.y_dtype = y_dtype;
    a.M = M;
    a.act = ql->act;
    if (f16tc_supported(ql->ctx, a) && M >= f16tc_min_rows()) return "tcgen05_f16";
    if (tc_supported(ql->ctx, a) && M >= tc_min_rows() && (!a.act || tc_pushes_fused(M))) return "tcgen05";
    if (gemv_mma_supported(ql->ctx, a)) return "gemv_mma";
    if (gemv_supported(ql->ctx, a)) return "gemv";
    return "unsupported";
}

bool qlinear_pushes_fused(const rusty_cuda_qlinear* ql, int x_dtype, uint32_t M, int y_dtype) {
    const char* plan = qlinear_plan(ql, x_dtype, M, y_dtype);
    return (strcmp(plan, "tcgen05") == 0 && tc_pushes_fused(M)) || strcmp(plan, "tcgen05_f16") == 0 || strcmp(plan, "gemv_mma") == 0;
}

// The int8 decode pair meets the other ranks in its own pre-pass; the bf16 kernel and the M <= 2 GEMV store to the peers
// from their epilogues but need the meeting as a kernel in front of them.
bool qlinear_meets_in_kernel(const rusty_cuda_qlinear* ql, int x_dtype, uint32_t M, int y_dtype) {
    return strcmp(qlinear_plan(ql, x_dtype, M, y_dtype), "tcgen05") == 0 && tc_pushes_fused(M);
}

bool qlinear_residual_fused(const rusty_cuda_qlinear* ql, int x_dtype, uint32_t M, int y_dtype) {
    const char* plan = qlinear_plan(ql, x_dtype, M, y_dtype);
    return !ql->act && (strcmp(plan, "tcgen05") == 0 || strcmp(plan, "tcgen05_f16") == 0);
}

bool qlinear_norm_fused(const rusty_cuda_ctx*, const rusty_cuda_qlinear* ql, int x_dtype, uint32_t M, int y_dtype) {
    return x_dtype == RUSTY_CUDA_F32 && strcmp(qlinear_plan(ql, x_dtype, M, y_dtype), "tcgen05") == 0 && tc_norm_fused(M, ql->K);
}

int qlinear_forward_cols(rusty_cuda_ctx* ctx, const rusty_cuda_qlinear* ql, const rusty_cuda_buf* x, int x_dtype,
                         uint32_t M, rusty_cuda_buf* y, int y_dtype, uint32_t ldy, uint32_t y_col0, const PeerPush* push,
                         const NormArgs* norm, const rusty_cuda_buf* residual) {
    if (!ql || !x || !y) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward: null argument");
    if (ql->ctx != ctx) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward: object belongs to another context");
    size_t xs = dtype_size(x_dtype), ys = dtype_size(y_dtype);
    if (!xs || !ys)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DATA_TYPE, "qlinear_forward: x/y must be f32 or bf16 (got %d, %d)", x_dtype,
                    y_dtype);
    const uint32_t out_cols = ql->act ? (y_col0 + ql->N) / 2 : y_col0 + ql->N;  // columns of y this call reaches
    if (ldy < out_cols)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_forward: row stride %u < first column %u + N %u%s", ldy,
                    y_col0, ql->N, ql->act ? " (pairs: halved)" : "");
    if (ql->act && (y_col0 & 1u))
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_forward: a shard of pairs starts at an even row, got %u", y_col0);
    if (x->bytes < (size_t)M * ql->K * xs)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_forward: x holds %zu bytes, [%u,%u] needs %zu", x->bytes, M,
                    ql->K, (size_t)M * ql->K * xs);
    if (y->bytes < (size_t)M * ldy * ys)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_forward: y holds %zu bytes, [%u,%u] needs %zu", y->bytes, M,
                    ldy, (size_t)M * ldy * ys);
    if (M == 0 || ql->N == 0) return RUSTY_CUDA_OK;
    QLinearArgs a{};
    a.w = (const uint8_t*)ql->weight->ptr;
    a.scales = (const float*)ql->scales->ptr;
    a.biases = ql->biases ? (const float*)ql->biases->ptr : nullptr;
    a.N = ql->N;
    a.K = ql->K;
    a.layout = ql->layout;
    a.qmode = ql->qmode;
    a.x = x->ptr;
    a.x_dtype = x_dtype;
    a.M = M;
    a.y = y->ptr;
    a.y_dtype = y_dtype;
    a.ldy = ldy;
    a.y_col0 = y_col0;
    a.act = ql->act;
    if (push && push->nranks > 1) {
        if (!qlinear_pushes_fused(ql, x_dtype, M, y_dtype))
            return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward: the kernel for this shape does not push to peers");
        a.push = push;
    }
    if (residual) {
        if (!qlinear_residual_fused(ql, x_dtype, M, y_dtype))
            return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward: the kernel for this shape does not add a residual");
        if (residual->bytes < (size_t)M * ldy * ys)
            return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_forward: residual holds %zu bytes, [%u,%u] needs %zu", residual->bytes, M, ldy, (size_t)M * ldy * ys);
        a.residual = residual->ptr;
    }
    if (norm) {
        if (!qlinear_norm_fused(ctx, ql, x_dtype, M, y_dtype))
            return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward: the kernel for this shape does not apply a norm");
        a.norm = norm;
    }
    DeviceGuard g(ctx->device);
    if (f16tc_supported(ctx, a) && M >= f16tc_min_rows()) return launch_f16tc(ctx, a);
    if (tc_supported(ctx, a) && M >= tc_min_rows() && (!a.act || tc_pushes_fused(M))) return launch_tc(ctx, a);
    if (gemv_mma_supported(ctx, a)) return launch_gemv_mma(ctx, a);
    if (gemv_supported(ctx, a)) return launch_gemv(ctx, a);
    return fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED,
                "qlinear_forward: no kernel for N=%u K=%u layout=%d (K %% 16 == 0 for [N,K], N %% 16 == 0 for [K,N])", ql->N,
                ql->K, ql->layout);
}

}  // namespace rusty

extern "C" {

int rusty_cuda_qlinear_create(rusty_cuda_ctx* ctx, rusty_cuda_buf* weight, rusty_cuda_buf* scales, rusty_cuda_buf* biases,
                              uint32_t N, uint32_t K, int layout, int qmode, rusty_cuda_qlinear** out) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!out) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_create: null out pointer");
    *out = nullptr;
    if (!weight || !scales) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_create: weight and scales are required");
    if (layout != RUSTY_CUDA_LAYOUT_NK && layout != RUSTY_CUDA_LAYOUT_KN)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_create: unknown layout %d", layout);
    const size_t n = (size_t)N * K;
    if (weight->bytes < n)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_create: weight holds %zu bytes, [%u,%u] needs %zu",
                    weight->bytes, N, K, n);
    if (qmode == RUSTY_CUDA_QMODE_AFFINE_G64) {
        if (!biases) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_create: AFFINE_G64 needs biases");
        // A 64-group must not straddle two rows of the stored matrix.
        uint32_t inner = layout == RUSTY_CUDA_LAYOUT_NK ? K : N;
        if (inner % 64 != 0)
            return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS,
                        "qlinear_create: AFFINE_G64 needs the contiguous dimension (%u) to be a multiple of 64", inner);
        size_t gbytes = n / 64 * 4;
        if (scales->bytes < gbytes || biases->bytes < gbytes)
            return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_create: scales/biases need %zu bytes each", gbytes);
    } else if (qmode == RUSTY_CUDA_QMODE_SYM_ROW) {
        if (biases) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_create: SYM_ROW takes no biases");
        if (scales->bytes < (size_t)N * 4)
            return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_create: scales need %zu bytes", (size_t)N * 4);
    } else {
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_create: unknown qmode %d", qmode);
    }
    {
        DeviceGuard g(ctx->device);
        int rc = tc_workspace_reserve(ctx);
        if (rc) return rc;
    }
    rusty_cuda_qlinear* q = new (std::nothrow) rusty_cuda_qlinear();
    if (!q) return fail(ctx, RUSTY_CUDA_ERR_MEMORY_ALLOCATION, "qlinear_create: host allocation failed");
    q->ctx = ctx;
    q->weight = weight;
    q->scales = scales;
    q->biases = biases;
    q->N = N;
    q->K = K;
    q->layout = layout;
    q->given_layout = layout;
    q->qmode = qmode;
    // rusty's own Linear stores [in,out] (rusty-graph/src/lib.rs:69-70: x . W).  The TMA / tensor-core kernels stream
    // rows of [out,in]; with one scale per output feature the two layouts hold the same numbers, so the weight is
    // re-laid-out ONCE here into a buffer the object owns (N*K more bytes of device memory; the caller's buffer is
    // not kept and may be released) and every later forward takes the fast kernels.  The reference re-lays its
    // weights at load as well (dequantisation to f32).  RUSTY_KN_RELAYOUT=0 keeps the [in,out] CUDA-core kernel.
    static const bool relayout = !(getenv("RUSTY_KN_RELAYOUT") && atoi(getenv("RUSTY_KN_RELAYOUT")) == 0);
    if (relayout && layout == RUSTY_CUDA_LAYOUT_KN && qmode == RUSTY_CUDA_QMODE_SYM_ROW && K % 16 == 0 && n > 0 && !ctx->capturing) {
        rusty_cuda_buf* own = nullptr;
        int rc = rusty_cuda_buf_alloc(ctx, n, 0, &own);
        if (!rc) {
            DeviceGuard g(ctx->device);
            rc = launch_transpose_u8(ctx, (const uint8_t*)weight->ptr, (uint8_t*)own->ptr, K, N);
            // the caller may free its buffer as soon as this call returns
            if (!rc) rc = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "qlinear_create: re-layout");
        }
        if (rc) {
            if (own) rusty_cuda_buf_release(own);
            delete q;
            return rc;
        }
        q->weight = own;   // the object's own reference
        q->layout = RUSTY_CUDA_LAYOUT_NK;
    } else if (relayout && layout == RUSTY_CUDA_LAYOUT_KN && qmode == RUSTY_CUDA_QMODE_AFFINE_G64 && K % 128 == 0 && N % 64 == 0 && n > 0 &&
               !ctx->capturing && gc_kernel_available(ctx, N, K)) {
        // The reference's own quantised format: [in,out] bytes with a (scale, bias) per 64 consecutive OUTPUT features
        // of an input row (rusty-loader/src/lib.rs:155-218).  Re-laid-out once as well: bytes to [out,in], scales and
        // biases to [N/64][K], all three into buffers the object owns; the tensor-core GEMV then multiplies the
        // activations by a group's scale vector instead of the weights (gemv_mma.cu).
        rusty_cuda_buf *own = nullptr, *os = nullptr, *ob = nullptr;
        const size_t gbytes = n / 64 * 4;
        int rc = rusty_cuda_buf_alloc(ctx, n, 0, &own);
        if (!rc) rc = rusty_cuda_buf_alloc(ctx, gbytes, 0, &os);
        if (!rc) rc = rusty_cuda_buf_alloc(ctx, gbytes, 0, &ob);
        if (!rc) {
            DeviceGuard g(ctx->device);
            rc = launch_transpose_u8(ctx, (const uint8_t*)weight->ptr, (uint8_t*)own->ptr, K, N);
            if (!rc) rc = launch_transpose_f32(ctx, (const float*)scales->ptr, (float*)os->ptr, K, N / 64);
            if (!rc) rc = launch_transpose_f32(ctx, (const float*)biases->ptr, (float*)ob->ptr, K, N / 64);
            if (!rc) rc = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "qlinear_create: re-layout");
        }
        if (rc) {
            if (own) rusty_cuda_buf_release(own);
            if (os) rusty_cuda_buf_release(os);
            if (ob) rusty_cuda_buf_release(ob);
            delete q;
            return rc;
        }
        q->weight = own;
        q->scales = os;
        q->biases = ob;
        q->layout = RUSTY_CUDA_LAYOUT_NK;
        q->qmode = QMODE_AFFINE_GC;
        *out = q;
        return RUSTY_CUDA_OK;
    } else {
        rusty_cuda_buf_retain(weight);
    }
    rusty_cuda_buf_retain(scales);
    if (biases) rusty_cuda_buf_retain(biases);
    *out = q;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_qlinear_set_activation(rusty_cuda_qlinear* ql, int act) {
    if (!ql) return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_set_activation: null qlinear");
    if (act != RUSTY_CUDA_ACT_NONE && act != RUSTY_CUDA_ACT_SWIGLU_PAIRS)
        return fail(ql->ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_set_activation: unknown activation %d", act);
    if (act == RUSTY_CUDA_ACT_SWIGLU_PAIRS) {
        if (ql->given_layout != RUSTY_CUDA_LAYOUT_NK || ql->qmode != RUSTY_CUDA_QMODE_SYM_ROW)
            return fail(ql->ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "qlinear_set_activation: pairs need [out,in] storage with one scale per row");
        if (ql->N % 2 != 0)
            return fail(ql->ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_set_activation: %u rows are not whole (gate, up) pairs", ql->N);
    }
    ql->act = act;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_qlinear_destroy(rusty_cuda_qlinear* ql) {
    if (!ql) return RUSTY_CUDA_OK;
    rusty_cuda_buf_release(ql->weight);
    rusty_cuda_buf_release(ql->scales);
    if (ql->biases) rusty_cuda_buf_release(ql->biases);
    delete ql;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_qlinear_forward(rusty_cuda_ctx* ctx, const rusty_cuda_qlinear* ql, const rusty_cuda_buf* x, int x_dtype,
                               uint32_t M, rusty_cuda_buf* y, int y_dtype) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!ql) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward: null qlinear");
    return qlinear_forward_cols(ctx, ql, x, x_dtype, M, y, y_dtype, ql->act ? ql->N / 2 : ql->N, 0);
}

int rusty_cuda_qlinear_forward_residual(rusty_cuda_ctx* ctx, const rusty_cuda_qlinear* ql, const rusty_cuda_buf* x, int x_dtype, uint32_t M,
                                        const rusty_cuda_buf* residual, rusty_cuda_buf* y, int y_dtype) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!ql || !x || !residual || !y) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_residual: null argument");
    if (ql->act) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_residual: not for a weight with the pair activation");
    const size_t ys = y_dtype == RUSTY_CUDA_BF16 ? 2 : y_dtype == RUSTY_CUDA_F32 ? 4 : 0;
    if (!ys) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DATA_TYPE, "qlinear_forward_residual: y must be f32 or bf16");
    const size_t out_b = (size_t)M * ql->N * ys;
    if (residual->bytes < out_b || y->bytes < out_b)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_forward_residual: residual / y smaller than [%u,%u] (%zu bytes)", M, ql->N, out_b);
    if (M == 0 || ql->N == 0) return RUSTY_CUDA_OK;
    if (qlinear_residual_fused(ql, x_dtype, M, y_dtype))
        return qlinear_forward_cols(ctx, ql, x, x_dtype, M, y, y_dtype, ql->N, 0, nullptr, nullptr, residual);
    // Other kernels: the Linear into y (or, when the residual IS y, into a buffer borrowed from the pool), then one add.
    rusty_cuda_buf* tmp = nullptr;
    rusty_cuda_buf* lin = y;
    if (residual->ptr == y->ptr) {
        int rc = rusty_cuda_buf_alloc(ctx, out_b, 1, &tmp);
        if (rc) return rc;
        lin = tmp;
    }
    int rc = qlinear_forward_cols(ctx, ql, x, x_dtype, M, lin, y_dtype, ql->N, 0);
    if (!rc) {
        DeviceGuard g(ctx->device);
        rc = launch_residual_add(ctx, lin->ptr, residual->ptr, y->ptr, (size_t)M * ql->N, y_dtype);
    }
    if (tmp) rusty_cuda_buf_release(tmp);
    return rc;
}

int rusty_cuda_qlinear_forward_normed(rusty_cuda_ctx* ctx, const rusty_cuda_qlinear* ql, const rusty_cuda_buf* x, const rusty_cuda_buf* residual,
                                      const rusty_cuda_buf* norm_weight, float eps, uint32_t M, rusty_cuda_buf* normed_out, rusty_cuda_buf* sum_out,
                                      rusty_cuda_buf* y, int y_dtype) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!ql || !x || !norm_weight || !y) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_normed: null argument");
    if (sum_out && !residual) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_normed: sum_out without a residual");
    if (!(eps >= 0.0f)) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_normed: eps must be >= 0");
    const uint32_t K = ql->K;
    if (K % 4 != 0) return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_forward_normed: K=%u must be a multiple of 4", K);
    const size_t rows_b = (size_t)M * K * 4;
    if (x->bytes < rows_b || (residual && residual->bytes < rows_b) || (normed_out && normed_out->bytes < rows_b) || (sum_out && sum_out->bytes < rows_b))
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_forward_normed: a buffer is smaller than [%u,%u] f32 (%zu bytes)", M, K, rows_b);
    if (norm_weight->bytes < (size_t)K * 4)
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_DIMENSIONS, "qlinear_forward_normed: norm weight holds %zu bytes, [%u] needs %zu", norm_weight->bytes, K, (size_t)K * 4);
    if ((normed_out && (normed_out == x || normed_out == residual)) || (sum_out && (sum_out == x || sum_out == normed_out)))
        return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_normed: normed_out must not alias an input, sum_out must not alias x or normed_out");
    const uint32_t ldy = ql->act ? ql->N / 2 : ql->N;
    if (M == 0) return RUSTY_CUDA_OK;
    if (qlinear_norm_fused(ctx, ql, RUSTY_CUDA_F32, M, y_dtype)) {
        NormArgs n{residual ? (const float*)residual->ptr : nullptr, (const float*)norm_weight->ptr, eps,
                   normed_out ? (float*)normed_out->ptr : nullptr, sum_out ? (float*)sum_out->ptr : nullptr};
        return qlinear_forward_cols(ctx, ql, x, RUSTY_CUDA_F32, M, y, y_dtype, ldy, 0, nullptr, &n);
    }
    // Other kernels: the norm as a kernel of its own, into normed_out or into a buffer borrowed from the pool.  The
    // pool hands a buffer back to later calls on the same stream only, so it can be released as soon as the Linear
    // that reads it has been enqueued.
    rusty_cuda_buf* tmp = nullptr;
    if (!normed_out) {
        int rc = rusty_cuda_buf_alloc(ctx, rows_b, 1, &tmp);
        if (rc) return rc;   // (under a stream capture this needs an idle pool buffer of that size: pass normed_out there)
        normed_out = tmp;
    }
    int rc;
    {
        DeviceGuard g(ctx->device);
        rc = launch_rms_norm(ctx, (const float*)x->ptr, residual ? (const float*)residual->ptr : nullptr, (const float*)norm_weight->ptr,
                             (float*)normed_out->ptr, sum_out ? (float*)sum_out->ptr : nullptr, M, K, eps);
    }
    if (!rc) rc = qlinear_forward_cols(ctx, ql, normed_out, RUSTY_CUDA_F32, M, y, y_dtype, ldy, 0);
    if (tmp) rusty_cuda_buf_release(tmp);
    return rc;
}

int rusty_cuda_qlinear_forward_batch(rusty_cuda_ctx* ctx, size_t n, const rusty_cuda_qlinear* const* qls,
                                     const rusty_cuda_buf* const* xs, int x_dtype, uint32_t M, rusty_cuda_buf* const* ys,
                                     int y_dtype) {
    RUSTY_REQUIRE_CTX(ctx);
    if (n && (!qls || !xs || !ys)) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_batch: null array");
    for (size_t i = 0; i < n; ++i) {
        if (!qls[i]) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_forward_batch: entry %zu is null", i);
        int rc = qlinear_forward_cols(ctx, qls[i], xs[i], x_dtype, M, ys[i], y_dtype, qls[i]->act ? qls[i]->N / 2 : qls[i]->N, 0);
        if (rc) return rc;
    }
    return RUSTY_CUDA_OK;
}

int rusty_cuda_qlinear_plan(const rusty_cuda_qlinear* ql, int x_dtype, uint32_t M, int y_dtype, char* dst, size_t dst_len) {
    if (!ql || !dst || !dst_len) return fail(nullptr, RUSTY_CUDA_ERR_INVALID_OPERATION, "qlinear_plan: null argument");
    snprintf(dst, dst_len, "%s", qlinear_plan(ql, x_dtype, M, y_dtype));
    return RUSTY_CUDA_OK;
}

}  // extern "C"
