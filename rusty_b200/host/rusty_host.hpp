// C++17 host mirror of rusty's tensor / engine / Linear surface over the C ABI
// (include/rusty_cuda.h).  Header-only; link against librusty_cuda.
//
//   rusty::CudaContext    <- WgpuContext          rusty-backend/src/lib.rs:11-53
//   rusty::DType          <- DType                lib.rs:56-76 (+ BF16, I8, U8)
//   rusty::UnifiedTensor  <- UnifiedTensor        lib.rs:78-241 (clone shares storage, drop releases)
//   rusty::ComputeEngine  <- ComputeEngine        lib.rs:343, ops :4019-4990
//   rusty::LoRAAdapter, rusty::Linear             rusty-graph/src/lib.rs:16-110
//   rusty::QWeight        <- the int8 weight Linear multiplies in place of the
//                            load-time-dequantised f32 copy (rusty-loader/src/lib.rs:155-218)
// The reference panics on failure; here every non-zero status becomes a
// rusty::BackendError carrying the BackendError variant name (error.rs:13-61).
#pragma once

#include <cstdint>
#include <cstring>
#include <memory>
#include <numeric>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "rusty_cuda.h"

namespace rusty {

class BackendError : public std::runtime_error {
public:
    BackendError(int code, const std::string& msg) : std::runtime_error(kind_of(code) + ": " + msg), code_(code) {}
    int code() const { return code_; }
    static std::string kind_of(int c) {
        static const char* names[] = {"Ok", "GpuInitialization", "MemoryAllocation", "InvalidDimensions", "InvalidDataType",
                                      "BufferOperation", "KernelExecution", "UnsupportedOperation", "DataTransfer",
                                      "InvalidOperation", "Timeout", "Other"};
        return (c >= 0 && c <= 11) ? names[c] : "Other";
    }
private:
    int code_;
};

inline void check(int rc, rusty_cuda_ctx* ctx = nullptr) {
    if (rc != RUSTY_CUDA_OK) throw BackendError(rc, rusty_cuda_last_error(ctx));
}

enum class DType : int { FP32 = RUSTY_CUDA_F32, FP16 = RUSTY_CUDA_F16, BF16 = RUSTY_CUDA_BF16, I8 = RUSTY_CUDA_I8, U8 = RUSTY_CUDA_U8 };
inline size_t size_bytes(DType d) { return d == DType::FP32 ? 4 : (d == DType::FP16 || d == DType::BF16) ? 2 : 1; }

class CudaContext {
public:
    explicit CudaContext(int device = 0) { check(rusty_cuda_ctx_create(device, &raw_)); }
    ~CudaContext() { rusty_cuda_ctx_destroy(raw_); }
    CudaContext(const CudaContext&) = delete;
    CudaContext& operator=(const CudaContext&) = delete;
    rusty_cuda_ctx* raw() const { return raw_; }
    std::string adapter_info() const {
        char buf[256];
        check(rusty_cuda_ctx_adapter_info(raw_, buf, sizeof buf), raw_);
        return buf;
    }
    void sync() const { check(rusty_cuda_sync(raw_), raw_); }
private:
    rusty_cuda_ctx* raw_ = nullptr;
};

inline size_t numel(const std::vector<size_t>& shape) {
    return std::accumulate(shape.begin(), shape.end(), size_t(1), [](size_t a, size_t b) { return a * b; });
}

class UnifiedTensor {
public:
    std::vector<size_t> shape;
    DType dtype = DType::FP32;

    // UnifiedTensor::new (lib.rs:115): fresh, initialised, not pooled
    static UnifiedTensor make(const CudaContext& ctx, const float* data, const std::vector<size_t>& shape) {
        return from_bytes(ctx, data, numel(shape) * 4, shape, DType::FP32);
    }
    // UnifiedTensor::empty (lib.rs:137): pooled, uninitialised
    static UnifiedTensor empty(const CudaContext& ctx, const std::vector<size_t>& shape, DType dt = DType::FP32) {
        UnifiedTensor t;
        t.bytes_ = numel(shape) * size_bytes(dt);
        check(rusty_cuda_buf_alloc(ctx.raw(), t.bytes_, 1, &t.buf_), ctx.raw());
        t.shape = shape;
        t.dtype = dt;
        return t;
    }
    static UnifiedTensor from_bytes(const CudaContext& ctx, const void* data, size_t bytes, const std::vector<size_t>& shape,
                                    DType dt) {
        UnifiedTensor t;
        t.bytes_ = bytes;
        check(rusty_cuda_buf_alloc(ctx.raw(), bytes, 0, &t.buf_), ctx.raw());
        check(rusty_cuda_buf_upload(ctx.raw(), t.buf_, 0, data, bytes), ctx.raw());
        t.shape = shape;
        t.dtype = dt;
        return t;
    }
    UnifiedTensor() = default;
    UnifiedTensor(const UnifiedTensor& o) : shape(o.shape), dtype(o.dtype), buf_(o.buf_), bytes_(o.bytes_) {
        if (buf_) rusty_cuda_buf_retain(buf_);
    }
    UnifiedTensor(UnifiedTensor&& o) noexcept : shape(std::move(o.shape)), dtype(o.dtype), buf_(o.buf_), bytes_(o.bytes_) { o.buf_ = nullptr; }
    UnifiedTensor& operator=(UnifiedTensor o) {
        std::swap(shape, o.shape);
        std::swap(dtype, o.dtype);
        std::swap(buf_, o.buf_);
        std::swap(bytes_, o.bytes_);
        return *this;
    }
    ~UnifiedTensor() {
        if (buf_) rusty_cuda_buf_release(buf_);
    }
    rusty_cuda_buf* buffer() const { return buf_; }
    size_t size_in_bytes() const { return bytes_; }
    // reshaped (lib.rs:198): a view sharing storage; sizes must match
    UnifiedTensor reshaped(const std::vector<size_t>& new_shape) const {
        if (numel(new_shape) != numel(shape)) throw std::invalid_argument("Cannot reshape tensor: element counts differ");
        UnifiedTensor v(*this);
        v.shape = new_shape;
        return v;
    }
    // to_vec (lib.rs:215): blocking readback as f32
    std::vector<float> to_vec(const CudaContext& ctx) const {
        std::vector<float> out(bytes_ / 4);
        check(rusty_cuda_buf_download(ctx.raw(), buf_, 0, out.data(), out.size() * 4), ctx.raw());
        return out;
    }
    void write_data(const CudaContext& ctx, const void* data, size_t bytes) const {
        check(rusty_cuda_buf_upload(ctx.raw(), buf_, 0, data, bytes), ctx.raw());
    }
private:
    rusty_cuda_buf* buf_ = nullptr;
    size_t bytes_ = 0;
};

// A weight kept in its 1-byte quantised form.
class QWeight {
public:
    QWeight(const CudaContext& ctx, const UnifiedTensor& w, const UnifiedTensor& scales, const UnifiedTensor* biases, uint32_t out_features,
            uint32_t in_features, int layout, int qmode)
        : N(out_features), K(in_features), keep_w_(w), keep_s_(scales) {
        if (biases) keep_b_ = *biases;
        check(rusty_cuda_qlinear_create(ctx.raw(), w.buffer(), scales.buffer(), biases ? biases->buffer() : nullptr, N, K, layout, qmode,
                                        &raw_),
              ctx.raw());
    }
    ~QWeight() { rusty_cuda_qlinear_destroy(raw_); }
    QWeight(const QWeight&) = delete;
    QWeight& operator=(const QWeight&) = delete;
    rusty_cuda_qlinear* raw() const { return raw_; }
    // RUSTY_CUDA_ACT_SWIGLU_PAIRS: rows (2j, 2j+1) are (gate_j, up_j); forwards then write silu(gate) * up, N/2 columns
    void set_activation(const CudaContext& ctx, int act) {
        check(rusty_cuda_qlinear_set_activation(raw_, act), ctx.raw());
        act_ = act;
    }
    uint32_t out_features() const { return act_ == RUSTY_CUDA_ACT_SWIGLU_PAIRS ? N / 2 : N; }
    const uint32_t N, K;
private:
    int act_ = RUSTY_CUDA_ACT_NONE;
    rusty_cuda_qlinear* raw_ = nullptr;
    UnifiedTensor keep_w_, keep_s_, keep_b_;
};

class ComputeEngine {
public:
    explicit ComputeEngine(const CudaContext&) {}
    void matmul(const CudaContext& ctx, const UnifiedTensor& a, const UnifiedTensor& b, const UnifiedTensor& out) const {
        check(rusty_cuda_matmul_f32(ctx.raw(), a.buffer(), b.buffer(), out.buffer(), (uint32_t)a.shape[0], (uint32_t)a.shape[1],
                                    (uint32_t)b.shape[1]),
              ctx.raw());
    }
    void matmul_bt(const CudaContext& ctx, const UnifiedTensor& a, const UnifiedTensor& b, const UnifiedTensor& out) const {
        check(rusty_cuda_matmul_bt_f32(ctx.raw(), a.buffer(), b.buffer(), out.buffer(), (uint32_t)a.shape[0], (uint32_t)a.shape[1],
                                       (uint32_t)b.shape[0]),
              ctx.raw());
    }
    void dequantize(const CudaContext& ctx, const UnifiedTensor& input, const UnifiedTensor& out) const {
        check(rusty_cuda_dequantize_u8(ctx.raw(), input.buffer(), out.buffer(), numel(input.shape)), ctx.raw());
    }
    void affine_dequantize(const CudaContext& ctx, const UnifiedTensor& w, const UnifiedTensor& scales, const UnifiedTensor& biases,
                           const UnifiedTensor& out) const {
        check(rusty_cuda_affine_dequantize_g64(ctx.raw(), w.buffer(), scales.buffer(), biases.buffer(), out.buffer(), numel(out.shape)),
              ctx.raw());
    }
    void add(const CudaContext& ctx, const UnifiedTensor& a, const UnifiedTensor& b, const UnifiedTensor& out) const {
        check(rusty_cuda_add_f32(ctx.raw(), a.buffer(), b.buffer(), out.buffer(), numel(out.shape)), ctx.raw());
    }
    // WGSL silu / mul (kernels.wgsl:104-113, :146-151): the glue of MLP::forward
    void silu(const CudaContext& ctx, const UnifiedTensor& x, const UnifiedTensor& out) const {
        check(rusty_cuda_silu_f32(ctx.raw(), x.buffer(), out.buffer(), numel(out.shape)), ctx.raw());
    }
    void mul(const CudaContext& ctx, const UnifiedTensor& a, const UnifiedTensor& b, const UnifiedTensor& out) const {
        check(rusty_cuda_mul_f32(ctx.raw(), a.buffer(), b.buffer(), out.buffer(), numel(out.shape)), ctx.raw());
    }
    void copy_tensor(const CudaContext& ctx, const UnifiedTensor& src, const UnifiedTensor& dst, size_t dst_offset) const {
        check(rusty_cuda_buf_copy(ctx.raw(), src.buffer(), dst.buffer(), dst_offset), ctx.raw());
    }
    void qlinear(const CudaContext& ctx, const UnifiedTensor& x, const QWeight& w, const UnifiedTensor& out) const {
        const size_t rows = numel(x.shape) / x.shape.back();
        check(rusty_cuda_qlinear_forward(ctx.raw(), w.raw(), x.buffer(), (int)x.dtype, (uint32_t)rows, out.buffer(), (int)out.dtype),
              ctx.raw());
    }
    // ComputeEngine::rms_norm (rusty-backend/src/lib.rs:4492) for every row of input[..., K]
    void rms_norm(const CudaContext& ctx, const UnifiedTensor& input, const UnifiedTensor& weight, const UnifiedTensor& out,
                  float eps = 1e-5f) const {
        const size_t K = input.shape.back(), rows = numel(input.shape) / K;
        check(rusty_cuda_rms_norm_f32(ctx.raw(), input.buffer(), nullptr, weight.buffer(), out.buffer(), nullptr, (uint32_t)rows, (uint32_t)K, eps),
              ctx.raw());
    }
    // ComputeEngine::rms_norm_residual (rusty-backend/src/lib.rs:5320), row by row; sum_out (optional) receives x + residual
    void rms_norm_residual(const CudaContext& ctx, const UnifiedTensor& x, const UnifiedTensor& residual, const UnifiedTensor& weight,
                           const UnifiedTensor& out, const UnifiedTensor* sum_out = nullptr, float eps = 1e-5f) const {
        const size_t K = x.shape.back(), rows = numel(x.shape) / K;
        check(rusty_cuda_rms_norm_f32(ctx.raw(), x.buffer(), residual.buffer(), weight.buffer(), out.buffer(),
                                      sum_out ? sum_out->buffer() : nullptr, (uint32_t)rows, (uint32_t)K, eps), ctx.raw());
    }
    // Embedding::forward (rusty-graph/src/lib.rs:121-135) with the ids (u32) in a device tensor
    void embedding(const CudaContext& ctx, const UnifiedTensor& table, const UnifiedTensor& ids, size_t n_ids, const UnifiedTensor& out) const {
        check(rusty_cuda_embedding_f32(ctx.raw(), table.buffer(), ids.buffer(), out.buffer(), n_ids, (uint32_t)table.shape[0],
                                       (uint32_t)table.shape[1]), ctx.raw());
    }
    // out = w(RMSNorm(x [+ residual]) * norm_weight): the norm rides in the Linear's activation pre-pass where it can
    void qlinear_normed(const CudaContext& ctx, const UnifiedTensor& x, const UnifiedTensor& norm_weight, const QWeight& w,
                        const UnifiedTensor& out, const UnifiedTensor* residual = nullptr, const UnifiedTensor* normed_out = nullptr,
                        const UnifiedTensor* sum_out = nullptr, float eps = 1e-5f) const {
        const size_t rows = numel(x.shape) / x.shape.back();
        check(rusty_cuda_qlinear_forward_normed(ctx.raw(), w.raw(), x.buffer(), residual ? residual->buffer() : nullptr, norm_weight.buffer(),
                                                eps, (uint32_t)rows, normed_out ? normed_out->buffer() : nullptr,
                                                sum_out ? sum_out->buffer() : nullptr, out.buffer(), (int)out.dtype), ctx.raw());
    }
    // out = residual + w(x): the residual add after o_proj / down_proj in the Linear's epilogue (out may be residual)
    void qlinear_residual(const CudaContext& ctx, const UnifiedTensor& x, const QWeight& w, const UnifiedTensor& residual,
                          const UnifiedTensor& out) const {
        const size_t rows = numel(x.shape) / x.shape.back();
        check(rusty_cuda_qlinear_forward_residual(ctx.raw(), w.raw(), x.buffer(), (int)x.dtype, (uint32_t)rows, residual.buffer(),
                                                  out.buffer(), (int)out.dtype), ctx.raw());
    }
};

struct LoRAAdapter {
    UnifiedTensor a;  // [in, rank], filled with 0.01 (rusty-graph/src/lib.rs:38-43)
    UnifiedTensor b;  // [rank, out], zeros
    float alpha;
    size_t rank;
    LoRAAdapter(const CudaContext& ctx, size_t in_dim, size_t out_dim, size_t r, float al) : alpha(al), rank(r) {
        std::vector<float> va(in_dim * r, 0.01f), vb(r * out_dim, 0.0f);
        a = UnifiedTensor::make(ctx, va.data(), {in_dim, r});
        b = UnifiedTensor::make(ctx, vb.data(), {r, out_dim});
    }
};

// Linear keeps the reference contract: forward(engine, x) = x . W[in,out] (+ (x.A).B, no alpha/rank scaling,
// rusty-graph/src/lib.rs:69-84); from_quantized routes the same call to the fused int8 kernels.
class Linear {
public:
    static Linear make(const CudaContext& ctx, UnifiedTensor weight) { return Linear(ctx, std::move(weight), nullptr, nullptr); }
    static Linear with_lora(const CudaContext& ctx, UnifiedTensor weight, std::shared_ptr<LoRAAdapter> lora) {
        return Linear(ctx, std::move(weight), nullptr, std::move(lora));
    }
    static Linear from_quantized(const CudaContext& ctx, std::shared_ptr<QWeight> q) { return Linear(ctx, UnifiedTensor(), std::move(q), nullptr); }

    UnifiedTensor forward(const ComputeEngine& engine, const UnifiedTensor& x, DType out_dtype = DType::FP32) const {
        const size_t k = q_ ? q_->K : weight_.shape[0];
        const size_t n = q_ ? q_->out_features() : weight_.shape[1];
        if (x.shape.empty() || x.shape.back() != k) throw std::invalid_argument("Linear: last dimension of x does not match in_features");
        const size_t rows = numel(x.shape) / k;
        UnifiedTensor x2 = x.reshaped({rows, k});
        UnifiedTensor out;
        if (q_) {
            out = UnifiedTensor::empty(ctx_, {rows, n}, out_dtype);
            engine.qlinear(ctx_, x2, *q_, out);
        } else {
            out = UnifiedTensor::empty(ctx_, {rows, n});
            engine.matmul(ctx_, x2, weight_, out);
        }
        if (lora_) {
            UnifiedTensor temp = UnifiedTensor::empty(ctx_, {rows, lora_->rank});
            engine.matmul(ctx_, x2, lora_->a, temp);
            UnifiedTensor lora_out = UnifiedTensor::empty(ctx_, {rows, n});
            engine.matmul(ctx_, temp, lora_->b, lora_out);
            UnifiedTensor summed = UnifiedTensor::empty(ctx_, {rows, n});
            engine.add(ctx_, out, lora_out, summed);
            out = summed;
        }
        std::vector<size_t> oshape(x.shape.begin(), x.shape.end() - 1);
        oshape.push_back(n);
        return out.reshaped(oshape);
    }
private:
    Linear(const CudaContext& ctx, UnifiedTensor w, std::shared_ptr<QWeight> q, std::shared_ptr<LoRAAdapter> l)
        : ctx_(ctx), weight_(std::move(w)), q_(std::move(q)), lora_(std::move(l)) {}
    const CudaContext& ctx_;
    UnifiedTensor weight_;
    std::shared_ptr<QWeight> q_;
    std::shared_ptr<LoRAAdapter> lora_;
};

// Several GPUs, one process each (no counterpart in the reference): an arena with the same layout on every rank whose
// buffers the fused linear of every rank writes into.  Handles (RUSTY_CUDA_IPC_HANDLE_BYTES each) travel over any
// host channel; all ranks issue the same sequence of pushed forwards.
class Arena {
public:
    Arena(const CudaContext& ctx, size_t bytes, int nranks, int rank) : ctx_(ctx), nranks_(nranks) {
        check(rusty_cuda_arena_create(ctx.raw(), bytes, nranks, rank, &raw_), ctx.raw());
    }
    ~Arena() { rusty_cuda_arena_destroy(raw_); }
    Arena(const Arena&) = delete;
    Arena& operator=(const Arena&) = delete;
    std::vector<unsigned char> export_handle() const {
        std::vector<unsigned char> h(RUSTY_CUDA_IPC_HANDLE_BYTES);
        check(rusty_cuda_arena_export(raw_, h.data()), ctx_.raw());
        return h;
    }
    // handles of all ranks back to back, in rank order
    void attach(const std::vector<unsigned char>& handles) {
        if (handles.size() != (size_t)nranks_ * RUSTY_CUDA_IPC_HANDLE_BYTES) throw std::invalid_argument("Arena::attach: one handle per rank");
        check(rusty_cuda_arena_attach(raw_, handles.data()), ctx_.raw());
    }
    // y_full[M, N] of a pushed forward: columns [rank*N/G, (rank+1)*N/G) come from rank's kernel
    void forward_pushed(const QWeight& shard, const UnifiedTensor& x, rusty_cuda_buf* y_full, DType y_dtype) const {
        const size_t rows = numel(x.shape) / x.shape.back();
        check(rusty_cuda_qlinear_forward_pushed(ctx_.raw(), raw_, shard.raw(), x.buffer(), (int)x.dtype, (uint32_t)rows, y_full, (int)y_dtype),
              ctx_.raw());
    }
    rusty_cuda_buf* buffer(size_t offset, size_t bytes) const {
        rusty_cuda_buf* b = nullptr;
        check(rusty_cuda_arena_buf(raw_, offset, bytes, &b), ctx_.raw());
        return b;  // release with rusty_cuda_buf_release
    }
    void wait() const { check(rusty_cuda_arena_wait(ctx_.raw(), raw_), ctx_.raw()); }
    rusty_cuda_arena* raw() const { return raw_; }
private:
    const CudaContext& ctx_;
    int nranks_;
    rusty_cuda_arena* raw_ = nullptr;
};

// MLP keeps the reference contract (rusty-graph/src/lib.rs:310-323): down(silu(gate(x)) * up(x)).  `fused` builds it
// from ONE pair-interleaved gate|up weight whose kernel applies silu(gate) * up in its epilogue.
class MLP {
public:
    MLP(const CudaContext& ctx, Linear gate, Linear up, Linear down)
        : ctx_(ctx), gate_(std::make_unique<Linear>(std::move(gate))), up_(std::make_unique<Linear>(std::move(up))),
          down_(std::make_unique<Linear>(std::move(down))) {}
    static MLP fused(const CudaContext& ctx, std::shared_ptr<QWeight> gate_up_pairs, Linear down) {
        gate_up_pairs->set_activation(ctx, RUSTY_CUDA_ACT_SWIGLU_PAIRS);
        MLP m(ctx, std::move(down));
        m.gate_up_ = std::make_unique<Linear>(Linear::from_quantized(ctx, std::move(gate_up_pairs)));
        return m;
    }
    UnifiedTensor forward(const ComputeEngine& engine, const UnifiedTensor& input) const {
        if (gate_up_) return down_->forward(engine, gate_up_->forward(engine, input));
        UnifiedTensor gate_linear = gate_->forward(engine, input);
        UnifiedTensor gate_act = UnifiedTensor::empty(ctx_, gate_linear.shape);
        engine.silu(ctx_, gate_linear, gate_act);
        UnifiedTensor up = up_->forward(engine, input);
        UnifiedTensor fused = UnifiedTensor::empty(ctx_, up.shape);
        engine.mul(ctx_, gate_act, up, fused);
        return down_->forward(engine, fused);
    }
private:
    MLP(const CudaContext& ctx, Linear down) : ctx_(ctx), down_(std::make_unique<Linear>(std::move(down))) {}
    const CudaContext& ctx_;
    std::unique_ptr<Linear> gate_, up_, down_, gate_up_;
};

}  // namespace rusty
