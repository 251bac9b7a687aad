// Exercises the C++ host mirror (rusty_b200/host/rusty_host.hpp) the way a test in rusty-backend / rusty-graph
// would: the ops_test.rs identity product, a quantised Linear against a scalar restatement of
// dequantise-then-matmul_bt, LoRA, views, and the error path.  Prints "ok" and exits 0 on success.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <random>

#include "rusty_host.hpp"

using namespace rusty;

#define REQUIRE(cond)                                                         \
    do {                                                                      \
        if (!(cond)) {                                                        \
            std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            return 1;                                                         \
        }                                                                     \
    } while (0)

int main() {
    CudaContext ctx(0);
    ComputeEngine engine(ctx);
    std::printf("%s\n", ctx.adapter_info().c_str());

    // rusty-backend/examples/ops_test.rs:9-17
    float a[4] = {1, 2, 3, 4}, id[4] = {1, 0, 0, 1};
    auto ta = UnifiedTensor::make(ctx, a, {2, 2});
    auto tb = UnifiedTensor::make(ctx, id, {2, 2});
    auto out = UnifiedTensor::empty(ctx, {2, 2});
    engine.matmul(ctx, ta, tb, out);
    auto v = out.to_vec(ctx);
    REQUIRE(v[0] == 1 && v[1] == 2 && v[2] == 3 && v[3] == 4);

    // a view shares storage
    auto view = ta.reshaped({4});
    REQUIRE(view.buffer() == ta.buffer());

    // quantised Linear, 3-D activations flattened to rows
    const size_t K = 256, N = 96, B = 2, S = 3;
    std::mt19937 rng(5);
    std::normal_distribution<float> nd(0.f, 1.f);
    std::uniform_int_distribution<int> qd(-127, 127);
    std::uniform_real_distribution<float> sd(0.001f, 0.02f);
    std::vector<float> x(B * S * K), sc(N);
    std::vector<int8_t> q(N * K);
    for (auto& e : x) e = nd(rng);
    for (auto& e : q) e = (int8_t)qd(rng);
    for (auto& e : sc) e = sd(rng);
    auto tq = UnifiedTensor::from_bytes(ctx, q.data(), q.size(), {N, K}, DType::I8);
    auto ts = UnifiedTensor::make(ctx, sc.data(), {N});
    auto qw = std::make_shared<QWeight>(ctx, tq, ts, nullptr, (uint32_t)N, (uint32_t)K, RUSTY_CUDA_LAYOUT_NK, RUSTY_CUDA_QMODE_SYM_ROW);
    Linear lin = Linear::from_quantized(ctx, qw);
    auto tx = UnifiedTensor::make(ctx, x.data(), {B, S, K});
    auto y = lin.forward(engine, tx);
    REQUIRE(y.shape.size() == 3 && y.shape[0] == B && y.shape[1] == S && y.shape[2] == N);
    auto yv = y.to_vec(ctx);
    double max_ref = 0, max_err = 0;
    for (size_t r = 0; r < B * S; ++r)
        for (size_t n = 0; n < N; ++n) {
            float acc = 0.0f;  // the reference arithmetic: k ascending, f32, W = f32(q) * scale
            for (size_t k = 0; k < K; ++k) acc = acc + x[r * K + k] * ((float)q[n * K + k] * sc[n]);
            max_ref = std::fmax(max_ref, std::fabs(acc));
            max_err = std::fmax(max_err, std::fabs((double)yv[r * N + n] - acc));
        }
    REQUIRE(max_err / max_ref <= 1e-5);

    // LoRA branch with B = 0 adds nothing
    std::vector<float> w(K * N);
    for (auto& e : w) e = nd(rng);
    auto tw = UnifiedTensor::make(ctx, w.data(), {K, N});
    auto plain = Linear::make(ctx, tw).forward(engine, tx).to_vec(ctx);
    auto lora = std::make_shared<LoRAAdapter>(ctx, K, N, 4, 16.0f);
    auto with = Linear::with_lora(ctx, tw, lora).forward(engine, tx).to_vec(ctx);
    REQUIRE(plain == with);

    // MLP::forward (rusty-graph/src/lib.rs:317-323): gate, silu, up, mul, down as separate operators, against the
    // same MLP built from ONE pair-interleaved gate|up weight whose kernel applies silu(gate) * up itself
    {
        const size_t F = 160;
        std::vector<int8_t> gq(F * K), uq(F * K), dq(K * F), pq(2 * F * K);
        std::vector<float> gs(F), us(F), ds(K), ps(2 * F);
        for (auto& e : gq) e = (int8_t)qd(rng);
        for (auto& e : uq) e = (int8_t)qd(rng);
        for (auto& e : dq) e = (int8_t)qd(rng);
        for (auto& e : gs) e = sd(rng) * 0.1f;
        for (auto& e : us) e = sd(rng);
        for (auto& e : ds) e = sd(rng);
        for (size_t j = 0; j < F; ++j) {
            std::copy(gq.begin() + j * K, gq.begin() + (j + 1) * K, pq.begin() + (2 * j) * K);
            std::copy(uq.begin() + j * K, uq.begin() + (j + 1) * K, pq.begin() + (2 * j + 1) * K);
            ps[2 * j] = gs[j];
            ps[2 * j + 1] = us[j];
        }
        auto mk = [&](const std::vector<int8_t>& qq, const std::vector<float>& ss, size_t n, size_t k) {
            auto t1 = UnifiedTensor::from_bytes(ctx, qq.data(), qq.size(), {n, k}, DType::I8);
            auto t2 = UnifiedTensor::make(ctx, ss.data(), {n});
            return std::make_shared<QWeight>(ctx, t1, t2, nullptr, (uint32_t)n, (uint32_t)k, RUSTY_CUDA_LAYOUT_NK, RUSTY_CUDA_QMODE_SYM_ROW);
        };
        MLP unfused(ctx, Linear::from_quantized(ctx, mk(gq, gs, F, K)), Linear::from_quantized(ctx, mk(uq, us, F, K)),
                    Linear::from_quantized(ctx, mk(dq, ds, K, F)));
        MLP fused = MLP::fused(ctx, mk(pq, ps, 2 * F, K), Linear::from_quantized(ctx, mk(dq, ds, K, F)));
        auto y1 = unfused.forward(engine, tx).to_vec(ctx);
        auto y2 = fused.forward(engine, tx).to_vec(ctx);
        REQUIRE(y1.size() == B * S * K && y2.size() == y1.size());
        double mref = 0, merr = 0;
        for (size_t i = 0; i < y1.size(); ++i) {
            mref = std::fmax(mref, std::fabs(y1[i]));
            merr = std::fmax(merr, std::fabs((double)y1[i] - y2[i]));
        }
        REQUIRE(mref > 0 && merr / mref <= 1e-5);
    }

    // errors are exceptions carrying the BackendError variant, and the context survives
    bool threw = false;
    try {
        auto small = UnifiedTensor::empty(ctx, {1, 1});
        engine.matmul(ctx, ta, tb, small);
    } catch (const BackendError& e) {
        threw = e.code() == RUSTY_CUDA_ERR_INVALID_DIMENSIONS;
    }
    REQUIRE(threw);
    ctx.sync();
    std::printf("ok\n");
    return 0;
}
