/*
 * CPU oracle for rusty's quantized-linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the four WGSL compute
 * shaders that make up the reference's int8-dequantize -> matmul path, plus
 * the compositions the reference builds from them at model-load and at
 * Linear::forward time.  It is the checker for the CUDA kernels; nothing that
 * ships links it, and no product code path may call it.
 *
 * PARITY UNPINNED: the reference has no test, golden vector or fixture that
 * asserts a matmul / matmul_bt / dequantize / affine_dequantize result, and
 * its Rust + WGSL sources cannot be compiled or run without a Rust toolchain
 * and a graphics stack.  The oracle is therefore pinned only by the shader
 * source it follows (cited per function) and by the one informal anchor the
 * reference holds (rusty-backend/examples/ops_test.rs:9-17, [[1,2],[3,4]] x I).
 *
 * Build: see oracle/Makefile.  The canonical build uses -ffp-contract=off so
 * every `acc = acc + a*b` is a rounded multiply followed by a rounded add, as
 * the WGSL text reads.  The *_fma variants use fmaf() explicitly: WGSL leaves
 * contraction to the driver, so the spread between the two is the reference's
 * own last-bit ambiguity.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------------------
 * matmul_tiled  (rusty-backend/src/kernels.wgsl:16-54; host dims lib.rs:4410-4412)
 * out[r,c] = sum_k a[r,k] * b[k,c];  a [M,K], b [K,N], out [M,N], row-major f32.
 * The shader walks k in tiles of 16 but each output's accumulator still sees
 * k = 0,1,2,... in ascending order, starting from 0.0; padded tail elements
 * contribute +0.0*0.0 which never changes the accumulator's value.
 * ------------------------------------------------------------------------- */
ORACLE_API void oracle_matmul_tiled(const float* a, const float* b, float* out,
                                    uint32_t M, uint32_t K, uint32_t N) {
    for (uint32_t r = 0; r < M; ++r)
        for (uint32_t c = 0; c < N; ++c) {
            float acc = 0.0f;
            for (uint32_t k = 0; k < K; ++k) acc = acc + a[(size_t)r * K + k] * b[(size_t)k * N + c];
            out[(size_t)r * N + c] = acc;
        }
}

ORACLE_API void oracle_matmul_tiled_fma(const float* a, const float* b, float* out,
                                        uint32_t M, uint32_t K, uint32_t N) {
    for (uint32_t r = 0; r < M; ++r)
        for (uint32_t c = 0; c < N; ++c) {
            float acc = 0.0f;
            for (uint32_t k = 0; k < K; ++k) acc = fmaf(a[(size_t)r * K + k], b[(size_t)k * N + c], acc);
            out[(size_t)r * N + c] = acc;
        }
}

/* ---------------------------------------------------------------------------
 * matmul_bt  (rusty-backend/src/kernels.wgsl:234-242; host dims lib.rs:4306-4308)
 * out[r,c] = sum_k a[r,k] * b[c,k];  a [M,K], b [N,K] (weights as [out,in]).
 * ------------------------------------------------------------------------- */
ORACLE_API void oracle_matmul_bt(const float* a, const float* b, float* out,
                                 uint32_t M, uint32_t K, uint32_t N) {
    for (uint32_t r = 0; r < M; ++r)
        for (uint32_t c = 0; c < N; ++c) {
            float acc = 0.0f;
            const float* ar = a + (size_t)r * K;
            const float* bc = b + (size_t)c * K;
            for (uint32_t k = 0; k < K; ++k) acc = acc + ar[k] * bc[k];
            out[(size_t)r * N + c] = acc;
        }
}

ORACLE_API void oracle_matmul_bt_fma(const float* a, const float* b, float* out,
                                     uint32_t M, uint32_t K, uint32_t N) {
    for (uint32_t r = 0; r < M; ++r)
        for (uint32_t c = 0; c < N; ++c) {
            float acc = 0.0f;
            const float* ar = a + (size_t)r * K;
            const float* bc = b + (size_t)c * K;
            for (uint32_t k = 0; k < K; ++k) acc = fmaf(ar[k], bc[k], acc);
            out[(size_t)r * N + c] = acc;
        }
}

/* ---------------------------------------------------------------------------
 * dequantize  (rusty-backend/src/kernels.wgsl:156-166; dispatch lib.rs:4872-4899)
 * The input buffer is viewed as little-endian u32 words.  Word i yields four
 * UNSIGNED bytes, least-significant first, each converted with f32(); there is
 * no scale and no zero point.  Threads are dispatched for ceil(n_in/4) words
 * rounded up to a multiple of 64; a thread returns if its word index is
 * outside the input array and guards each of its four stores by the output
 * length.  `in_words` is arrayLength(&deq_in), `n_in` is the product of the
 * input tensor's shape (what the host sizes the dispatch from), `n_out` is
 * arrayLength(&deq_out).
 * ------------------------------------------------------------------------- */
ORACLE_API void oracle_dequantize(const uint32_t* in, size_t in_words, size_t n_in,
                                  float* out, size_t n_out) {
    size_t u32_elements = (n_in + 3) / 4;
    size_t threads = ((u32_elements + 63) / 64) * 64;
    for (size_t i = 0; i < threads; ++i) {
        size_t base = i * 4;
        if (i >= in_words) continue;
        uint32_t p = in[i];
        if (base < n_out) out[base] = (float)(p & 0xFFu);
        if (base + 1 < n_out) out[base + 1] = (float)((p >> 8) & 0xFFu);
        if (base + 2 < n_out) out[base + 2] = (float)((p >> 16) & 0xFFu);
        if (base + 3 < n_out) out[base + 3] = (float)((p >> 24) & 0xFFu);
    }
}

/* ---------------------------------------------------------------------------
 * affine_dequantize  (rusty-backend/src/kernels.wgsl:385-400)
 * out[i] = f32(byte i of the weight buffer) * scales[i/64] + biases[i/64],
 * i the flat row-major element index, group size fixed at 64.  One rounded
 * multiply then one rounded add in the canonical build.
 * This is the INTENDED semantics: every element i < n is written.
 * ------------------------------------------------------------------------- */
static inline float affine_one(const uint32_t* w, const float* scales, const float* biases, size_t i) {
    size_t u32_idx = i / 4;
    uint32_t byte_inner = (uint32_t)(i % 4);
    uint32_t val_u32 = w[u32_idx];
    float val_u8 = (float)((val_u32 >> (byte_inner * 8u)) & 0xFFu);
    size_t group_idx = i / 64;
    return val_u8 * scales[group_idx] + biases[group_idx];
}

ORACLE_API void oracle_affine_dequantize(const uint32_t* w, const float* scales, const float* biases,
                                         float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = affine_one(w, scales, biases, i);
}

ORACLE_API void oracle_affine_dequantize_fma(const uint32_t* w, const float* scales, const float* biases,
                                             float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        uint32_t v = (w[i / 4] >> ((uint32_t)(i % 4) * 8u)) & 0xFFu;
        out[i] = fmaf((float)v, scales[i / 64], biases[i / 64]);
    }
}

/* affine_dequantize exactly AS DISPATCHED by the reference host code
 * (rusty-backend/src/lib.rs:4976-4987): above 65 535 workgroups the host
 * launches a 2-D grid but the shader indexes by global_id.x alone
 * (kernels.wgsl:387), so only elements below 65 535*64 = 4 194 240 are ever
 * written; the rest of `out` is left untouched.  Kept to document that defect;
 * the CUDA path implements the intended semantics above. */
ORACLE_API void oracle_affine_dequantize_as_dispatched(const uint32_t* w, const float* scales,
                                                       const float* biases, float* out, size_t n) {
    size_t workgroups = (n + 63) / 64;
    size_t x_threads = (workgroups <= 65535 ? workgroups : 65535) * 64;
    for (size_t i = 0; i < x_threads && i < n; ++i) out[i] = affine_one(w, scales, biases, i);
}

/* ---------------------------------------------------------------------------
 * Compositions.  The reference dequantises once at load
 * (rusty-loader/src/lib.rs:155-218) and runs an f32 matmul per Linear::forward
 * (rusty-graph/src/lib.rs:69-70).  `layout_nk` != 0: weight stored [N,K]
 * ([out,in], contraction of matmul_bt); 0: stored [K,N] ([in,out], contraction
 * of matmul_tiled).  `wf` is caller-provided scratch of N*K floats.
 * ------------------------------------------------------------------------- */

/* Mode A: u8 affine, group-64 over the flat index. */
ORACLE_API void oracle_qlinear_affine(const float* x, const uint32_t* w_u8, const float* scales,
                                      const float* biases, float* wf, float* y,
                                      uint32_t M, uint32_t K, uint32_t N, int layout_nk) {
    oracle_affine_dequantize(w_u8, scales, biases, wf, (size_t)N * K);
    if (layout_nk) oracle_matmul_bt(x, wf, y, M, K, N);
    else oracle_matmul_tiled(x, wf, y, M, K, N);
}

/* Mode B: signed int8, one f32 scale per output feature.  Bytes are unpacked
 * in the dequantize shader's lane order (kernels.wgsl:161-165) and then
 * sign-extended; W_f32[n,k] = f32(q[n,k]) * scale[n]. */
ORACLE_API void oracle_dequantize_rowscale(const int8_t* q, const float* scale, float* wf,
                                           uint32_t K, uint32_t N, int layout_nk) {
    if (layout_nk) {
        for (uint32_t n = 0; n < N; ++n)
            for (uint32_t k = 0; k < K; ++k) wf[(size_t)n * K + k] = (float)q[(size_t)n * K + k] * scale[n];
    } else {
        for (uint32_t k = 0; k < K; ++k)
            for (uint32_t n = 0; n < N; ++n) wf[(size_t)k * N + n] = (float)q[(size_t)k * N + n] * scale[n];
    }
}

ORACLE_API void oracle_qlinear_rowscale(const float* x, const int8_t* q, const float* scale, float* wf,
                                        float* y, uint32_t M, uint32_t K, uint32_t N, int layout_nk) {
    oracle_dequantize_rowscale(q, scale, wf, K, N, layout_nk);
    if (layout_nk) oracle_matmul_bt(x, wf, y, M, K, N);
    else oracle_matmul_tiled(x, wf, y, M, K, N);
}

/* ---------------------------------------------------------------------------
 * Threaded variants, used only to TIME the CPU baseline (same arithmetic as
 * above, rows spread over host threads; the per-output summation order is
 * unchanged so results are bit-identical to the scalar versions).
 * ------------------------------------------------------------------------- */
/* Fix the thread count of the threaded variants explicitly (a launcher may have exported OMP_NUM_THREADS=1). */
ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Reference-faithful step: f32 x pre-dequantised f32 weight [N,K]. */
ORACLE_API void oracle_matmul_bt_mt(const float* a, const float* b, float* out,
                                    uint32_t M, uint32_t K, uint32_t N) {
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < (int64_t)N; ++c) {
        const float* bc = b + (size_t)c * K;
        for (uint32_t r = 0; r < M; ++r) {
            const float* ar = a + (size_t)r * K;
            float acc = 0.0f;
            for (uint32_t k = 0; k < K; ++k) acc = acc + ar[k] * bc[k];
            out[(size_t)r * N + c] = acc;
        }
    }
}

/* Fused CPU form: int8 read and per-row-scale dequant inside the dot product
 * (the same data movement the CUDA kernels perform). */
ORACLE_API void oracle_qlinear_rowscale_fused_mt(const float* x, const int8_t* q, const float* scale,
                                                 float* y, uint32_t M, uint32_t K, uint32_t N) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < (int64_t)N; ++n) {
        const int8_t* qn = q + (size_t)n * K;
        float s = scale[n];
        for (uint32_t r = 0; r < M; ++r) {
            const float* xr = x + (size_t)r * K;
            float acc = 0.0f;
            for (uint32_t k = 0; k < K; ++k) acc = acc + xr[k] * ((float)qn[k] * s);
            y[(size_t)r * N + n] = acc;
        }
    }
}

ORACLE_API void oracle_affine_dequantize_mt(const uint32_t* w, const float* scales, const float* biases,
                                            float* out, size_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = affine_one(w, scales, biases, (size_t)i);
}

/* float64 dot products (exact products, double accumulate) used by the tests
 * to bound how far BOTH the oracle and the CUDA kernels sit from the true sum. */
ORACLE_API void oracle_matmul_bt_f64(const float* a, const float* b, double* out,
                                     uint32_t M, uint32_t K, uint32_t N) {
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < (int64_t)N; ++c) {
        const float* bc = b + (size_t)c * K;
        for (uint32_t r = 0; r < M; ++r) {
            const float* ar = a + (size_t)r * K;
            double acc = 0.0;
            for (uint32_t k = 0; k < K; ++k) acc += (double)ar[k] * (double)bc[k];
            out[(size_t)r * N + c] = acc;
        }
    }
}

/* Vectorised timing variants: the same products, but each output's sum is
 * split over SIMD lanes (order differs from the shader's, so these are NOT
 * used for parity, only as the strongest CPU number the baseline can report). */
ORACLE_API void oracle_matmul_bt_mt_simd(const float* a, const float* b, float* out,
                                         uint32_t M, uint32_t K, uint32_t N) {
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < (int64_t)N; ++c) {
        const float* bc = b + (size_t)c * K;
        for (uint32_t r = 0; r < M; ++r) {
            const float* ar = a + (size_t)r * K;
            float acc = 0.0f;
#pragma omp simd reduction(+ : acc)
            for (uint32_t k = 0; k < K; ++k) acc += ar[k] * bc[k];
            out[(size_t)r * N + c] = acc;
        }
    }
}

ORACLE_API void oracle_qlinear_rowscale_fused_mt_simd(const float* x, const int8_t* q, const float* scale,
                                                      float* y, uint32_t M, uint32_t K, uint32_t N) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < (int64_t)N; ++n) {
        const int8_t* qn = q + (size_t)n * K;
        float s = scale[n];
        for (uint32_t r = 0; r < M; ++r) {
            const float* xr = x + (size_t)r * K;
            float acc = 0.0f;
#pragma omp simd reduction(+ : acc)
            for (uint32_t k = 0; k < K; ++k) acc += xr[k] * (float)qn[k];
            y[(size_t)r * N + n] = acc * s;
        }
    }
}

/* ---- SwiGLU glue of the MLP (the step between gate|up and down) ------------
 * WGSL `silu` (rusty-backend/src/kernels.wgsl:104-113): out = x * (1.0 / (1.0 + exp(-x))).
 * WGSL `mul`  (kernels.wgsl:146-151): out = a * b.
 * MLP::forward (rusty-graph/src/lib.rs:317-323) applies SiLU to the GATE projection and multiplies by UP
 * (the unused `silu_gate_fused` shader, kernels.wgsl:527-542, applies it to `up`; MLP::forward is followed).
 * exp is libm's expf here; WGSL leaves its accuracy to the driver, so results are compared with a tolerance. */
ORACLE_API void oracle_silu(const float* x, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = x[i] * (1.0f / (1.0f + expf(-x[i])));
}

ORACLE_API void oracle_mul(const float* a, const float* b, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = a[i] * b[i];
}

/* s is [M, 2F] with gate_j in column 2j and up_j in column 2j+1 (the row order of a pair-interleaved gate|up
 * weight); out[M, F] = silu(gate) * up, composed from the two shaders above. */
ORACLE_API void oracle_swiglu_pairs(const float* s, float* out, uint32_t M, uint32_t F) {
    for (uint32_t m = 0; m < M; ++m)
        for (uint32_t j = 0; j < F; ++j) {
            float g = s[(size_t)m * 2 * F + 2 * j], u = s[(size_t)m * 2 * F + 2 * j + 1], act;
            oracle_silu(&g, &act, 1);
            oracle_mul(&act, &u, &out[(size_t)m * F + j], 1);
        }
}

/* ---- the steps in front of a layer's Linears -------------------------------
 * WGSL `rms_norm` (rusty-backend/src/kernels.wgsl:87-102), the body the shader runs for row 0, applied to one row:
 *   ss = 0; for i: ss = ss + x[i]*x[i];  ss = ss / f32(size);  inv_rms = 1.0 / sqrt(ss + 1e-5);
 *   out[i] = x[i] * inv_rms * weight[i]
 * and WGSL `rms_norm_residual` (kernels.wgsl:579-597): the same over val = x[i] + residual[i].  Sequential f32
 * accumulation in index order, as the shader text reads (canonical build: no contraction).  eps is a parameter;
 * the shaders hard-code 1e-5.  residual and sum_out may be NULL; sum_out receives x + residual. */
ORACLE_API void oracle_rms_norm_row(const float* x, const float* residual, const float* weight, float* out, float* sum_out,
                                    uint32_t size, float eps) {
    float ss = 0.0f;
    for (uint32_t i = 0; i < size; ++i) {
        float val = residual ? x[i] + residual[i] : x[i];
        if (sum_out) sum_out[i] = val;
        out[i] = val; /* temp store, like the residual shader */
        ss = ss + val * val;
    }
    ss = ss / (float)size;
    float inv_rms = 1.0f / sqrtf(ss + eps);
    for (uint32_t i = 0; i < size; ++i) out[i] = out[i] * inv_rms * weight[i];
}

/* Every row of x[M, K] on its own: what RMSNorm::forward (rusty-graph/src/lib.rs:148-170) means to compute; the
 * shader as written stops after row 0. */
ORACLE_API void oracle_rms_norm_rows(const float* x, const float* residual, const float* weight, float* out, float* sum_out,
                                     uint32_t M, uint32_t K, float eps) {
    for (uint32_t m = 0; m < M; ++m)
        oracle_rms_norm_row(x + (size_t)m * K, residual ? residual + (size_t)m * K : NULL, weight, out + (size_t)m * K,
                            sum_out ? sum_out + (size_t)m * K : NULL, K, eps);
}

/* Embedding::forward (rusty-graph/src/lib.rs:121-135): out[t, :] = table[ids[t], :].  Returns the number of ids
 * outside the table (the reference panics on the first; their rows are zeroed here). */
ORACLE_API uint32_t oracle_embedding(const float* table, const uint32_t* ids, float* out, size_t n_ids, uint32_t vocab, uint32_t dim) {
    uint32_t bad = 0;
    for (size_t t = 0; t < n_ids; ++t) {
        if (ids[t] < vocab) {
            memcpy(out + t * dim, table + (size_t)ids[t] * dim, (size_t)dim * sizeof(float));
        } else {
            memset(out + t * dim, 0, (size_t)dim * sizeof(float));
            ++bad;
        }
    }
    return bad;
}

/* ---- the step after the LM head -------------------------------------------
 * Greedy sampling (rusty-loader/src/tokenizer.rs:151-158, temperature <= 0): the index of the maximum logit;
 * Iterator::max_by keeps the LAST of several equal maxima; an empty slice gives 0.  (partial_cmp().unwrap()
 * panics on NaN there; NaN is skipped here.) */
ORACLE_API uint32_t oracle_greedy_sample(const float* logits, size_t n) {
    uint32_t best = 0;
    int have = 0;
    float bv = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float v = logits[i];
        if (v != v) continue;
        if (!have || v >= bv) {
            bv = v;
            best = (uint32_t)i;
            have = 1;
        }
    }
    return best;
}

/* WGSL `top_k` (rusty-backend/src/kernels.wgsl:168-188): k rounds of "first index of the largest value not taken
 * yet", starting each round from max_v = -1e9 and max_idx = 0 with a strict `>`. */
ORACLE_API void oracle_top_k(const float* in, size_t len, uint32_t k, uint32_t* out_idx) {
    for (uint32_t i = 0; i < k; ++i) {
        float max_v = -1e9f;
        uint32_t max_idx = 0;
        for (size_t j = 0; j < len; ++j) {
            float v = in[j];
            int used = 0;
            for (uint32_t p = 0; p < i; ++p)
                if (out_idx[p] == (uint32_t)j) {
                    used = 1;
                    break;
                }
            if (!used && v > max_v) {
                max_v = v;
                max_idx = (uint32_t)j;
            }
        }
        out_idx[i] = max_idx;
    }
}
