/*
 * t0_oracle.c -- CPU restatement of the T0-GPU reference math for the bf16 GEMM hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker: the GPU library is compared against it.
 * Nothing in the product path (the CUDA library, the Python package) may call it; only the tests,
 * the smoke check and the CPU-baseline leg of the benchmark do.
 *
 * Parity status: PINNED.  The reference is Rust and cannot be compiled in this environment, so
 * every function restates a reference function (cited below, paths relative to the reference
 * project root) and the restatement is checked against the reference's own golden vectors
 * (benchmarks/torch_ref/*.bin, a torch-generated fixture that src/t0/precision_vs_torch.rs
 * consumes) and against every closed-form known-answer test the reference's unit tests hold.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -shared -fPIC (see oracle/build.py).
 * -ffp-contract=off matters: the reference accumulates `acc += a * b` as a separate f32 multiply
 * and f32 add (Rust never fuses), and bit-identical oracle output depends on that.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define T0O_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------------------------------------
 * bf16 helpers
 * ------------------------------------------------------------------------------------------- */

static inline float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

/* Round-to-nearest-even f32 -> bf16.  examples/test_gemm_correctness.rs:15-20 and
 * src/ignis/ops/bf16_matmul.rs:371-374: ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16). */
T0O_API uint16_t t0o_f32_to_bf16_rne(float x) {
    uint32_t bits = f32_bits(x);
    uint32_t round = ((bits >> 16) & 1u) + 0x7FFFu;
    return (uint16_t)((bits + round) >> 16);
}

/* Truncating f32 -> bf16.  src/t0/tile_ir.rs:3205-3207, src/t0/test_tile_gemm_suite.rs:22. */
T0O_API uint16_t t0o_f32_to_bf16_trunc(float x) { return (uint16_t)(f32_bits(x) >> 16); }

/* bf16 -> f32 widen.  examples/test_gemm_correctness.rs:22-24. */
T0O_API float t0o_bf16_to_f32(uint16_t x) { return bits_f32((uint32_t)x << 16); }

T0O_API void t0o_f32_to_bf16_rne_array(const float *src, uint16_t *dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = t0o_f32_to_bf16_rne(src[i]);
}

T0O_API void t0o_bf16_to_f32_array(const uint16_t *src, float *dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = t0o_bf16_to_f32(src[i]);
}

/* ---------------------------------------------------------------------------------------------
 * Seeded input generators (they pin the data of every parity run)
 * ------------------------------------------------------------------------------------------- */

/* xorshift64 -> uniform[-1,1] -> RNE bf16.  examples/test_gemm_correctness.rs:45-58.
 * The reference computes ((state >> 32) as f32 / u32::MAX as f32) * 2.0 - 1.0 entirely in f32. */
T0O_API void t0o_rand_bf16(uint16_t *out, size_t n, uint64_t seed) {
    uint64_t state = seed ^ 0xDEADBEEFCAFEBABEull;
    const float denom = (float)UINT32_MAX;
    for (size_t i = 0; i < n; ++i) {
        state ^= state << 13;
        state ^= state >> 7;
        state ^= state << 17;
        float f = ((float)(state >> 32) / denom) * 2.0f - 1.0f;
        out[i] = t0o_f32_to_bf16_rne(f);
    }
}

/* LCG -> {-1.00 .. 0.99} step 0.01 -> truncated bf16.  src/t0/test_tile_gemm_suite.rs:17-24. */
T0O_API void t0o_lcg_bf16(uint16_t *out, size_t n, uint64_t seed) {
    uint64_t s = seed;
    for (size_t i = 0; i < n; ++i) {
        s = s * 6364136223846793005ull + 1ull;
        float f = ((float)((uint32_t)(s >> 33) % 200u) - 100.0f) * 0.01f;
        out[i] = t0o_f32_to_bf16_trunc(f);
    }
}

/* Periodic pattern ((i % period) - offset) * 0.01 -> truncated bf16.  src/t0/tile_ir.rs:3542-3543
 * uses (17, 8) for X and (13, 6) for W. */
T0O_API void t0o_periodic_bf16(uint16_t *out, size_t n, uint32_t period, int32_t offset) {
    for (size_t i = 0; i < n; ++i) {
        float f = ((float)(i % period) - (float)offset) * 0.01f;
        out[i] = t0o_f32_to_bf16_trunc(f);
    }
}

/* ---------------------------------------------------------------------------------------------
 * GEMM (bf16 in, f32 accumulate, f32 out)
 *
 * All variants share one loop nest: for i, for j, acc = 0; for kk ascending: acc += a * b, with a
 * separate f32 multiply and add.  examples/test_gemm_correctness.rs:28-42 is the NT form; the
 * identical copies are src/t0/tile_ir.rs:3511-3528, src/t0/test_tile_gemm_suite.rs:26-35 and
 * src/t0/tile_boundary_tests.rs:27-39.  trans_a / trans_b select how an element is addressed:
 *   trans_a = 0: A[i, kk] at a[i * lda + kk]      (A stored [M, K])
 *   trans_a = 1: A[i, kk] at a[kk * lda + i]      (A stored [K, M])
 *   trans_b = 0: B[kk, j] at b[kk * ldb + j]      (B stored [K, N]  -- "NN")
 *   trans_b = 1: B[kk, j] at b[j * ldb + kk]      (B stored [N, K]  -- "NT", the reference default)
 * Backward forms: examples/test_gemm_backward.rs:44-77 (cpu_backward_data is trans_a=0,trans_b=0;
 * cpu_backward_weight is trans_a=1,trans_b=0).
 * ------------------------------------------------------------------------------------------- */

typedef struct {
    const uint16_t *a, *b;
    float *c;
    int64_t m, n, k, lda, ldb, ldc;
    int trans_a, trans_b;
    int64_t row_begin, row_end;
} gemm_job_t;

static void gemm_rows(const gemm_job_t *g) {
    const int64_t n = g->n, k = g->k;
    /* Widen one operand row/column at a time so the inner loop is pure f32; the order of the
     * floating-point operations per output element is unchanged (kk ascending, mul then add). */
    float *arow = (float *)malloc((size_t)k * sizeof(float));
    float *bcol = (float *)malloc((size_t)k * sizeof(float));
    for (int64_t i = g->row_begin; i < g->row_end; ++i) {
        for (int64_t kk = 0; kk < k; ++kk) {
            uint16_t av = g->trans_a ? g->a[kk * g->lda + i] : g->a[i * g->lda + kk];
            arow[kk] = t0o_bf16_to_f32(av);
        }
        for (int64_t j = 0; j < n; ++j) {
            float acc = 0.0f;
            if (g->trans_b) {
                const uint16_t *bp = g->b + j * g->ldb;
                for (int64_t kk = 0; kk < k; ++kk) {
                    float prod = arow[kk] * t0o_bf16_to_f32(bp[kk]);
                    acc = acc + prod;
                }
            } else {
                for (int64_t kk = 0; kk < k; ++kk) bcol[kk] = t0o_bf16_to_f32(g->b[kk * g->ldb + j]);
                for (int64_t kk = 0; kk < k; ++kk) {
                    float prod = arow[kk] * bcol[kk];
                    acc = acc + prod;
                }
            }
            g->c[i * g->ldc + j] = acc;
        }
    }
    free(arow);
    free(bcol);
}

static void *gemm_thread(void *p) { gemm_rows((const gemm_job_t *)p); return NULL; }

/* Row-parallel driver.  Splitting output rows over threads leaves every element's summation order
 * untouched, so the result is bit-identical for any thread count.  rows [row_begin, row_end) only
 * (used to time a bounded slice of a large problem). */
T0O_API void t0o_gemm_bf16(const uint16_t *a, const uint16_t *b, float *c, int64_t m, int64_t n, int64_t k,
                           int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b,
                           int64_t row_begin, int64_t row_end, int threads) {
    if (row_end > m) row_end = m;
    if (row_begin < 0) row_begin = 0;
    int64_t rows = row_end - row_begin;
    if (rows <= 0) return;
    if (threads < 1) threads = 1;
    if (threads > rows) threads = (int)rows;
    if (threads > 256) threads = 256;
    gemm_job_t jobs[256];
    pthread_t tids[256];
    for (int t = 0; t < threads; ++t) {
        gemm_job_t g = {a, b, c, m, n, k, lda, ldb, ldc, trans_a, trans_b,
                        row_begin + rows * t / threads, row_begin + rows * (t + 1) / threads};
        jobs[t] = g;
    }
    if (threads == 1) { gemm_rows(&jobs[0]); return; }
    for (int t = 0; t < threads; ++t) pthread_create(&tids[t], NULL, gemm_thread, &jobs[t]);
    for (int t = 0; t < threads; ++t) pthread_join(tids[t], NULL);
}

/* Split-K slab reduce: y[i] = sum over s = 0..sk-1 (in that order) of partials[s * total + i],
 * starting from 0.0.  examples/test_gemm_correctness.rs:190-207. */
T0O_API void t0o_splitk_reduce(const float *partials, float *y, size_t total, int sk) {
    for (size_t i = 0; i < total; ++i) y[i] = 0.0f;
    for (int s = 0; s < sk; ++s)
        for (size_t i = 0; i < total; ++i) y[i] = y[i] + partials[(size_t)s * total + i];
}

/* GEMM over a K range [k_begin, k_end) -- one split-K slab as the reference kernel writes it
 * (src/t0/gemm_gen.rs:746-752: slab id covers a contiguous K chunk of K / split_k). NT only. */
T0O_API void t0o_gemm_bf16_nt_krange(const uint16_t *x, const uint16_t *wt, float *y, int64_t m, int64_t n,
                                     int64_t k, int64_t k_begin, int64_t k_end) {
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            float acc = 0.0f;
            for (int64_t kk = k_begin; kk < k_end; ++kk) {
                float prod = t0o_bf16_to_f32(x[i * k + kk]) * t0o_bf16_to_f32(wt[j * k + kk]);
                acc = acc + prod;
            }
            y[i * n + j] = acc;
        }
}

/* bf16 transpose A[rows, cols] -> At[cols, rows].  examples/test_gemm_backward.rs:79-88. */
T0O_API void t0o_transpose_bf16(const uint16_t *a, uint16_t *out, int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) out[c * rows + r] = a[r * cols + c];
}

/* Fused store-phase epilogues of the generator: bias add, bias add + ReLU
 * (src/t0/gemm_gen.rs:40-49, 1280-1334).  bias is f32[N], broadcast over rows. */
T0O_API void t0o_epilogue_bias(float *y, const float *bias, int64_t m, int64_t n, int64_t ldc, int relu) {
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            float v = y[i * ldc + j] + bias[j];
            if (relu) v = v > 0.0f ? v : 0.0f;
            y[i * ldc + j] = v;
        }
}

/* ---------------------------------------------------------------------------------------------
 * RMSNorm.  src/t0/rmsnorm_kernels.rs:140-174 (forward; backward dX).
 * ------------------------------------------------------------------------------------------- */

T0O_API void t0o_rmsnorm_forward(const float *input, const float *weight, float *output, float *inv_rms_out,
                                 int64_t rows, int64_t cols, float eps) {
    for (int64_t r = 0; r < rows; ++r) {
        const float *row = input + r * cols;
        float *out = output + r * cols;
        float sum = 0.0f;
        for (int64_t c = 0; c < cols; ++c) sum = sum + row[c] * row[c];
        float mean_sq = sum / (float)cols;
        float rstd = 1.0f / sqrtf(mean_sq + eps);
        if (inv_rms_out) inv_rms_out[r] = rstd;
        for (int64_t c = 0; c < cols; ++c) out[c] = row[c] * rstd * weight[c];
    }
}

T0O_API void t0o_rmsnorm_backward(const float *dy, const float *x, const float *weight, float *dx,
                                  int64_t rows, int64_t cols, float eps) {
    float *dx_hat = (float *)malloc((size_t)cols * sizeof(float));
    for (int64_t r = 0; r < rows; ++r) {
        const float *dy_row = dy + r * cols;
        const float *x_row = x + r * cols;
        float *dx_row = dx + r * cols;
        float sum = 0.0f;
        for (int64_t c = 0; c < cols; ++c) sum = sum + x_row[c] * x_row[c];
        float mean_sq = sum / (float)cols;
        float rstd = 1.0f / sqrtf(mean_sq + eps);
        for (int64_t c = 0; c < cols; ++c) dx_hat[c] = dy_row[c] * weight[c];
        float dot = 0.0f;
        for (int64_t c = 0; c < cols; ++c) dot = dot + x_row[c] * dx_hat[c];
        float dot_val = dot / (float)cols;
        for (int64_t c = 0; c < cols; ++c) dx_row[c] = rstd * (dx_hat[c] - x_row[c] * rstd * rstd * dot_val);
    }
    free(dx_hat);
}

/* dgamma[c] = sum over rows (ascending) of dy[r,c] * x[r,c] * inv_rms[r].
 * src/ignis/ops/rmsnorm.rs:239-293 accumulates the same terms with unordered global atomics; the
 * oracle fixes the order to row-ascending. */
T0O_API void t0o_rmsnorm_dgamma(const float *dy, const float *x, float *dgamma, int64_t rows, int64_t cols,
                                float eps) {
    for (int64_t c = 0; c < cols; ++c) dgamma[c] = 0.0f;
    for (int64_t r = 0; r < rows; ++r) {
        const float *x_row = x + r * cols;
        float sum = 0.0f;
        for (int64_t c = 0; c < cols; ++c) sum = sum + x_row[c] * x_row[c];
        float rstd = 1.0f / sqrtf(sum / (float)cols + eps);
        for (int64_t c = 0; c < cols; ++c) dgamma[c] = dgamma[c] + dy[r * cols + c] * x_row[c] * rstd;
    }
}

/* ---------------------------------------------------------------------------------------------
 * Softmax.  src/t0/softmax_kernels.rs:123-146.
 * ------------------------------------------------------------------------------------------- */

T0O_API void t0o_softmax_forward(const float *input, float *output, int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        const float *row = input + r * cols;
        float *out = output + r * cols;
        float max_val = -INFINITY;
        for (int64_t c = 0; c < cols; ++c) max_val = row[c] > max_val ? row[c] : max_val;
        float exp_sum = 0.0f;
        for (int64_t c = 0; c < cols; ++c) exp_sum = exp_sum + expf(row[c] - max_val);
        for (int64_t c = 0; c < cols; ++c) out[c] = expf(row[c] - max_val) / exp_sum;
    }
}

T0O_API void t0o_softmax_backward(const float *dy, const float *y, float *dx, int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        const float *dy_row = dy + r * cols;
        const float *y_row = y + r * cols;
        float *dx_row = dx + r * cols;
        float dot = 0.0f;
        for (int64_t c = 0; c < cols; ++c) dot = dot + dy_row[c] * y_row[c];
        for (int64_t c = 0; c < cols; ++c) dx_row[c] = y_row[c] * (dy_row[c] - dot);
    }
}

/* ---------------------------------------------------------------------------------------------
 * Cross-entropy.  src/t0/ce_loss_kernels.rs:166-192.
 * ------------------------------------------------------------------------------------------- */

T0O_API void t0o_ce_loss_forward(const float *logits, const uint32_t *targets, float *losses, int64_t rows,
                                 int64_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        const float *row = logits + r * cols;
        int64_t target = targets[r];
        float max_val = -INFINITY;
        for (int64_t c = 0; c < cols; ++c) max_val = row[c] > max_val ? row[c] : max_val;
        float exp_sum = 0.0f;
        for (int64_t c = 0; c < cols; ++c) exp_sum = exp_sum + expf(row[c] - max_val);
        losses[r] = logf(exp_sum) + max_val - row[target];
    }
}

T0O_API void t0o_ce_loss_backward(const float *logits, const uint32_t *targets, float *dlogits, int64_t rows,
                                  int64_t cols, float scale) {
    for (int64_t r = 0; r < rows; ++r) {
        const float *row = logits + r * cols;
        int64_t target = targets[r];
        float max_val = -INFINITY;
        for (int64_t c = 0; c < cols; ++c) max_val = row[c] > max_val ? row[c] : max_val;
        float exp_sum = 0.0f;
        for (int64_t c = 0; c < cols; ++c) exp_sum = exp_sum + expf(row[c] - max_val);
        for (int64_t c = 0; c < cols; ++c) {
            float softmax_val = expf(row[c] - max_val) / exp_sum;
            float one_hot = (c == target) ? 1.0f : 0.0f;
            dlogits[r * cols + c] = (softmax_val - one_hot) * scale;
        }
    }
}

/* Mean loss the way the Ignis op forms it from probabilities: -mean(ln(max(p[target], 1e-10))).
 * src/ignis/ops/cross_entropy.rs:70-78; the raw-ISA kernel clamps the same way
 * (examples/kernels/softmax_ce_loss.rs:253-263). */
T0O_API float t0o_ce_mean_loss_from_probs(const float *probs, const uint32_t *targets, int64_t rows, int64_t cols) {
    float total = 0.0f;
    for (int64_t b = 0; b < rows; ++b) {
        int64_t t = targets[b];
        if (t < cols) {
            float p = probs[b * cols + t];
            p = p > 1e-10f ? p : 1e-10f;
            total = total + (-logf(p));
        }
    }
    return total / (float)rows;
}

/* ---------------------------------------------------------------------------------------------
 * SiLU gate (src/ignis/ops/silu.rs:32-152): out = silu(gate) * up; backward formulas at :118-130.
 * ------------------------------------------------------------------------------------------- */

T0O_API void t0o_silu_gate_forward(const float *gate, const float *up, float *out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float sig = 1.0f / (1.0f + expf(-gate[i]));
        out[i] = gate[i] * sig * up[i];
    }
}

T0O_API void t0o_silu_gate_backward(const float *grad, const float *gate, const float *up, float *dgate, float *dup,
                                    size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float sig = 1.0f / (1.0f + expf(-gate[i]));
        float silu = gate[i] * sig;
        dup[i] = grad[i] * silu;
        dgate[i] = grad[i] * up[i] * sig * (1.0f + gate[i] * (1.0f - sig));
    }
}

/* ---------------------------------------------------------------------------------------------
 * Elementwise neighbours of the GEMMs in the training step.
 * ------------------------------------------------------------------------------------------- */

/* y += x.  src/ignis/tape.rs:343-367, src/t0/elementwise_kernels.rs:41-61. */
T0O_API void t0o_residual_add(float *y, const float *x, size_t n) {
    for (size_t i = 0; i < n; ++i) y[i] = y[i] + x[i];
}

/* Embedding lookup: output[t, :] = table[indices[t], :].  src/t0/embedding_kernels.rs:100-110. */
T0O_API void t0o_embedding_forward(const float *table, const uint32_t *indices, float *output, size_t num_tokens,
                                   size_t dim) {
    for (size_t t = 0; t < num_tokens; ++t) {
        size_t idx = indices[t];
        for (size_t d = 0; d < dim; ++d) output[t * dim + d] = table[idx * dim + d];
    }
}

/* Embedding gradient: grad_table[indices[t], :] += grad_output[t, :], tokens in ascending order.
 * src/t0/embedding_kernels.rs:113-124. */
T0O_API void t0o_embedding_backward(float *grad_table, const uint32_t *indices, const float *grad_output,
                                    size_t num_tokens, size_t dim) {
    for (size_t t = 0; t < num_tokens; ++t) {
        size_t idx = indices[t];
        for (size_t d = 0; d < dim; ++d) grad_table[idx * dim + d] = grad_table[idx * dim + d] + grad_output[t * dim + d];
    }
}

/* Fused AdamW step.  src/t0/adamw_kernels.rs:105-119. */
T0O_API void t0o_adamw_step(float *params, const float *grads, float *m, float *v, size_t n, float lr, float beta1,
                            float beta2, float eps, float weight_decay, uint32_t t) {
    float bc1 = 1.0f / (1.0f - powf(beta1, (float)t));
    float bc2 = 1.0f / (1.0f - powf(beta2, (float)t));
    for (size_t i = 0; i < n; ++i) {
        m[i] = beta1 * m[i] + (1.0f - beta1) * grads[i];
        v[i] = beta2 * v[i] + (1.0f - beta2) * grads[i] * grads[i];
        float m_hat = m[i] * bc1;
        float v_hat = v[i] * bc2;
        params[i] = params[i] * (1.0f - lr * weight_decay) - lr * m_hat / (sqrtf(v_hat) + eps);
    }
}
