/*
 * CPU oracle: a plain-C restatement of Tempest.jl's reference CPU path for the
 * fused-kernel hot path.  TEST INFRASTRUCTURE ONLY: the tests, the smoke check
 * and the benchmark's CPU-baseline leg link this file; the product never does.
 *
 * Parity pinning: the reference is Julia and cannot run where this file is
 * built, and its tests hold no stored tensors.  The restatement is pinned on
 * the known-answer literals the reference documents (sum(abs2,[1,2,3,4]) = 30,
 * src/Compiler/runtime/compile.jl:36-39; contract([1 2;3 4],[5 6;7 8]) =
 * [19 22;43 50], src/Compiler/program/tracing.jl:872-875; 4096 BFloat16
 * gradients of 0.01 sum to 41, test/codegen/floor.jl:28-32) and on fp64
 * closed forms of each operator.
 *
 * What it follows in the reference (paths inside the Tempest.jl project):
 *   - kernel order: one item after another, a sequential left fold over the
 *     reduced axis, the fold observed once, then a second sweep for the outputs
 *     of full shape (src/Compiler/codegen/scalar.jl:200-256;
 *     src/Compiler/runtime/target.jl:308-327);
 *   - fold algebra: SumFold, Relative{Exponential} (online log-sum-exp) and
 *     Relative{Square} (Welford/Chan) with their rebase rules
 *     (src/Compiler/IR/folds.jl:66-89, 123-198, 229);
 *   - half precision: sums and relative folds accumulate in Float32 and the
 *     observed value rounds once to the element type (folds.jl:42-55, 306-309);
 *     every map rounds to the element type (scalar.jl:89);
 *   - products of half-precision factors widen to Float32, accumulate there
 *     and round once (src/Compiler/program/interpret.jl:59-63);
 *   - x / 2^k is lowered to x * 2^-k (src/Compiler/index/lower.jl:590-599).
 *
 * Layout: Julia arrays are dense column-major; a Julia (n, rows) matrix reduced
 * over its first axis is a row-major [rows][n] buffer reduced over the
 * innermost index.  "ld" is the distance between rows in elements.
 *
 * Every function here runs on the calling thread, items in order, as the
 * reference's CPU kernels do.  Rows are independent items, so a caller that
 * wants more cores hands disjoint row ranges to several threads (oracle.py
 * does); no result changes.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef uint16_t bf16_t;

static inline float bf16_to_f32(bf16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round to nearest even, NaN kept quiet: what BFloat16s.BFloat16(::Float32) does */
static inline bf16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (bf16_t)(u >> 16);
}

static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

void oracle_bf16_from_f32(const float *x, bf16_t *y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = f32_to_bf16(x[i]);
}
void oracle_f32_from_bf16(const bf16_t *x, float *y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = bf16_to_f32(x[i]);
}

/* ---------------------------------------------------------------- folds -- */

/* Relative{Exponential}: state (m, s) = (maximum, sum of exp(y - m)).
 * folds.jl:184 lse_shift; :153-158 statistic; :176 rebase; :187-198 combine. */
typedef struct { float m, s; } lse_state;
static inline float lse_shift(float m) { return isfinite(m) ? m : 0.0f; }
static inline lse_state lse_init(void) { lse_state a = { -INFINITY, 0.0f }; return a; }
static inline lse_state lse_lift(float y) { lse_state a = { y, 1.0f }; return a; }
static inline lse_state lse_combine(lse_state a, lse_state b) {
    lse_state r;
    r.m = fmaxf(a.m, b.m);
    float sh = lse_shift(r.m);
    r.s = a.s * expf(a.m - sh) + b.s * expf(b.m - sh);
    return r;
}
static inline float lse_observe(lse_state a) { return a.m + logf(a.s); }

/* Relative{Square}: state (n, sum, M2) with M2 = sum of (y - mean)^2.
 * folds.jl:159-162 statistic; :177 rebase. */
typedef struct { float n, sum, m2; } sq_state;
static inline sq_state sq_init(void) { sq_state a = { 0.0f, 0.0f, 0.0f }; return a; }
static inline sq_state sq_lift(float y) { sq_state a = { 1.0f, y, 0.0f }; return a; }
static inline float sq_rebase(float a, float n, float sum, float m) {
    if (n == 0.0f) return a;
    float d = sum / n - m;
    return a + n * (d * d);
}
static inline sq_state sq_combine(sq_state a, sq_state b) {
    sq_state r;
    r.n = a.n + b.n;
    r.sum = a.sum + b.sum;
    float m = r.sum / r.n;
    r.m2 = sq_rebase(a.m2, a.n, a.sum, m) + sq_rebase(b.m2, b.n, b.sum, m);
    return r;
}

/* SumFold over n elements in order (folds.jl:66-71). */
float oracle_sum_f32(const float *x, int64_t n) {
    float s = 0.0f;
    for (int64_t i = 0; i < n; i++) s = s + x[i];
    return s;
}
float oracle_sum_abs2_f32(const float *x, int64_t n) {
    float s = 0.0f;
    for (int64_t i = 0; i < n; i++) s = s + x[i] * x[i];
    return s;
}
/* A half-precision sum accumulates in Float32 and rounds once (folds.jl:307). */
bf16_t oracle_sum_bf16(const bf16_t *x, int64_t n) {
    float s = 0.0f;
    for (int64_t i = 0; i < n; i++) s = s + bf16_to_f32(x[i]);
    return f32_to_bf16(s);
}
float oracle_logsumexp_f32(const float *x, int64_t n) {
    lse_state st = lse_init();
    for (int64_t i = 0; i < n; i++) st = lse_combine(st, lse_lift(x[i]));
    return lse_observe(st);
}
/* mean and biased variance by the Relative{Square} fold, observed as the
 * statistic and as Sum(1) * 2^-k or / n */
void oracle_mean_var_f32(const float *x, int64_t n, float *mean, float *var) {
    sq_state st = sq_init();
    for (int64_t i = 0; i < n; i++) st = sq_combine(st, sq_lift(x[i]));
    *mean = st.sum / st.n;
    *var = st.m2 / (float)n;
}

/* --------------------------------------------------------------- softmax -- */
/* softmax_columns(x) = exp.(x .- logsumexp(x; dims = 1))
 * (test/fixtures/programs.jl:8; ext/NNlibExt.jl:17). */

void oracle_softmax_fwd_f32(const float *x, float *y, float *lse, int64_t n, int64_t rows,
                            int64_t ld) {
    for (int64_t r = 0; r < rows; r++) {
        const float *xr = x + r * ld;
        float *yr = y + r * ld;
        lse_state st = lse_init();
        for (int64_t i = 0; i < n; i++) st = lse_combine(st, lse_lift(xr[i]));
        float l = lse_observe(st);
        if (lse) lse[r] = l;
        for (int64_t i = 0; i < n; i++) yr[i] = expf(xr[i] - l);
    }
}

/* BFloat16, as the reference CPU path rounds: the fold in Float32 observed to
 * BFloat16, then x - lse and exp each rounded to BFloat16 (scalar.jl:89).
 * faithful = 0 keeps Float32 between the loads and the one final rounding: the
 * "fp32 CPU reference" half-precision results are compared with. */
void oracle_softmax_fwd_bf16(const bf16_t *x, bf16_t *y, float *lse, int64_t n, int64_t rows,
                             int64_t ld, int faithful) {
    for (int64_t r = 0; r < rows; r++) {
        const bf16_t *xr = x + r * ld;
        bf16_t *yr = y + r * ld;
        lse_state st = lse_init();
        for (int64_t i = 0; i < n; i++) st = lse_combine(st, lse_lift(bf16_to_f32(xr[i])));
        float l = lse_observe(st);
        if (faithful) l = round_bf16(l);
        if (lse) lse[r] = l;
        for (int64_t i = 0; i < n; i++) {
            float d = bf16_to_f32(xr[i]) - l;
            if (faithful) d = round_bf16(d);
            yr[i] = f32_to_bf16(expf(d));
        }
    }
}

/* Backward of the same program with upstream g (differentiate.jl:118 exp,
 * :110 minus, :215-218 log-sum-exp): t = g*y; dx = t - exp(x - lse) * sum(t),
 * the sum a SumFold over the row in order. */
void oracle_softmax_bwd_f32(const float *y, const float *g, float *dx, int64_t n, int64_t rows,
                            int64_t ld) {
    for (int64_t r = 0; r < rows; r++) {
        const float *yr = y + r * ld, *gr = g + r * ld;
        float *dr = dx + r * ld;
        float s = 0.0f;
        for (int64_t i = 0; i < n; i++) s = s + gr[i] * yr[i];
        for (int64_t i = 0; i < n; i++) dr[i] = gr[i] * yr[i] - yr[i] * s;
    }
}

void oracle_softmax_bwd_bf16(const bf16_t *y, const bf16_t *g, bf16_t *dx, int64_t n,
                             int64_t rows, int64_t ld, int faithful) {
    for (int64_t r = 0; r < rows; r++) {
        const bf16_t *yr = y + r * ld, *gr = g + r * ld;
        bf16_t *dr = dx + r * ld;
        float s = 0.0f;
        for (int64_t i = 0; i < n; i++) {
            float t = bf16_to_f32(gr[i]) * bf16_to_f32(yr[i]);
            if (faithful) t = round_bf16(t);
            s = s + t;
        }
        if (faithful) s = round_bf16(s);
        for (int64_t i = 0; i < n; i++) {
            float yv = bf16_to_f32(yr[i]);
            float t = bf16_to_f32(gr[i]) * yv, u = yv * s;
            if (faithful) { t = round_bf16(t); u = round_bf16(u); }
            dr[i] = f32_to_bf16(t - u);
        }
    }
}

/* ------------------------------------------------------------- layernorm -- */
/* layernorm(x, w): m = sum(x)/n; v = sum(abs2, x - m)/n;
 * y = (x - m) / sqrt(v + eps) * w (+ b)   (test/fixtures/programs.jl:13-17).
 * With the rewrites the CPU target applies (runtime/target.jl:222) the two
 * sums are one Relative{Square} fold (plan/rewrites.jl:6-13).  inv_n is
 * 1/n, exact when n is a power of two (index/lower.jl:590-599). */

void oracle_layernorm_fwd_f32(const float *x, const float *gamma, const float *beta, float *y,
                              float *mean, float *rstd, float eps, int64_t n, int64_t rows,
                              int64_t ld) {
    int pow2 = (n & (n - 1)) == 0;
    float inv_n = 1.0f / (float)n;
    for (int64_t r = 0; r < rows; r++) {
        const float *xr = x + r * ld;
        float *yr = y + r * ld;
        sq_state st = sq_init();
        for (int64_t i = 0; i < n; i++) st = sq_combine(st, sq_lift(xr[i]));
        float m = st.sum / st.n;
        float v = pow2 ? st.m2 * inv_n : st.m2 / (float)n;
        float sd = sqrtf(v + eps);
        if (mean) mean[r] = m;
        if (rstd) rstd[r] = 1.0f / sd;
        for (int64_t i = 0; i < n; i++) {
            float t = (xr[i] - m) / sd * gamma[i];
            yr[i] = beta ? t + beta[i] : t;
        }
    }
}

void oracle_layernorm_fwd_bf16(const bf16_t *x, const bf16_t *gamma, const bf16_t *beta, bf16_t *y,
                               float *mean, float *rstd, float eps, int64_t n, int64_t rows,
                               int64_t ld, int faithful) {
    int pow2 = (n & (n - 1)) == 0;
    float inv_n = 1.0f / (float)n;
    for (int64_t r = 0; r < rows; r++) {
        const bf16_t *xr = x + r * ld;
        bf16_t *yr = y + r * ld;
        sq_state st = sq_init();
        for (int64_t i = 0; i < n; i++) st = sq_combine(st, sq_lift(bf16_to_f32(xr[i])));
        float m = st.sum / st.n;
        float v = pow2 ? st.m2 * inv_n : st.m2 / (float)n;
        if (faithful) { m = round_bf16(m); v = round_bf16(v); }
        float sd = sqrtf(v + (faithful ? round_bf16(eps) : eps));
        if (faithful) sd = round_bf16(sd);
        if (mean) mean[r] = m;
        if (rstd) rstd[r] = 1.0f / sd;
        for (int64_t i = 0; i < n; i++) {
            float c = bf16_to_f32(xr[i]) - m;
            if (faithful) c = round_bf16(c);
            float q = c / sd;
            if (faithful) q = round_bf16(q);
            float t = q * bf16_to_f32(gamma[i]);
            if (beta) { if (faithful) t = round_bf16(t); t = t + bf16_to_f32(beta[i]); }
            yr[i] = f32_to_bf16(t);
        }
    }
}

/* Backward of layernorm with upstream g, the closed form the tape's rules
 * (differentiate.jl:106-155, 214) reduce to:
 *   xh = (x - m) * rstd, gh = g * gamma,
 *   dx = rstd * (gh - mean(gh) - xh * mean(gh * xh)),
 *   dgamma[i] = sum over rows of g * xh, dbeta[i] = sum over rows of g.
 * Row sums are SumFolds in order; dgamma and dbeta fold the rows in order.
 * Accumulation is Float32 for either element type; wide = 1 keeps Float64
 * accumulators for dgamma/dbeta (a tighter yardstick for the long column sums). */
void oracle_layernorm_bwd_f32(const float *x, const float *gamma, const float *g, float *dx,
                              float *dgamma, float *dbeta, float eps, int64_t n, int64_t rows,
                              int64_t ld, int wide) {
    float inv_n = 1.0f / (float)n;
    double *dgw = (double *)calloc((size_t)n * 2, sizeof(double));
    double *dbw = dgw + n;
    float *rs = (float *)malloc((size_t)rows * 2 * sizeof(float));
    for (int64_t r = 0; r < rows; r++) {
        const float *xr = x + r * ld, *gr = g + r * ld;
        float *dr = dx + r * ld;
        sq_state st = sq_init();
        for (int64_t i = 0; i < n; i++) st = sq_combine(st, sq_lift(xr[i]));
        float m = st.sum / st.n;
        float v = st.m2 * inv_n;
        float rstd = 1.0f / sqrtf(v + eps);
        float s1 = 0.0f, s2 = 0.0f;
        for (int64_t i = 0; i < n; i++) {
            float xh = (xr[i] - m) * rstd, gh = gr[i] * gamma[i];
            s1 = s1 + gh;
            s2 = s2 + gh * xh;
        }
        float c1 = s1 * inv_n, c2 = s2 * inv_n;
        for (int64_t i = 0; i < n; i++) {
            float xh = (xr[i] - m) * rstd, gh = gr[i] * gamma[i];
            dr[i] = rstd * (gh - c1 - xh * c2);
        }
        rs[2 * r] = m;
        rs[2 * r + 1] = rstd;
    }
    if (dgamma || dbeta) {
        if (wide) {
            for (int64_t r = 0; r < rows; r++) {
                float m = rs[2 * r], rstd = rs[2 * r + 1];
                for (int64_t i = 0; i < n; i++) {
                    float xh = (x[r * ld + i] - m) * rstd;
                    dgw[i] += (double)g[r * ld + i] * (double)xh;
                    dbw[i] += (double)g[r * ld + i];
                }
            }
            for (int64_t i = 0; i < n; i++) {
                if (dgamma) dgamma[i] = (float)dgw[i];
                if (dbeta) dbeta[i] = (float)dbw[i];
            }
        } else {
            float *dg = (float *)calloc((size_t)n * 2, sizeof(float)), *db = dg + n;
            for (int64_t r = 0; r < rows; r++) {
                float m = rs[2 * r], rstd = rs[2 * r + 1];
                for (int64_t i = 0; i < n; i++) {
                    float xh = (x[r * ld + i] - m) * rstd;
                    dg[i] = dg[i] + g[r * ld + i] * xh;
                    db[i] = db[i] + g[r * ld + i];
                }
            }
            for (int64_t i = 0; i < n; i++) {
                if (dgamma) dgamma[i] = dg[i];
                if (dbeta) dbeta[i] = db[i];
            }
            free(dg);
        }
    }
    free(rs);
    free(dgw);
}

/* BFloat16 inputs widened to Float32, Float32 inside, outputs rounded once
 * (the fp32 CPU reference for half precision). */
void oracle_layernorm_bwd_bf16(const bf16_t *x, const bf16_t *gamma, const bf16_t *g, bf16_t *dx,
                               bf16_t *dgamma, bf16_t *dbeta, float eps, int64_t n, int64_t rows,
                               int64_t ld, int wide) {
    size_t tot = (size_t)rows * (size_t)n;
    float *xf = (float *)malloc(tot * 3 * sizeof(float) + (size_t)n * 3 * sizeof(float));
    float *gf = xf + tot, *df = gf + tot, *gam = df + tot, *dg = gam + n, *db = dg + n;
    for (int64_t r = 0; r < rows; r++)
        for (int64_t i = 0; i < n; i++) {
            xf[r * n + i] = bf16_to_f32(x[r * ld + i]);
            gf[r * n + i] = bf16_to_f32(g[r * ld + i]);
        }
    for (int64_t i = 0; i < n; i++) gam[i] = bf16_to_f32(gamma[i]);
    oracle_layernorm_bwd_f32(xf, gam, gf, df, dg, db, eps, n, rows, n, wide);
    for (int64_t r = 0; r < rows; r++)
        for (int64_t i = 0; i < n; i++) dx[r * ld + i] = f32_to_bf16(df[r * n + i]);
    for (int64_t i = 0; i < n; i++) {
        if (dgamma) dgamma[i] = f32_to_bf16(dg[i]);
        if (dbeta) dbeta[i] = f32_to_bf16(db[i]);
    }
    free(xf);
}

/* ------------------------------------------------------------------ GEMM -- */
/* A product is a SumFold over the shared axis of the term a*b
 * (src/Compiler/program/interpret.jl:59-63; scalar.jl:200-256): for each output
 * element, k runs in order.  Row-major C[M][N] = A[M][K] * B, with B given
 * either as [K][N] (b_kn = 1: a Julia (out,in) weight stored [in][out]) or as
 * [N][K] (b_kn = 0).  a_km = 1 reads A as [K][M].
 * epilogue: 0 none, 1 +bias[N], 2 gelu_tanh(+bias), 3 tanh(+bias).
 * gelu(x) = x/2 * (1 + tanh(0.7978846 (x + 0.044715 x^3)))
 * (test/fixtures/programs.jl:19). */

static inline float gelu_tanh_f(float x) {
    return x * 0.5f * (1.0f + tanhf(0.7978846f * (x + 0.044715f * x * x * x)));
}
static inline float gelu_tanh_grad_f(float x) {
    float u = 0.7978846f * (x + 0.044715f * x * x * x);
    float t = tanhf(u);
    float du = 0.7978846f * (1.0f + 3.0f * 0.044715f * x * x);
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
}
float oracle_gelu_tanh(float x) { return gelu_tanh_f(x); }
float oracle_gelu_tanh_grad(float x) { return gelu_tanh_grad_f(x); }

static inline float epilogue_f(float acc, const float *bias, int64_t j, int epilogue) {
    if (epilogue >= 1 && bias) acc = acc + bias[j];
    if (epilogue == 2) acc = gelu_tanh_f(acc);
    if (epilogue == 3) acc = tanhf(acc);
    return acc;
}

void oracle_gemm_f32(const float *A, const float *B, const float *bias, float *C, int64_t M,
                     int64_t N, int64_t K, int a_km, int b_kn, int epilogue) {
    for (int64_t i = 0; i < M; i++)
        for (int64_t j = 0; j < N; j++) {
            float acc = 0.0f;
            for (int64_t k = 0; k < K; k++) {
                float a = a_km ? A[k * M + i] : A[i * K + k];
                float b = b_kn ? B[k * N + j] : B[j * K + k];
                acc = acc + a * b;
            }
            C[i * N + j] = epilogue_f(acc, bias, j, epilogue);
        }
}

/* BFloat16 factors widen to Float32; the accumulator is Float32; the product
 * rounds once.  pre (optional, Float32 [M][N]) receives the value before the
 * activation, as the backward of the activation reads it. */
void oracle_gemm_bf16(const bf16_t *A, const bf16_t *B, const bf16_t *bias, bf16_t *C, float *pre,
                      int64_t M, int64_t N, int64_t K, int a_km, int b_kn, int epilogue) {
    for (int64_t i = 0; i < M; i++)
        for (int64_t j = 0; j < N; j++) {
            float acc = 0.0f;
            for (int64_t k = 0; k < K; k++) {
                float a = bf16_to_f32(a_km ? A[k * M + i] : A[i * K + k]);
                float b = bf16_to_f32(b_kn ? B[k * N + j] : B[j * K + k]);
                acc = acc + a * b;
            }
            if (epilogue >= 1 && bias) acc = acc + bf16_to_f32(bias[j]);
            if (pre) pre[i * N + j] = acc;
            if (epilogue == 2) acc = gelu_tanh_f(acc);
            if (epilogue == 3) acc = tanhf(acc);
            C[i * N + j] = f32_to_bf16(acc);
        }
}

/* ---------------------------------------------------- README loss + grad -- */
/* loss(w, b, x) = sum(abs2, tanh.(w' * x .+ b)), w (I,J), b (J), x (I,N)
 * (README.md:15).  Buffers are the Julia arrays' memory: w[j*I + i],
 * x[n*I + i], z[n*J + j].  Gradients by the reference's rules
 * (differentiate.jl:127 abs2, :134 tanh, :214 sum, :461-467 contract):
 *   y = tanh z, gz = 2y * (1 - y*y),
 *   dw[i,j] = sum_n x[i,n] gz[j,n], db[j] = sum_n gz[j,n],
 *   dx[i,n] = sum_j w[i,j] gz[j,n]. */
float oracle_readme_loss_grad(const float *w, const float *b, const float *x, float *dw, float *db,
                              float *dx, int64_t I, int64_t J, int64_t N) {
    float *gz = (float *)malloc((size_t)(J * N) * sizeof(float));
    float loss = 0.0f;
    for (int64_t n = 0; n < N; n++)
        for (int64_t j = 0; j < J; j++) {
            float acc = 0.0f;
            for (int64_t i = 0; i < I; i++) acc = acc + w[j * I + i] * x[n * I + i];
            float y = tanhf(acc + b[j]);
            loss = loss + y * y;
            gz[n * J + j] = (2.0f * y) * (1.0f - y * y);
        }
    for (int64_t j = 0; j < J; j++) {
        for (int64_t i = 0; i < I; i++) {
            float acc = 0.0f;
            for (int64_t n = 0; n < N; n++) acc = acc + x[n * I + i] * gz[n * J + j];
            dw[j * I + i] = acc;
        }
        float s = 0.0f;
        for (int64_t n = 0; n < N; n++) s = s + gz[n * J + j];
        db[j] = s;
    }
    for (int64_t n = 0; n < N; n++)
        for (int64_t i = 0; i < I; i++) {
            float acc = 0.0f;
            for (int64_t j = 0; j < J; j++) acc = acc + w[j * I + i] * gz[n * J + j];
            dx[n * I + i] = acc;
        }
    free(gz);
    return loss;
}

/* ---- scans ------------------------------------------------------------------------------------------
 * The running fold of a vector taken in sequence, one state carried from element to element, as the
 * reference's CPU path sweeps a scan (src/Compiler/codegen/scalar.jl:200-256 with the scanned axis kept;
 * folds: src/Compiler/IR/folds.jl:66-89, the GenericFold recurrence :279-288, Welford's variance named
 * with GenericFold test/fixtures/programs.jl:40-44).  op: 0 sum, 1 prod, 2 max, 3 min, 4 affine
 * (h = a h + b from (x[i], x2[i]), h starting at 0), 5 running population variance.  `stride` is the
 * distance between consecutive scanned elements; `reverse` starts at the far end. */
void oracle_scan_f32(const float *x, const float *x2, float *y, int64_t count, int64_t stride, int op, int reverse) {
    float acc = op == 1 ? 1.0f : op == 2 ? -INFINITY : op == 3 ? INFINITY : 0.0f;
    float n = 0.0f, mean = 0.0f, m2 = 0.0f;
    for (int64_t p = 0; p < count; p++) {
        const int64_t i = (reverse ? count - 1 - p : p) * stride;
        const float v = x[i];
        switch (op) {
            case 0: acc = acc + v; break;
            case 1: acc = acc * v; break;
            case 2: acc = v > acc ? v : acc; break;
            case 3: acc = v < acc ? v : acc; break;
            case 4: acc = v * acc + x2[i]; break;
            default: {   /* Welford: one element joins the state */
                n += 1.0f;
                const float d = v - mean;
                mean += d / n;
                m2 += d * (v - mean);
                acc = m2 / n;
            }
        }
        y[i] = acc;
    }
}
