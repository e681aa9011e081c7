/*
 * CPU oracle, attention: a plain-C restatement of the reference's attention program and of its
 * derivative.  TEST INFRASTRUCTURE ONLY (see tempest_oracle.c).
 *
 * Forward (test/fixtures/operations.jl:21-76): arrays (features, heads, positions, batch), memory
 * [batch][position][head][feature]; query head h reads key/value head h / (heads / kv_heads);
 *   s[n] = scale * sum_d k[d,n] q[d,m]     in Float32 from the BFloat16 inputs widened (:52, :57)
 *   causal keeps n <= m, else -Inf (typemin) (:59)
 *   lse[m] = logsumexp_n s   (the Relative{Exponential} fold, src/Compiler/IR/folds.jl:187-198, 229)
 *   o[d,m] = sum_n v[d,n] exp(s[n] - lse[m]), rounded to the inputs' type (:74); lse stays Float32.
 * round_p = 1 rounds the weights exp(s - lse) to BFloat16 before the second product, as the GPU
 * kernels of the reference do (docs/src/cuda.md:40-46, ext/cuTileExt/emit.jl:914-921).
 *
 * Backward (differentiate.jl:215-218 for the log-sum-exp, :461-467 for the products): with upstream dO,
 *   p = exp(s - lse), delta[m] = sum_d dO[d,m] o[d,m] (o as stored: docs/src/cuda.md:54-63),
 *   dv[n] += p dO[m], dp = v[n].dO[m], ds = p (dp - delta), dq[m] += scale ds k[n], dk[n] += scale ds q[m].
 * All sums in order, Float32; results rounded once to BFloat16.
 *
 * Parity pinning: the reference holds no stored tensors for this path; these functions are checked
 * against Float64 closed forms in tests/test_oracle.py. Beyond that parity is unpinned.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef uint16_t bf16_t;

static inline float bf(bf16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline bf16_t to_bf(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (bf16_t)(u >> 16);
}

typedef struct {
    int batch, heads, kv_heads, queries, keys, d, causal;
    float scale;
} attn_shape;

static inline int64_t at(const attn_shape *s, int heads, int positions, int b, int pos, int h) {
    return (((int64_t)b * positions + pos) * heads + h) * s->d;
}

/* queries [m0, m1) of one (batch, head) */
void oracle_attention_fwd_rows(const bf16_t *q, const bf16_t *k, const bf16_t *v, bf16_t *o, float *lse,
                               int batch, int heads, int kv_heads, int queries, int keys, int d, int causal,
                               float scale, int b, int h, int m0, int m1, int round_p) {
    attn_shape sh = { batch, heads, kv_heads, queries, keys, d, causal, scale };
    const int hk = h / (heads / kv_heads);
    float *s = (float *)malloc(sizeof(float) * (size_t)keys);
    float *acc = (float *)malloc(sizeof(float) * (size_t)d);
    for (int m = m0; m < m1; m++) {
        const bf16_t *qm = q + at(&sh, heads, queries, b, m, h);
        float mx = -INFINITY, sum = 0.0f;   /* the online fold: state (maximum, rebased sum) */
        for (int n = 0; n < keys; n++) {
            float t;
            if (causal && n > m) t = -INFINITY;
            else {
                const bf16_t *kn = k + at(&sh, kv_heads, keys, b, n, hk);
                float a = 0.0f;
                for (int i = 0; i < d; i++) a = a + bf(kn[i]) * bf(qm[i]);
                t = a * scale;
            }
            s[n] = t;
            const float nm = fmaxf(mx, t);
            const float shift = isfinite(nm) ? nm : 0.0f;
            sum = sum * expf(mx - shift) + expf(t - shift);
            mx = nm;
        }
        const float l = mx + logf(sum);
        if (lse) lse[((int64_t)b * queries + m) * heads + h] = l;
        for (int i = 0; i < d; i++) acc[i] = 0.0f;
        for (int n = 0; n < keys; n++) {
            float w = expf(s[n] - l);
            if (round_p) w = bf(to_bf(w));
            if (w == 0.0f) continue;
            const bf16_t *vn = v + at(&sh, kv_heads, keys, b, n, hk);
            for (int i = 0; i < d; i++) acc[i] = acc[i] + bf(vn[i]) * w;
        }
        bf16_t *om = o + at(&sh, heads, queries, b, m, h);
        for (int i = 0; i < d; i++) om[i] = to_bf(acc[i]);
    }
    free(s);
    free(acc);
}

/* One (batch, key/value head): dq for the query heads that read it, dk and dv summed over them.
 * round_p rounds p and ds to BFloat16 before they enter a product, as the GPU kernels do. */
void oracle_attention_bwd_head(const bf16_t *q, const bf16_t *k, const bf16_t *v, const bf16_t *o, const float *lse,
                               const bf16_t *dout, bf16_t *dq, bf16_t *dk, bf16_t *dv, int batch, int heads,
                               int kv_heads, int queries, int keys, int d, int causal, float scale, int b, int hk,
                               int round_p) {
    attn_shape sh = { batch, heads, kv_heads, queries, keys, d, causal, scale };
    const int group = heads / kv_heads;
    float *dkf = (float *)calloc((size_t)keys * d, sizeof(float));
    float *dvf = (float *)calloc((size_t)keys * d, sizeof(float));
    float *dqf = (float *)malloc(sizeof(float) * (size_t)d);
    for (int g = 0; g < group; g++) {
        const int h = hk * group + g;
        for (int m = 0; m < queries; m++) {
            const bf16_t *qm = q + at(&sh, heads, queries, b, m, h);
            const bf16_t *om = o + at(&sh, heads, queries, b, m, h);
            const bf16_t *gm = dout + at(&sh, heads, queries, b, m, h);
            const float l = lse[((int64_t)b * queries + m) * heads + h];
            float delta = 0.0f;
            for (int i = 0; i < d; i++) delta = delta + bf(gm[i]) * bf(om[i]);
            for (int i = 0; i < d; i++) dqf[i] = 0.0f;
            const int last = causal ? (m < keys - 1 ? m : keys - 1) : keys - 1;
            for (int n = 0; n <= last; n++) {
                const bf16_t *kn = k + at(&sh, kv_heads, keys, b, n, hk);
                const bf16_t *vn = v + at(&sh, kv_heads, keys, b, n, hk);
                float a = 0.0f, dp = 0.0f;
                for (int i = 0; i < d; i++) {
                    a = a + bf(kn[i]) * bf(qm[i]);
                    dp = dp + bf(vn[i]) * bf(gm[i]);
                }
                float p = expf(a * scale - l);
                float ds = p * (dp - delta);
                if (round_p) { p = bf(to_bf(p)); ds = bf(to_bf(ds)); }
                float *dkn = dkf + (size_t)n * d, *dvn = dvf + (size_t)n * d;
                for (int i = 0; i < d; i++) {
                    dvn[i] = dvn[i] + p * bf(gm[i]);
                    dkn[i] = dkn[i] + ds * bf(qm[i]);
                    dqf[i] = dqf[i] + ds * bf(kn[i]);
                }
            }
            bf16_t *dqm = dq + at(&sh, heads, queries, b, m, h);
            for (int i = 0; i < d; i++) dqm[i] = to_bf(dqf[i] * scale);
        }
    }
    for (int n = 0; n < keys; n++) {
        bf16_t *dkn = dk + at(&sh, kv_heads, keys, b, n, hk), *dvn = dv + at(&sh, kv_heads, keys, b, n, hk);
        for (int i = 0; i < d; i++) {
            dkn[i] = to_bf(dkf[(size_t)n * d + i] * scale);
            dvn[i] = to_bf(dvf[(size_t)n * d + i]);
        }
    }
    free(dkf);
    free(dvf);
    free(dqf);
}
