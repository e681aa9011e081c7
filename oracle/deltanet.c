/*
 * CPU oracle, gated DeltaNet: the rule token by token, the reference the example itself checks its
 * chunked form against (examples/deltanet.jl:89-101, `sequential`), in Float64:
 *     S_t = exp(a_t) (S_{t-1} - beta_t k_t (k_t' S_{t-1})) + beta_t k_t v_t',   o_t = S_t' q_t
 * with S a (dk x dv) state per head, zero at t = 0.  TEST INFRASTRUCTURE ONLY.
 *
 * Layout: q, k are Julia (dk, T, heads) arrays = memory [head][t][dk]; v is (dv, T, heads) =
 * [head][t][dv]; a, beta are (T, heads) = [head][t]; the result is (T, dv, heads) = memory
 * [head][dv][t] (examples/deltanet.jl:56-57, 85).  q, k, v arrive as BFloat16 bit patterns and are
 * widened; a and beta are Float32.  The output is Float64 (callers round).
 *
 * Parity pinning: no stored tensors exist in the reference for this path; the chunked algebra
 * (examples/deltanet.jl:58-85) equals this recurrence exactly in exact arithmetic, which is what the
 * example prints.  Beyond that parity is unpinned.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline double bfd(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return (double)f;
}

/* one head */
void oracle_deltanet_head(const uint16_t *q, const uint16_t *k, const uint16_t *v, const float *a, const float *beta,
                          double *o, int T, int dk, int dv, int head) {
    const uint16_t *qh = q + (size_t)head * T * dk, *kh = k + (size_t)head * T * dk, *vh = v + (size_t)head * T * dv;
    const float *ah = a + (size_t)head * T, *bh = beta + (size_t)head * T;
    double *oh = o + (size_t)head * dv * T;
    double *S = (double *)calloc((size_t)dk * dv, sizeof(double));
    double *kS = (double *)malloc(sizeof(double) * dv);
    double *kt = (double *)malloc(sizeof(double) * dk);
    for (int t = 0; t < T; t++) {
        for (int i = 0; i < dk; i++) kt[i] = bfd(kh[(size_t)t * dk + i]);
        for (int j = 0; j < dv; j++) kS[j] = 0.0;
        for (int i = 0; i < dk; i++)
            for (int j = 0; j < dv; j++) kS[j] += kt[i] * S[(size_t)i * dv + j];
        const double g = exp((double)ah[t]), b = (double)bh[t];
        for (int i = 0; i < dk; i++)
            for (int j = 0; j < dv; j++)
                S[(size_t)i * dv + j] = g * (S[(size_t)i * dv + j] - b * kt[i] * kS[j]) +
                                        b * kt[i] * bfd(vh[(size_t)t * dv + j]);
        for (int j = 0; j < dv; j++) {
            double acc = 0.0;
            for (int i = 0; i < dk; i++) acc += S[(size_t)i * dv + j] * bfd(qh[(size_t)t * dk + i]);
            oh[(size_t)j * T + t] = acc;
        }
    }
    free(S);
    free(kS);
    free(kt);
}
