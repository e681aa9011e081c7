/*
 * CPU oracle for generic map -> fold row groups.  TEST INFRASTRUCTURE ONLY.
 *
 * The reference's floor for a reduction group (src/Compiler/codegen/scalar.jl:200-256), restated over the
 * descriptor of include/tempest_b200.h (which only declares the data layout: nothing of the product is
 * linked here): one row after another on the calling thread; for each phase initialise the states, sweep the
 * folded axis in order combining each lifted element into the state, observe; a last sweep writes the
 * outputs of full shape.  Terms are evaluated per element in Float32, one after another (IR/terms.jl:12-87);
 * the fold algebra is IR/folds.jl:66-89 (sum, max, min, prod), :187-198 (log-sum-exp: (max, sum of
 * exp(y - max)), rebased when the max moves), :143, 166-182 (Welford's update of (count, mean, centred sum
 * of squares)).  Outputs round once to their element type.
 *
 * `oracle_group_rows` works in Float32 as the floor does; `oracle_group_rows_f64` is the same evaluator in
 * Float64 (inputs widened, outputs rounded once), the yardstick for how far the Float32 floor itself drifts
 * on long rows.
 *
 * Parity unpinned for this file: the reference holds no stored vectors for arbitrary groups; the tests pin
 * it on the named operators' oracles (softmax, LayerNorm), which are pinned on the reference's known
 * answers, and on Float64 closed forms.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "../include/tempest_b200.h"

typedef uint16_t bf16_t;

static float widen(bf16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static bf16_t narrow(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (bf16_t)(u >> 16);
}

static int arity(int op) {
    if (op <= TB200_T_STAT2) return 0;
    if (op <= TB200_T_MIN) return 2;
    if (op == TB200_T_FMA || op == TB200_T_SELECT) return 3;
    return 1;
}


#define REAL float
#define NAME(x) x
#define R_MAX fmaxf
#define R_MIN fminf
#define R_EXP expf
#define R_LOG logf
#define R_TANH tanhf
#define R_SQRT sqrtf
#define R_ABS fabsf
#define R_FMA fmaf
#include "group_body.inc"
#undef REAL
#undef NAME
#undef R_MAX
#undef R_MIN
#undef R_EXP
#undef R_LOG
#undef R_TANH
#undef R_SQRT
#undef R_ABS
#undef R_FMA

#define REAL double
#define NAME(x) x##_f64
#define R_MAX fmax
#define R_MIN fmin
#define R_EXP exp
#define R_LOG log
#define R_TANH tanh
#define R_SQRT sqrt
#define R_ABS fabs
#define R_FMA fma
#include "group_body.inc"
