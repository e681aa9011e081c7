// Generic fused map -> fold row groups: a term DAG run by a small interpreter.
//
// What the named row kernels (softmax, LayerNorm and their pullbacks) hard-code, this file takes as data:
// the terms of src/Compiler/IR/terms.jl:12-87 (Load, Lit, Ix, Apply, Stat, Cast) in topological order, the
// folds of src/Compiler/IR/folds.jl:66-89 and :123-198, and the phases of the reference's floor
// (src/Compiler/codegen/scalar.jl:200-256): per row, every fold of phase 0 in one sweep, then the folds that
// read those results, ..., then one sweep for the full-shape outputs.  The fold algebra is the reference's:
// log-sum-exp keeps (max, sum of exp(y - max)) and rebases when the max moves (folds.jl:187-198); mean and
// variance keep (count, mean, centred sum of squares) with Welford's update and Chan's merge
// (folds.jl:143, 166-182); all states are Float32 whatever the stored type (folds.jl:306-309) and every output
// rounds once.
//
// Schedule: a row belongs to a group of 8..256 threads of a 256-thread block; each thread walks the row in
// steps of four consecutive elements, evaluates the terms the current phase needs (a bit mask worked out on
// the host) for those four elements, and feeds the phase's folds; partial states meet through shuffles and,
// above 32 threads, shared memory.  Rows are read again in every phase -- from L1/L2, since a row group's
// working set is a few rows -- so HBM traffic stays one read per input and one write per output.  The
// interpreter costs instructions, not bytes: expect a fraction of the named kernels' rate.
#include "common.cuh"
#include "generic.cuh"

namespace tb200 {
namespace {

constexpr int kThreads = 256;
constexpr int kV = 4;
constexpr int kMaxT = TB200_GROUP_MAX_TERMS;
constexpr int kMaxF = TB200_GROUP_MAX_FOLDS;
constexpr int kMaxPhases = kMaxF + 1;

struct GenericArgs {
    tb200_group_desc d;
    const void *in[TB200_GROUP_MAX_INPUTS];
    void *out[TB200_GROUP_MAX_OUTPUTS];
    unsigned long long need[kMaxPhases];   // terms to evaluate in each phase
    int phases;                            // fold phases; phase `phases` is the output sweep
    int tpr;                               // threads per row
    unsigned vec_in, vec_out;              // bit i: input / output i takes 4-element accesses
};

struct State { float a, b, c; };

__device__ __forceinline__ State fold_init(int kind) {
    switch (kind) {
        case TB200_FOLD_MAX: return {-INFINITY, 0.0f, 0.0f};
        case TB200_FOLD_MIN: return {INFINITY, 0.0f, 0.0f};
        case TB200_FOLD_PROD: return {1.0f, 0.0f, 0.0f};
        case TB200_FOLD_LOGSUMEXP: return {-INFINITY, 0.0f, 0.0f};
        default: return {0.0f, 0.0f, 0.0f};
    }
}

__device__ __forceinline__ void fold_lift(int kind, State &s, float y) {
    switch (kind) {
        case TB200_FOLD_SUM: s.a += y; break;
        case TB200_FOLD_MAX: s.a = fmaxf(s.a, y); break;
        case TB200_FOLD_MIN: s.a = fminf(s.a, y); break;
        case TB200_FOLD_PROD: s.a *= y; break;
        case TB200_FOLD_LOGSUMEXP: {
            const float m = fmaxf(s.a, y);
            if (m > -INFINITY) s.b = s.b * __expf(s.a - m) + __expf(y - m);
            s.a = m;
            break;
        }
        default: {   // Welford
            s.a += 1.0f;
            const float d = y - s.b;
            s.b += __fdividef(d, s.a);
            s.c = fmaf(d, y - s.b, s.c);
        }
    }
}

// `s` holds the earlier elements, `o` the later ones
__device__ __forceinline__ void fold_merge(int kind, State &s, const State &o) {
    switch (kind) {
        case TB200_FOLD_SUM: s.a += o.a; break;
        case TB200_FOLD_MAX: s.a = fmaxf(s.a, o.a); break;
        case TB200_FOLD_MIN: s.a = fminf(s.a, o.a); break;
        case TB200_FOLD_PROD: s.a *= o.a; break;
        case TB200_FOLD_LOGSUMEXP: {
            const float m = fmaxf(s.a, o.a);
            if (m > -INFINITY) s.b = s.b * __expf(s.a - m) + o.b * __expf(o.a - m);
            s.a = m;
            break;
        }
        default: {   // Chan
            const float n = s.a + o.a;
            if (n > 0.0f) {
                const float d = o.b - s.b, w = o.a / n;
                s.c = s.c + o.c + d * d * s.a * w;
                s.b = fmaf(d, w, s.b);
            }
            s.a = n;
        }
    }
}

__device__ __forceinline__ void fold_observe(int kind, const State &s, float &first, float &second) {
    second = 0.0f;
    switch (kind) {
        case TB200_FOLD_LOGSUMEXP: first = s.a > -INFINITY ? s.a + logf(s.b) : -INFINITY; break;
        case TB200_FOLD_MEANVAR: first = s.b; second = s.a > 0.0f ? s.c / s.a : 0.0f; break;
        default: first = s.a;
    }
}

__device__ __forceinline__ State shuffle_xor(const State &s, int offset) {
    return {__shfl_xor_sync(0xffffffffu, s.a, offset), __shfl_xor_sync(0xffffffffu, s.b, offset),
            __shfl_xor_sync(0xffffffffu, s.c, offset)};
}

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ void load_input(const GenericArgs &A, int idx, long long row, long long i0, float *r) {
    const tb200_group_input in = A.d.inputs[idx];
    const bool bf = in.dtype == TB200_BF16;
    if (in.shape == TB200_SHAPE_PER_ROW || in.shape == TB200_SHAPE_SCALAR) {
        const long long at = in.shape == TB200_SHAPE_SCALAR ? 0 : row;
        const float x = bf ? __bfloat162float(static_cast<const __nv_bfloat16 *>(A.in[idx])[at])
                           : __ldg(static_cast<const float *>(A.in[idx]) + at);
#pragma unroll
        for (int e = 0; e < kV; e++) r[e] = x;
        return;
    }
    const long long base = (in.shape == TB200_SHAPE_FULL ? row * in.ld : 0) + i0;
    if (((A.vec_in >> idx) & 1u) && i0 + kV <= A.d.n) {
        if (bf) {
            const uint2 w = __ldg(reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(A.in[idx]) + base));
            unpack_bf16x2(w.x, r[0], r[1]);
            unpack_bf16x2(w.y, r[2], r[3]);
        } else {
            const float4 w = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(A.in[idx]) + base));
            r[0] = w.x; r[1] = w.y; r[2] = w.z; r[3] = w.w;
        }
        return;
    }
#pragma unroll
    for (int e = 0; e < kV; e++) {
        float x = 0.0f;
        if (i0 + e < A.d.n)
            x = bf ? __bfloat162float(static_cast<const __nv_bfloat16 *>(A.in[idx])[base + e])
                   : __ldg(static_cast<const float *>(A.in[idx]) + base + e);
        r[e] = x;
    }
}

__device__ __forceinline__ void store_output(const GenericArgs &A, int idx, long long row, long long i0, const float *r) {
    const tb200_group_output out = A.d.outputs[idx];
    const long long base = row * out.ld + i0;
    const bool bf = out.dtype == TB200_BF16;
    if (((A.vec_out >> idx) & 1u) && i0 + kV <= A.d.n) {
        if (bf) {
            uint2 w;
            w.x = pack_bf16x2(r[0], r[1]);
            w.y = pack_bf16x2(r[2], r[3]);
            __stcs(reinterpret_cast<uint2 *>(static_cast<__nv_bfloat16 *>(A.out[idx]) + base), w);
        } else {
            __stcs(reinterpret_cast<float4 *>(static_cast<float *>(A.out[idx]) + base), make_float4(r[0], r[1], r[2], r[3]));
        }
        return;
    }
#pragma unroll
    for (int e = 0; e < kV; e++)
        if (i0 + e < A.d.n) {
            if (bf) static_cast<__nv_bfloat16 *>(A.out[idx])[base + e] = __float2bfloat16_rn(r[e]);
            else static_cast<float *>(A.out[idx])[base + e] = r[e];
        }
}

#define TB200_UNARY(expr)                          \
    _Pragma("unroll") for (int e = 0; e < kV; e++) { \
        const float x = va[e];                     \
        r[e] = (expr);                             \
    }                                              \
    break
#define TB200_BINARY(expr)                         \
    _Pragma("unroll") for (int e = 0; e < kV; e++) { \
        const float x = va[e], y = vb[e];          \
        r[e] = (expr);                             \
    }                                              \
    break

__global__ void __launch_bounds__(kThreads) generic_rows_kernel(const __grid_constant__ GenericArgs A) {
    __shared__ State xchg[kThreads / 32][kMaxF];
    const int tid = threadIdx.x, tpr = A.tpr;
    const int rows_per_block = kThreads / tpr;
    const int group = tid / tpr, t = tid % tpr;
    const int warps_per_row = tpr / 32;
    const long long n = A.d.n;
    float val[kMaxT][kV];
    float obs[kMaxF][2];

    for (long long row_base = static_cast<long long>(blockIdx.x) * rows_per_block; row_base < A.d.rows;
         row_base += static_cast<long long>(gridDim.x) * rows_per_block) {
        const long long row = row_base + group;
        const bool active = row < A.d.rows;
        for (int phase = 0; phase <= A.phases; phase++) {
            const unsigned long long need = A.need[phase];
            State st[kMaxF];
#pragma unroll
            for (int f = 0; f < kMaxF; f++) st[f] = fold_init(f < A.d.n_folds ? A.d.folds[f].kind : 0);
            if (active) {
                for (long long i0 = static_cast<long long>(t) * kV; i0 < n; i0 += static_cast<long long>(tpr) * kV) {
                    for (int k = 0; k < A.d.n_terms; k++) {
                        if (!((need >> k) & 1ull)) continue;
                        const tb200_term T = A.d.terms[k];
                        float *r = val[k];
                        const float *va = val[T.a < 0 || T.a >= kMaxT ? 0 : T.a], *vb = val[T.b < 0 || T.b >= kMaxT ? 0 : T.b],
                                    *vc = val[T.c < 0 || T.c >= kMaxT ? 0 : T.c];
                        switch (T.op) {
                            case TB200_T_LOAD: load_input(A, T.a, row, i0, r); break;
                            case TB200_T_LIT:
#pragma unroll
                                for (int e = 0; e < kV; e++) r[e] = T.imm;
                                break;
                            case TB200_T_INDEX:
#pragma unroll
                                for (int e = 0; e < kV; e++) r[e] = static_cast<float>(i0 + e);
                                break;
                            case TB200_T_STAT:
#pragma unroll
                                for (int e = 0; e < kV; e++) r[e] = obs[T.a][0];
                                break;
                            case TB200_T_STAT2:
#pragma unroll
                                for (int e = 0; e < kV; e++) r[e] = obs[T.a][1];
                                break;
                            case TB200_T_ADD: TB200_BINARY(x + y);
                            case TB200_T_SUB: TB200_BINARY(x - y);
                            case TB200_T_MUL: TB200_BINARY(x * y);
                            case TB200_T_DIV: TB200_BINARY(x / y);
                            case TB200_T_MAX: TB200_BINARY(fmaxf(x, y));
                            case TB200_T_MIN: TB200_BINARY(fminf(x, y));
                            case TB200_T_NEG: TB200_UNARY(-x);
                            case TB200_T_EXP: TB200_UNARY(expf(x));
                            case TB200_T_LOG: TB200_UNARY(logf(x));
                            case TB200_T_TANH: TB200_UNARY(tanhf(x));
                            case TB200_T_SQRT: TB200_UNARY(sqrtf(x));
                            case TB200_T_RSQRT: TB200_UNARY(1.0f / sqrtf(x));
                            case TB200_T_ABS: TB200_UNARY(fabsf(x));
                            case TB200_T_ABS2: TB200_UNARY(x * x);
                            case TB200_T_RECIP: TB200_UNARY(1.0f / x);
                            case TB200_T_SIGMOID: TB200_UNARY(1.0f / (1.0f + expf(-x)));
                            case TB200_T_ROUND_BF16: TB200_UNARY(round_bf16(x));
                            case TB200_T_FMA:
#pragma unroll
                                for (int e = 0; e < kV; e++) r[e] = fmaf(va[e], vb[e], vc[e]);
                                break;
                            case TB200_T_SELECT:
#pragma unroll
                                for (int e = 0; e < kV; e++) r[e] = va[e] > 0.0f ? vb[e] : vc[e];
                                break;
                            default: break;
                        }
                    }
                    if (phase < A.phases) {
#pragma unroll
                        for (int f = 0; f < kMaxF; f++)
                            if (f < A.d.n_folds && A.d.folds[f].phase == phase) {
                                const float *y = val[A.d.folds[f].term];
                                const int kind = A.d.folds[f].kind;
#pragma unroll
                                for (int e = 0; e < kV; e++)
                                    if (i0 + e < n) fold_lift(kind, st[f], y[e]);
                            }
                    } else {
                        for (int o = 0; o < A.d.n_outputs; o++)
                            if (A.d.outputs[o].from == 0) store_output(A, o, row, i0, val[A.d.outputs[o].index]);
                    }
                }
            }
            if (phase == A.phases) break;
            // the partial states of a row meet: lanes first (earlier elements on the left), then warps
#pragma unroll
            for (int f = 0; f < kMaxF; f++)
                if (f < A.d.n_folds && A.d.folds[f].phase == phase) {
                    const int kind = A.d.folds[f].kind;
                    for (int offset = 1; offset < min(tpr, 32); offset <<= 1) {
                        const State other = shuffle_xor(st[f], offset);
                        if ((tid & offset) == 0) fold_merge(kind, st[f], other);
                        else { State mine = st[f]; st[f] = other; fold_merge(kind, st[f], mine); }
                    }
                    if (warps_per_row > 1 && (tid & 31) == 0) xchg[tid >> 5][f] = st[f];
                }
            if (warps_per_row > 1) {
                __syncthreads();
#pragma unroll
                for (int f = 0; f < kMaxF; f++)
                    if (f < A.d.n_folds && A.d.folds[f].phase == phase) {
                        const int kind = A.d.folds[f].kind;
                        State total = xchg[group * warps_per_row][f];
                        for (int w = 1; w < warps_per_row; w++) fold_merge(kind, total, xchg[group * warps_per_row + w][f]);
                        st[f] = total;
                    }
                __syncthreads();
            }
#pragma unroll
            for (int f = 0; f < kMaxF; f++)
                if (f < A.d.n_folds && A.d.folds[f].phase == phase) fold_observe(A.d.folds[f].kind, st[f], obs[f][0], obs[f][1]);
        }
        if (active && t == 0)
            for (int o = 0; o < A.d.n_outputs; o++) {
                const tb200_group_output out = A.d.outputs[o];
                if (out.from == 0) continue;
                const float x = obs[out.index][out.from - 1];
                if (out.dtype == TB200_BF16) static_cast<__nv_bfloat16 *>(A.out[o])[row] = __float2bfloat16_rn(x);
                else static_cast<float *>(A.out[o])[row] = x;
            }
    }
}

int arity(int op) {
    switch (op) {
        case TB200_T_LOAD: case TB200_T_LIT: case TB200_T_INDEX: case TB200_T_STAT: case TB200_T_STAT2: return 0;
        case TB200_T_ADD: case TB200_T_SUB: case TB200_T_MUL: case TB200_T_DIV: case TB200_T_MAX: case TB200_T_MIN: return 2;
        case TB200_T_FMA: case TB200_T_SELECT: return 3;
        default: return op >= TB200_T_NEG && op <= TB200_T_ROUND_BF16 ? 1 : -1;
    }
}

// Fills the phase masks; returns a status.
int plan_generic(const tb200_group_desc *d, GenericArgs *A) {
    if (!d) return TB200_ERR_NULL;
    if (d->n < 0 || d->rows < 0) return TB200_ERR_SHAPE;
    if (d->n_inputs < 0 || d->n_inputs > TB200_GROUP_MAX_INPUTS || d->n_terms < 0 || d->n_terms > kMaxT || d->n_folds < 0 ||
        d->n_folds > kMaxF || d->n_outputs < 1 || d->n_outputs > TB200_GROUP_MAX_OUTPUTS)
        return TB200_ERR_UNSUPPORTED;
    for (int i = 0; i < d->n_inputs; i++) {
        const tb200_group_input &in = d->inputs[i];
        if (in.shape < TB200_SHAPE_FULL || in.shape > TB200_SHAPE_SCALAR) return TB200_ERR_UNSUPPORTED;
        if (in.dtype != TB200_F32 && in.dtype != TB200_BF16) return TB200_ERR_DTYPE;
        if (in.shape == TB200_SHAPE_FULL && in.ld < d->n) return TB200_ERR_SHAPE;
    }
    int phases = 0;
    for (int f = 0; f < d->n_folds; f++) {
        const tb200_fold &fo = d->folds[f];
        if (fo.kind < TB200_FOLD_SUM || fo.kind > TB200_FOLD_MEANVAR) return TB200_ERR_UNSUPPORTED;
        if (fo.term < 0 || fo.term >= d->n_terms || fo.phase < 0 || fo.phase >= kMaxF) return TB200_ERR_SHAPE;
        phases = fo.phase + 1 > phases ? fo.phase + 1 : phases;
    }
    for (int k = 0; k < d->n_terms; k++) {
        const tb200_term &T = d->terms[k];
        const int ar = arity(T.op);
        if (ar < 0) return TB200_ERR_UNSUPPORTED;
        const int args[3] = {T.a, T.b, T.c};
        for (int j = 0; j < ar; j++)
            if (args[j] < 0 || args[j] >= k) return TB200_ERR_SHAPE;   // arguments come before uses
        if (T.op == TB200_T_LOAD && (T.a < 0 || T.a >= d->n_inputs)) return TB200_ERR_SHAPE;
        if ((T.op == TB200_T_STAT || T.op == TB200_T_STAT2) && (T.a < 0 || T.a >= d->n_folds)) return TB200_ERR_SHAPE;
        if (T.op == TB200_T_STAT2 && d->folds[T.a].kind != TB200_FOLD_MEANVAR) return TB200_ERR_SHAPE;
    }
    for (int o = 0; o < d->n_outputs; o++) {
        const tb200_group_output &out = d->outputs[o];
        if (out.dtype != TB200_F32 && out.dtype != TB200_BF16) return TB200_ERR_DTYPE;
        if (out.from == 0) {
            if (out.index < 0 || out.index >= d->n_terms) return TB200_ERR_SHAPE;
            if (out.ld < d->n) return TB200_ERR_SHAPE;
        } else if (out.from == 1 || out.from == 2) {
            if (out.index < 0 || out.index >= d->n_folds) return TB200_ERR_SHAPE;
            if (out.from == 2 && d->folds[out.index].kind != TB200_FOLD_MEANVAR) return TB200_ERR_SHAPE;
        } else {
            return TB200_ERR_UNSUPPORTED;
        }
    }
    // what each phase evaluates: everything its folds (or, last, the outputs) reach, stopping at statistics,
    // which must come from an earlier phase
    for (int p = 0; p <= phases; p++) {
        unsigned long long need = 0;
        for (int f = 0; f < d->n_folds; f++)
            if (p < phases && d->folds[f].phase == p) need |= 1ull << d->folds[f].term;
        if (p == phases)
            for (int o = 0; o < d->n_outputs; o++)
                if (d->outputs[o].from == 0) need |= 1ull << d->outputs[o].index;
        for (int k = d->n_terms - 1; k >= 0; k--) {
            if (!((need >> k) & 1ull)) continue;
            const tb200_term &T = d->terms[k];
            const int ar = arity(T.op);
            const int args[3] = {T.a, T.b, T.c};
            for (int j = 0; j < ar; j++) need |= 1ull << args[j];
            if ((T.op == TB200_T_STAT || T.op == TB200_T_STAT2) && d->folds[T.a].phase >= p) return TB200_ERR_SHAPE;
        }
        if (A) A->need[p] = need;
    }
    if (A) A->phases = phases;
    return TB200_OK;
}

}  // namespace

int group_phases(const tb200_group_desc *d, unsigned long long *need, int *phases) {
    GenericArgs A{};
    const int st = plan_generic(d, &A);
    if (st) return st;
    for (int p = 0; p <= A.phases; p++) need[p] = A.need[p];
    *phases = A.phases;
    return TB200_OK;
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_rowreduce_generic_check(const tb200_group_desc *d) { return plan_generic(d, nullptr); }

extern "C" int tb200_rowreduce_generic(const tb200_group_desc *d, const void *const *inputs, void *const *outputs,
                                       void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    GenericArgs A{};
    int st = plan_generic(d, &A);
    if (st) return st;
    if (d->n == 0 || d->rows == 0) return TB200_OK;
    if (!outputs || (d->n_inputs > 0 && !inputs)) return TB200_ERR_NULL;
    A.d = *d;
    for (int i = 0; i < d->n_inputs; i++) {
        if (!inputs[i]) return TB200_ERR_NULL;
        const size_t es = dtype_size(d->inputs[i].dtype);
        if (!aligned_to(inputs[i], es)) return TB200_ERR_ALIGN;
        A.in[i] = inputs[i];
        const bool rows_wide = d->inputs[i].shape == TB200_SHAPE_FULL ? d->inputs[i].ld % kV == 0 : true;
        if ((d->inputs[i].shape == TB200_SHAPE_FULL || d->inputs[i].shape == TB200_SHAPE_ALONG) && rows_wide &&
            aligned_to(inputs[i], es * kV))
            A.vec_in |= 1u << i;
    }
    for (int o = 0; o < d->n_outputs; o++) {
        if (!outputs[o]) return TB200_ERR_NULL;
        const size_t es = dtype_size(d->outputs[o].dtype);
        if (!aligned_to(outputs[o], es)) return TB200_ERR_ALIGN;
        A.out[o] = outputs[o];
        if (d->outputs[o].from == 0 && d->outputs[o].ld % kV == 0 && aligned_to(outputs[o], es * kV)) A.vec_out |= 1u << o;
    }
    DeviceInfo dev;
    if ((st = current_device(&dev))) return st;
    int tpr = next_pow2(ceil_div(d->n, kV));
    tpr = tpr < 8 ? 8 : tpr > kThreads ? kThreads : tpr;
    A.tpr = tpr;
    const int64_t blocks = ceil_div(d->rows, kThreads / tpr);
    const int64_t cap = static_cast<int64_t>(dev.sms) * 8;
    generic_rows_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), kThreads, 0, stream>>>(A);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}
