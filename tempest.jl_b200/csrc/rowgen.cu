// Kernel generator for map -> fold row groups: the descriptor compiled to its own sm_100a kernel.
//
// The term interpreter of generic.cu pays instructions for every term of every element.  Here the same
// descriptor is turned into CUDA source -- terms as straight-line Float32 code, folds as the states their
// kinds need, the extents, element types, alignment and schedule as compile-time constants -- compiled by
// NVRTC for sm_100a, cached by descriptor, and launched through the driver API.  This is what the
// reference's generator does with a group (ext/cuTileExt/build.jl:138-286 emits a kernel per `unsplit` row
// group, ext/cuTileExt/cache.jl:59 compiles and caches it); the schedule is the named row kernels':
//   * a row belongs to 8..256 threads; each thread owns `K` chunks of `V` consecutive elements, V sized for
//     128-bit accesses;
//   * when the row fits in registers it is read once (streaming loads) and stays there through every phase
//     ("resident", ext/cuTileExt/cuTileExt.jl:438-444); vectors along the row (a LayerNorm weight) are read
//     where they are used, from L1, which costs fewer registers than holding them; longer rows are re-read
//     per phase through L1/L2;
//   * log-sum-exp takes the maximum of a chunk first and rebases once per chunk; mean/variance forms each
//     chunk's (count, mean, centred squares) and merges it with Chan's rule -- the fold algebra of
//     src/Compiler/IR/folds.jl:143-198 applied chunk-wise;
//   * partial states meet through shuffles, then shared memory.
// NVRTC is loaded with dlopen when first needed; without it the entries return TB200_ERR_UNSUPPORTED and the
// interpreter remains.
#include <cuda.h>
#include <dlfcn.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "generic.cuh"

namespace tb200 {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxF = TB200_GROUP_MAX_FOLDS;

struct Schedule {
    int V, tpr, K, rpb;
    bool resident, unrolled, whole_chunks, whole_elems;
    unsigned vec_in, vec_out;
    int phases;
    unsigned long long need[kMaxF + 1];
};

struct LaunchParams {
    const void *in[TB200_GROUP_MAX_INPUTS];
    void *out[TB200_GROUP_MAX_OUTPUTS];
    long long rows;
    long long ld_in[TB200_GROUP_MAX_INPUTS];
    long long ld_out[TB200_GROUP_MAX_OUTPUTS];
};

// ------------------------------------------------------------------ source emission ----

struct Emitter {
    std::string s;
    void line(int indent, const std::string &text) {
        s.append(static_cast<size_t>(indent) * 4, ' ');
        s += text;
        s += '\n';
    }
};

std::string num(long long v) { return std::to_string(v); }
std::string fbits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    char buf[40];
    snprintf(buf, sizeof buf, "__uint_as_float(0x%08xu)", u);
    return buf;
}

int term_arity(int op) {
    if (op <= TB200_T_STAT2 || op == TB200_T_ROW_INDEX || op == TB200_T_STATE) return 0;
    if (op <= TB200_T_MIN) return 2;
    if (op == TB200_T_FMA || op == TB200_T_SELECT) return 3;
    return 1;
}

const char *fold_identity(int kind) {
    switch (kind) {
        case TB200_FOLD_MAX: case TB200_FOLD_LOGSUMEXP: return "NEG_INF";
        case TB200_FOLD_MIN: return "POS_INF";
        case TB200_FOLD_PROD: return "1.0f";
        default: return "0.0f";
    }
}

// merges state (oa, ob, oc) -- the later elements -- into (a, b, c)
void emit_merge(Emitter &E, int ind, int kind, const std::string &a, const std::string &b, const std::string &c,
                const std::string &oa, const std::string &ob, const std::string &oc) {
    switch (kind) {
        case TB200_FOLD_SUM: E.line(ind, a + " += " + oa + ";"); break;
        case TB200_FOLD_MAX: E.line(ind, a + " = fmaxf(" + a + ", " + oa + ");"); break;
        case TB200_FOLD_MIN: E.line(ind, a + " = fminf(" + a + ", " + oa + ");"); break;
        case TB200_FOLD_PROD: E.line(ind, a + " *= " + oa + ";"); break;
        case TB200_FOLD_LOGSUMEXP:
            E.line(ind, "{ const float m_ = fmaxf(" + a + ", " + oa + ");");
            E.line(ind, "  if (m_ > NEG_INF) " + b + " = " + b + " * __expf(" + a + " - m_) + " + ob + " * __expf(" + oa + " - m_);");
            E.line(ind, "  " + a + " = m_; }");
            break;
        default:
            E.line(ind, "{ const float n_ = " + a + " + " + oa + ";");
            E.line(ind, "  if (n_ > 0.0f) { const float d_ = " + ob + " - " + b + ", w_ = __fdividef(" + oa + ", n_);");
            E.line(ind, "    " + c + " = " + c + " + " + oc + " + d_ * d_ * " + a + " * w_; " + b + " = fmaf(d_, w_, " + b + "); }");
            E.line(ind, "  " + a + " = n_; }");
    }
}

std::string term_expr(const tb200_group_desc &d, int k, const std::string &chunk_index) {
    const tb200_term &T = d.terms[k];
    auto t = [](int i) { return "t" + num(i); };
    switch (T.op) {
        case TB200_T_LOAD: {
            const int shape = d.inputs[T.a].shape;
            if (shape == TB200_SHAPE_PER_ROW) return "pr" + num(T.a);
            if (shape == TB200_SHAPE_SCALAR) return "sc" + num(T.a);
            return "c" + num(T.a) + (shape == TB200_SHAPE_FULL ? chunk_index : "") + "[e]";
        }
        case TB200_T_LIT: return fbits(T.imm);
        case TB200_T_INDEX: return "(float)(i0 + e)";
        case TB200_T_STAT: return "s" + num(T.a);
        case TB200_T_STAT2: return "s" + num(T.a) + "b";
        case TB200_T_ADD: return t(T.a) + " + " + t(T.b);
        case TB200_T_SUB: return t(T.a) + " - " + t(T.b);
        case TB200_T_MUL: return t(T.a) + " * " + t(T.b);
        case TB200_T_DIV: return t(T.a) + " / " + t(T.b);
        case TB200_T_MAX: return "fmaxf(" + t(T.a) + ", " + t(T.b) + ")";
        case TB200_T_MIN: return "fminf(" + t(T.a) + ", " + t(T.b) + ")";
        case TB200_T_NEG: return "-" + t(T.a);
        case TB200_T_EXP:
            if (d.terms[T.a].op == TB200_T_SUB) return "exp_diff(" + t(d.terms[T.a].a) + ", " + t(d.terms[T.a].b) + ")";
            return "__expf(" + t(T.a) + ")";
        case TB200_T_LOG: return "logf(" + t(T.a) + ")";
        case TB200_T_TANH: return "tanhf(" + t(T.a) + ")";
        case TB200_T_SQRT: return "sqrtf(" + t(T.a) + ")";
        case TB200_T_RSQRT: return "rsqrtf(" + t(T.a) + ")";
        case TB200_T_ABS: return "fabsf(" + t(T.a) + ")";
        case TB200_T_ABS2: return t(T.a) + " * " + t(T.a);
        case TB200_T_RECIP: return "1.0f / " + t(T.a);
        case TB200_T_SIGMOID: return "1.0f / (1.0f + __expf(-" + t(T.a) + "))";
        case TB200_T_FMA: return "fmaf(" + t(T.a) + ", " + t(T.b) + ", " + t(T.c) + ")";
        case TB200_T_SELECT: return "(" + t(T.a) + " > 0.0f ? " + t(T.b) + " : " + t(T.c) + ")";
        case TB200_T_ROUND_BF16: return "bf2f(f2bf(" + t(T.a) + "))";
        case TB200_T_STATE: return "st" + num(T.a);
        case TB200_T_ROW_INDEX: return "(float)row";
        default: return "0.0f";
    }
}

// loads one chunk of input `i` (shape full or along) into `dst`[0..V)
void emit_chunk_load(Emitter &E, int ind, const tb200_group_desc &d, const Schedule &S, int i, const std::string &dst,
                     bool streaming) {
    const bool bf = d.inputs[i].dtype == TB200_BF16;
    const bool full = d.inputs[i].shape == TB200_SHAPE_FULL;
    const std::string type = bf ? "u16" : "float";
    const std::string base = std::string("((const ") + type + " *)p.in[" + num(i) + "] + " +
                             (full ? "row * p.ld_in[" + num(i) + "] + " : "") + "i0)";
    const std::string ld = streaming && full ? "__ldcs" : "__ldg";
    if ((S.vec_in >> i) & 1u) {
        if (bf) {
            if (S.V == 8) {
                E.line(ind, "{ const uint4 w_ = " + ld + "((const uint4 *)" + base + ");");
                E.line(ind, "  " + dst + "[0] = bf_lo(w_.x); " + dst + "[1] = bf_hi(w_.x); " + dst + "[2] = bf_lo(w_.y); " + dst +
                                "[3] = bf_hi(w_.y);");
                E.line(ind, "  " + dst + "[4] = bf_lo(w_.z); " + dst + "[5] = bf_hi(w_.z); " + dst + "[6] = bf_lo(w_.w); " + dst +
                                "[7] = bf_hi(w_.w); }");
            } else {
                E.line(ind, "{ const uint2 w_ = " + ld + "((const uint2 *)" + base + ");");
                E.line(ind, "  " + dst + "[0] = bf_lo(w_.x); " + dst + "[1] = bf_hi(w_.x); " + dst + "[2] = bf_lo(w_.y); " + dst +
                                "[3] = bf_hi(w_.y); }");
            }
        } else {
            for (int q = 0; q < S.V / 4; q++) {
                E.line(ind, "{ const float4 w_ = " + ld + "((const float4 *)" + base + " + " + num(q) + ");");
                E.line(ind, "  " + dst + "[" + num(4 * q) + "] = w_.x; " + dst + "[" + num(4 * q + 1) + "] = w_.y; " + dst + "[" +
                                num(4 * q + 2) + "] = w_.z; " + dst + "[" + num(4 * q + 3) + "] = w_.w; }");
            }
        }
        return;
    }
    E.line(ind, "#pragma unroll");
    E.line(ind, "for (int e = 0; e < V; e++) {");
    const std::string value = bf ? "bf2f(" + base + "[e])" : ld + "(" + base + " + e)";
    if (S.whole_elems) E.line(ind + 1, dst + "[e] = " + value + ";");
    else E.line(ind + 1, dst + "[e] = i0 + e < N ? " + value + " : 0.0f;");
    E.line(ind, "}");
}

void emit_chunk_store(Emitter &E, int ind, const tb200_group_desc &d, const Schedule &S, int o, const std::string &src) {
    const bool bf = d.outputs[o].dtype == TB200_BF16;
    const std::string type = bf ? "u16" : "float";
    const std::string base = std::string("((") + type + " *)p.out[" + num(o) + "] + row * p.ld_out[" + num(o) + "] + i0)";
    if ((S.vec_out >> o) & 1u) {
        if (bf) {
            auto pack = [&](int a) { return "pack2(" + src + "[" + num(a) + "], " + src + "[" + num(a + 1) + "])"; };
            if (S.V == 8)
                E.line(ind, "__stcs((uint4 *)" + base + ", make_uint4(" + pack(0) + ", " + pack(2) + ", " + pack(4) + ", " + pack(6) + "));");
            else
                E.line(ind, "__stcs((uint2 *)" + base + ", make_uint2(" + pack(0) + ", " + pack(2) + "));");
        } else {
            for (int q = 0; q < S.V / 4; q++)
                E.line(ind, "__stcs((float4 *)" + base + " + " + num(q) + ", make_float4(" + src + "[" + num(4 * q) + "], " + src + "[" +
                                num(4 * q + 1) + "], " + src + "[" + num(4 * q + 2) + "], " + src + "[" + num(4 * q + 3) + "]));");
        }
        return;
    }
    E.line(ind, "#pragma unroll");
    E.line(ind, "for (int e = 0; e < V; e++)");
    const std::string guard = S.whole_elems ? "" : "if (i0 + e < N) ";
    if (bf) E.line(ind + 1, guard + base + "[e] = (u16)f2bf(" + src + "[e]);");
    else E.line(ind + 1, guard + base + "[e] = " + src + "[e];");
}

std::string generate(const tb200_group_desc &d, const Schedule &S) {
    Emitter E;
    E.line(0, "typedef unsigned short u16; typedef unsigned int u32; typedef long long i64;");
    E.line(0, "struct Params { const void *in[8]; void *out[8]; i64 rows; i64 ld_in[8]; i64 ld_out[8]; };");
    E.line(0, "#define NEG_INF __uint_as_float(0xff800000u)");
    E.line(0, "#define POS_INF __uint_as_float(0x7f800000u)");
    E.line(0, "#define LOG2E 1.4426950408889634f");
    E.line(0, "static __device__ __forceinline__ float ex2(float x) { float y; asm(\"ex2.approx.ftz.f32 %0, %1;\" : \"=f\"(y) : \"f\"(x)); return y; }");
    E.line(0, "// exp(a - b) as one multiply-add and one ex2: b * LOG2E is hoisted when b is a row statistic");
    E.line(0, "static __device__ __forceinline__ float exp_diff(float a, float b) { return ex2(fmaf(a, LOG2E, -(b * LOG2E))); }");
    E.line(0, "static __device__ __forceinline__ float bf2f(u32 h) { return __uint_as_float(h << 16); }");
    E.line(0, "static __device__ __forceinline__ float bf_lo(u32 w) { return __uint_as_float(w << 16); }");
    E.line(0, "static __device__ __forceinline__ float bf_hi(u32 w) { return __uint_as_float(w & 0xffff0000u); }");
    E.line(0, "static __device__ __forceinline__ u32 f2bf(float f) { u16 r; asm(\"cvt.rn.bf16.f32 %0, %1;\" : \"=h\"(r) : \"f\"(f)); return r; }");
    E.line(0, "static __device__ __forceinline__ u32 pack2(float lo, float hi) { u32 r; asm(\"cvt.rn.bf16x2.f32 %0, %1, %2;\" : \"=r\"(r) : \"f\"(hi), \"f\"(lo)); return r; }");
    E.line(0, "constexpr int N = " + num(d.n) + ", V = " + num(S.V) + ", TPR = " + num(S.tpr) + ", K = " + num(S.K) +
                  ", RPB = " + num(S.rpb) + ";");
    E.line(0, "extern \"C\" __global__ void __launch_bounds__(" + num(kThreads) + ") tb200_group(const Params p) {");
    E.line(1, "const int tid = threadIdx.x, t = tid % TPR, g = tid / TPR;");
    const int warps_per_row = S.tpr / 32;
    if (warps_per_row > 1 && d.n_folds > 0) E.line(1, "__shared__ float xch[" + num(kThreads / 32) + "][" + num(3 * d.n_folds) + "];");

    // which inputs any phase loads
    unsigned long long any = 0;
    for (int p = 0; p <= S.phases; p++) any |= S.need[p];
    bool used[TB200_GROUP_MAX_INPUTS] = {};
    for (int k = 0; k < d.n_terms; k++)
        if (((any >> k) & 1ull) && d.terms[k].op == TB200_T_LOAD) used[d.terms[k].a] = true;

    const std::string unroll = S.unrolled ? "#pragma unroll" : "#pragma unroll 1";
    auto chunk_guard_open = [&](int ind) {
        E.line(ind, "const int i0 = (k * TPR + t) * V;");
        if (!S.whole_chunks) E.line(ind, "if (i0 < N) {");
    };
    auto chunk_guard_close = [&](int ind) {
        if (!S.whole_chunks) E.line(ind, "}");
    };

    for (int i = 0; i < d.n_inputs; i++) {
        if (!used[i]) continue;
        if (d.inputs[i].shape == TB200_SHAPE_SCALAR) {
            E.line(1, std::string("const float sc") + num(i) + " = " +
                          (d.inputs[i].dtype == TB200_BF16 ? "bf2f(((const u16 *)p.in[" + num(i) + "])[0]);"
                                                           : "((const float *)p.in[" + num(i) + "])[0];"));
        }
    }

    E.line(1, "for (i64 base = (i64)blockIdx.x * RPB; base < p.rows; base += (i64)gridDim.x * RPB) {");
    E.line(2, "const i64 row = base + g;");
    E.line(2, "const bool active = row < p.rows;");
    for (int i = 0; i < d.n_inputs; i++) {
        if (!used[i]) continue;
        if (d.inputs[i].shape == TB200_SHAPE_PER_ROW) {
            E.line(2, std::string("float pr") + num(i) + " = 0.0f;");
            E.line(2, std::string("if (active) pr") + num(i) + " = " +
                          (d.inputs[i].dtype == TB200_BF16 ? "bf2f(((const u16 *)p.in[" + num(i) + "])[row]);"
                                                           : "((const float *)p.in[" + num(i) + "])[row];"));
        } else if (d.inputs[i].shape == TB200_SHAPE_FULL && S.resident) {
            E.line(2, "float c" + num(i) + "[K][V];");
            E.line(2, "if (active) {");
            E.line(3, unroll);
            E.line(3, "for (int k = 0; k < K; k++) {");
            chunk_guard_open(4);
            emit_chunk_load(E, S.whole_chunks ? 4 : 5, d, S, i, "c" + num(i) + "[k]", true);
            chunk_guard_close(4);
            E.line(3, "}");
            E.line(2, "}");
        }
    }

    for (int p = 0; p <= S.phases; p++) {
        const bool last = p == S.phases;
        const unsigned long long need = S.need[p];
        E.line(2, std::string("// ") + (last ? "outputs" : "folds of phase " + num(p)));
        for (int f = 0; f < d.n_folds; f++)
            if (!last && d.folds[f].phase == p) {
                const std::string n = "f" + num(f);
                E.line(2, "float " + n + "a = " + fold_identity(d.folds[f].kind) + ", " + n + "b = 0.0f, " + n + "c = 0.0f;");
            }
        bool any_full_output = false;
        for (int o = 0; o < d.n_outputs; o++) any_full_output |= d.outputs[o].from == 0;
        if (last && !any_full_output) break;
        E.line(2, "if (active) {");
        E.line(3, unroll);
        E.line(3, "for (int k = 0; k < K; k++) {");
        chunk_guard_open(4);
        const int ind = S.whole_chunks ? 4 : 5;
        // inputs of this phase
        for (int i = 0; i < d.n_inputs; i++) {
            bool here = false;
            for (int k = 0; k < d.n_terms; k++)
                if (((need >> k) & 1ull) && d.terms[k].op == TB200_T_LOAD && d.terms[k].a == i) here = true;
            if (!here) continue;
            const bool along = d.inputs[i].shape == TB200_SHAPE_ALONG;
            if (along || (d.inputs[i].shape == TB200_SHAPE_FULL && !S.resident)) {
                E.line(ind, "float c" + num(i) + "[V];");
                emit_chunk_load(E, ind, d, S, i, "c" + num(i), false);
            }
        }
        const std::string chunk_index = S.resident ? "[k]" : "";
        if (last) {
            for (int o = 0; o < d.n_outputs; o++)
                if (d.outputs[o].from == 0) E.line(ind, "float o" + num(o) + "[V];");
        } else {
            for (int f = 0; f < d.n_folds; f++)
                if (d.folds[f].phase == p) E.line(ind, "float y" + num(f) + "[V];");
        }
        E.line(ind, "#pragma unroll");
        E.line(ind, "for (int e = 0; e < V; e++) {");
        for (int k = 0; k < d.n_terms; k++)
            if ((need >> k) & 1ull) E.line(ind + 1, "const float t" + num(k) + " = " + term_expr(d, k, chunk_index) + ";");
        if (last) {
            for (int o = 0; o < d.n_outputs; o++)
                if (d.outputs[o].from == 0) E.line(ind + 1, "o" + num(o) + "[e] = t" + num(d.outputs[o].index) + ";");
        } else {
            for (int f = 0; f < d.n_folds; f++)
                if (d.folds[f].phase == p) {
                    const std::string v = "t" + num(d.folds[f].term);
                    if (S.whole_elems || d.folds[f].kind == TB200_FOLD_MEANVAR) E.line(ind + 1, "y" + num(f) + "[e] = " + v + ";");
                    else E.line(ind + 1, "y" + num(f) + "[e] = i0 + e < N ? " + v + " : " + fold_identity(d.folds[f].kind) + ";");
                }
        }
        E.line(ind, "}");
        if (last) {
            for (int o = 0; o < d.n_outputs; o++)
                if (d.outputs[o].from == 0) emit_chunk_store(E, ind, d, S, o, "o" + num(o));
        } else {
            for (int f = 0; f < d.n_folds; f++) {
                if (d.folds[f].phase != p) continue;
                const std::string n = "f" + num(f), y = "y" + num(f);
                const int kind = d.folds[f].kind;
                if (kind == TB200_FOLD_LOGSUMEXP) {
                    // the chunk's maximum first, one rebase per chunk
                    E.line(ind, "{ float cm_ = " + y + "[0];");
                    E.line(ind, "#pragma unroll");
                    E.line(ind, "  for (int e = 1; e < V; e++) cm_ = fmaxf(cm_, " + y + "[e]);");
                    E.line(ind, "  const float m_ = fmaxf(" + n + "a, cm_);");
                    E.line(ind, "  if (m_ > NEG_INF) { float cs_ = 0.0f;");
                    E.line(ind, "#pragma unroll");
                    E.line(ind, "    for (int e = 0; e < V; e++) cs_ += exp_diff(" + y + "[e], m_);");
                    E.line(ind, "    " + n + "b = " + n + "b * exp_diff(" + n + "a, m_) + cs_; }");
                    E.line(ind, "  " + n + "a = m_; }");
                } else if (kind == TB200_FOLD_MEANVAR) {
                    const std::string valid = S.whole_elems ? "" : "if (i0 + e < N) ";
                    E.line(ind, "{ float cn_ = 0.0f, cs_ = 0.0f;");
                    E.line(ind, "#pragma unroll");
                    E.line(ind, "  for (int e = 0; e < V; e++) " + valid + "{ cn_ += 1.0f; cs_ += " + y + "[e]; }");
                    E.line(ind, "  const float cmean_ = cs_ / cn_; float cq_ = 0.0f;");
                    E.line(ind, "#pragma unroll");
                    E.line(ind, "  for (int e = 0; e < V; e++) " + valid + "{ const float d_ = " + y + "[e] - cmean_; cq_ = fmaf(d_, d_, cq_); }");
                    emit_merge(E, ind + 1, kind, n + "a", n + "b", n + "c", "cn_", "cmean_", "cq_");
                    E.line(ind, "}");
                } else {
                    E.line(ind, "#pragma unroll");
                    E.line(ind, "for (int e = 0; e < V; e++) {");
                    emit_merge(E, ind + 1, kind, n + "a", n + "b", n + "c", y + "[e]", "0.0f", "0.0f");
                    E.line(ind, "}");
                }
            }
        }
        chunk_guard_close(4);
        E.line(3, "}");
        E.line(2, "}");
        if (last) break;
        // partial states meet
        const int lanes = S.tpr < 32 ? S.tpr : 32;
        for (int f = 0; f < d.n_folds; f++) {
            if (d.folds[f].phase != p) continue;
            const std::string n = "f" + num(f);
            const int kind = d.folds[f].kind;
            const bool wide = kind == TB200_FOLD_LOGSUMEXP || kind == TB200_FOLD_MEANVAR;
            for (int offset = 1; offset < lanes; offset <<= 1) {
                E.line(2, "{ float oa_ = __shfl_xor_sync(0xffffffffu, " + n + "a, " + num(offset) + "), ob_ = 0.0f, oc_ = 0.0f;");
                if (wide) E.line(2, "  ob_ = __shfl_xor_sync(0xffffffffu, " + n + "b, " + num(offset) + ");");
                if (kind == TB200_FOLD_MEANVAR) E.line(2, "  oc_ = __shfl_xor_sync(0xffffffffu, " + n + "c, " + num(offset) + ");");
                if (wide) {
                    // both lanes of a pair combine in the same order, so they agree bit for bit
                    E.line(2, "  if (tid & " + num(offset) + ") { float x_; x_ = " + n + "a; " + n + "a = oa_; oa_ = x_; x_ = " + n + "b; " + n +
                                  "b = ob_; ob_ = x_; x_ = " + n + "c; " + n + "c = oc_; oc_ = x_; }");
                }
                emit_merge(E, 3, kind, n + "a", n + "b", n + "c", "oa_", "ob_", "oc_");
                E.line(2, "}");
            }
        }
        if (warps_per_row > 1) {
            bool any_fold = false;
            for (int f = 0; f < d.n_folds; f++) any_fold |= d.folds[f].phase == p;
            if (any_fold) {
                E.line(2, "if ((tid & 31) == 0) {");
                for (int f = 0; f < d.n_folds; f++)
                    if (d.folds[f].phase == p)
                        E.line(3, "xch[tid >> 5][" + num(3 * f) + "] = f" + num(f) + "a; xch[tid >> 5][" + num(3 * f + 1) + "] = f" + num(f) +
                                      "b; xch[tid >> 5][" + num(3 * f + 2) + "] = f" + num(f) + "c;");
                E.line(2, "}");
                E.line(2, "__syncthreads();");
                for (int f = 0; f < d.n_folds; f++) {
                    if (d.folds[f].phase != p) continue;
                    const std::string n = "f" + num(f);
                    const std::string w0 = "xch[g * " + num(warps_per_row) + "]";
                    E.line(2, n + "a = " + w0 + "[" + num(3 * f) + "]; " + n + "b = " + w0 + "[" + num(3 * f + 1) + "]; " + n + "c = " + w0 + "[" +
                                  num(3 * f + 2) + "];");
                    E.line(2, "#pragma unroll");
                    E.line(2, "for (int w = 1; w < " + num(warps_per_row) + "; w++) {");
                    const std::string ww = "xch[g * " + num(warps_per_row) + " + w]";
                    emit_merge(E, 3, d.folds[f].kind, n + "a", n + "b", n + "c", ww + "[" + num(3 * f) + "]", ww + "[" + num(3 * f + 1) + "]",
                               ww + "[" + num(3 * f + 2) + "]");
                    E.line(2, "}");
                }
                E.line(2, "__syncthreads();");
            }
        }
        for (int f = 0; f < d.n_folds; f++) {
            if (d.folds[f].phase != p) continue;
            const std::string n = "f" + num(f), s = "s" + num(f);
            switch (d.folds[f].kind) {
                case TB200_FOLD_LOGSUMEXP:
                    E.line(2, "const float " + s + " = " + n + "a > NEG_INF ? " + n + "a + logf(" + n + "b) : NEG_INF;");
                    break;
                case TB200_FOLD_MEANVAR:
                    E.line(2, "const float " + s + " = " + n + "b, " + s + "b = " + n + "a > 0.0f ? " + n + "c / " + n + "a : 0.0f;");
                    break;
                default: E.line(2, "const float " + s + " = " + n + "a;");
            }
            E.line(2, "(void)" + s + ";");
        }
    }
    bool any_stat_output = false;
    for (int o = 0; o < d.n_outputs; o++) any_stat_output |= d.outputs[o].from != 0;
    if (any_stat_output) {
        E.line(2, "if (active && t == 0) {");
        for (int o = 0; o < d.n_outputs; o++) {
            if (d.outputs[o].from == 0) continue;
            const std::string v = "s" + num(d.outputs[o].index) + (d.outputs[o].from == 2 ? "b" : "");
            if (d.outputs[o].dtype == TB200_BF16) E.line(3, "((u16 *)p.out[" + num(o) + "])[row] = (u16)f2bf(" + v + ");");
            else E.line(3, "((float *)p.out[" + num(o) + "])[row] = " + v + ";");
        }
        E.line(2, "}");
    }
    E.line(1, "}");
    E.line(0, "}");
    return E.s;
}

// ------------------------------------------------------------------------ schedule ----

int make_schedule(const tb200_group_desc *d, unsigned vec_in, unsigned vec_out, Schedule *S) {
    int st = group_phases(d, S->need, &S->phases);
    if (st) return st;
    if (d->n <= 0 || d->n > (1ll << 30)) return d->n == 0 ? TB200_OK : TB200_ERR_UNSUPPORTED;
    bool any_f32 = false;
    int held = 0;   // full-shape inputs: what a resident schedule keeps in registers
    for (int i = 0; i < d->n_inputs; i++)
        if (d->inputs[i].shape == TB200_SHAPE_FULL || d->inputs[i].shape == TB200_SHAPE_ALONG) {
            any_f32 |= d->inputs[i].dtype == TB200_F32;
            held += d->inputs[i].shape == TB200_SHAPE_FULL;
        }
    for (int o = 0; o < d->n_outputs; o++)
        if (d->outputs[o].from == 0) any_f32 |= d->outputs[o].dtype == TB200_F32;
    S->V = any_f32 ? 4 : 8;
    // four chunks per thread where the row allows: four independent 128-bit loads in flight per thread is what
    // keeps HBM busy at the occupancy these kernels reach (two left BFloat16 rows at half the rate)
    int tpr = next_pow2(ceil_div(d->n, static_cast<int64_t>(S->V) * 4));
    S->tpr = tpr < 8 ? 8 : tpr > kThreads ? kThreads : tpr;
    S->K = static_cast<int>(ceil_div(d->n, static_cast<int64_t>(S->tpr) * S->V));
    S->rpb = kThreads / S->tpr;
    S->whole_elems = d->n % S->V == 0;
    S->whole_chunks = d->n % (static_cast<int64_t>(S->tpr) * S->V) == 0;
    S->resident = held * S->K * S->V <= 96 && S->K <= 16;
    S->unrolled = S->K <= 16;
    // 128-bit accesses need whole elements' worth of rows as well as what the caller checked
    S->vec_in = S->whole_elems ? vec_in : 0;
    S->vec_out = S->whole_elems ? vec_out : 0;
    return TB200_OK;
}

// ---------------------------------------------------------------------- NVRTC, driver ----

struct Nvrtc {
    void *handle = nullptr;
    int (*create)(void **, const char *, const char *, int, const char *const *, const char *const *) = nullptr;
    int (*compile)(void *, int, const char *const *) = nullptr;
    int (*cubin_size)(void *, size_t *) = nullptr;
    int (*cubin)(void *, char *) = nullptr;
    int (*log_size)(void *, size_t *) = nullptr;
    int (*log)(void *, char *) = nullptr;
    int (*destroy)(void **) = nullptr;
    bool ok = false;
};

Nvrtc &nvrtc() {
    static Nvrtc n;
    static std::once_flag once;
    std::call_once(once, [] {
        const char *names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                               "/usr/local/cuda/lib64/libnvrtc.so"};
        for (const char *name : names)
            if ((n.handle = dlopen(name, RTLD_NOW | RTLD_LOCAL))) break;
        if (!n.handle) return;
        auto sym = [&](const char *s) { return dlsym(n.handle, s); };
        n.create = reinterpret_cast<decltype(n.create)>(sym("nvrtcCreateProgram"));
        n.compile = reinterpret_cast<decltype(n.compile)>(sym("nvrtcCompileProgram"));
        n.cubin_size = reinterpret_cast<decltype(n.cubin_size)>(sym("nvrtcGetCUBINSize"));
        n.cubin = reinterpret_cast<decltype(n.cubin)>(sym("nvrtcGetCUBIN"));
        n.log_size = reinterpret_cast<decltype(n.log_size)>(sym("nvrtcGetProgramLogSize"));
        n.log = reinterpret_cast<decltype(n.log)>(sym("nvrtcGetProgramLog"));
        n.destroy = reinterpret_cast<decltype(n.destroy)>(sym("nvrtcDestroyProgram"));
        n.ok = n.create && n.compile && n.cubin_size && n.cubin && n.log_size && n.log && n.destroy;
    });
    return n;
}

struct Driver {
    CUresult (*module_load)(CUmodule *, const void *) = nullptr;
    CUresult (*get_function)(CUfunction *, CUmodule, const char *) = nullptr;
    CUresult (*launch)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void **,
                       void **) = nullptr;
    CUresult (*occupancy)(int *, CUfunction, int, size_t) = nullptr;
    bool ok = false;
};

int driver(Driver **out) {
    static Driver d;
    static std::mutex lock;
    std::lock_guard<std::mutex> hold(lock);
    if (!d.ok) {
        auto get = [](const char *name, void **fn) -> int {
            cudaDriverEntryPointQueryResult q;
            TB200_CUDA(cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q));
            return (*fn && q == cudaDriverEntryPointSuccess) ? TB200_OK : TB200_ERR_UNSUPPORTED;
        };
        int st;
        if ((st = get("cuModuleLoadData", reinterpret_cast<void **>(&d.module_load)))) return st;
        if ((st = get("cuModuleGetFunction", reinterpret_cast<void **>(&d.get_function)))) return st;
        if ((st = get("cuLaunchKernel", reinterpret_cast<void **>(&d.launch)))) return st;
        if ((st = get("cuOccupancyMaxActiveBlocksPerMultiprocessor", reinterpret_cast<void **>(&d.occupancy)))) return st;
        d.ok = true;
    }
    *out = &d;
    return TB200_OK;
}

struct Compiled {
    Schedule schedule;
    std::vector<char> cubin;
    CUfunction function[64] = {};
    int blocks_per_sm[64] = {};
};

std::mutex g_cache_lock;
std::map<std::string, Compiled *> g_cache;   // entries live as long as the process
std::string g_log;

std::string cache_key(const tb200_group_desc *d, unsigned vec_in, unsigned vec_out) {
    tb200_group_desc c;
    memset(&c, 0, sizeof c);
    c.n = d->n;   // rows stay out of the key: the kernel takes them at launch
    c.n_inputs = d->n_inputs; c.n_terms = d->n_terms; c.n_folds = d->n_folds; c.n_outputs = d->n_outputs;
    for (int i = 0; i < d->n_inputs; i++) { c.inputs[i].shape = d->inputs[i].shape; c.inputs[i].dtype = d->inputs[i].dtype; }
    for (int i = 0; i < d->n_terms; i++) {
        const int ar = term_arity(d->terms[i].op);
        c.terms[i].op = d->terms[i].op;
        c.terms[i].a = (ar > 0 || d->terms[i].op == TB200_T_LOAD || d->terms[i].op == TB200_T_STAT || d->terms[i].op == TB200_T_STAT2)
                           ? d->terms[i].a : 0;
        c.terms[i].b = ar > 1 ? d->terms[i].b : 0;
        c.terms[i].c = ar > 2 ? d->terms[i].c : 0;
        c.terms[i].imm = d->terms[i].op == TB200_T_LIT ? d->terms[i].imm : 0.0f;
    }
    for (int i = 0; i < d->n_folds; i++) c.folds[i] = d->folds[i];
    for (int i = 0; i < d->n_outputs; i++) {
        c.outputs[i].from = d->outputs[i].from; c.outputs[i].index = d->outputs[i].index; c.outputs[i].dtype = d->outputs[i].dtype;
    }
    std::string key(reinterpret_cast<const char *>(&c), sizeof c);
    key.append(reinterpret_cast<const char *>(&vec_in), sizeof vec_in);
    key.append(reinterpret_cast<const char *>(&vec_out), sizeof vec_out);
    return key;
}

int compile_group(const tb200_group_desc *d, unsigned vec_in, unsigned vec_out, Compiled **out) {
    Schedule S{};
    int st = make_schedule(d, vec_in, vec_out, &S);
    if (st) return st;
    const std::string key = cache_key(d, S.vec_in, S.vec_out);
    std::lock_guard<std::mutex> hold(g_cache_lock);
    auto it = g_cache.find(key);
    if (it != g_cache.end()) {
        *out = it->second;
        return TB200_OK;
    }
    Nvrtc &n = nvrtc();
    if (!n.ok) return TB200_ERR_UNSUPPORTED;
    const std::string source = generate(*d, S);
    void *prog = nullptr;
    if (n.create(&prog, source.c_str(), "tb200_group.cu", 0, nullptr, nullptr) != 0) return TB200_ERR_UNSUPPORTED;
    const char *options[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device", "--extra-device-vectorization", "--disable-warnings"};
    const int rc = n.compile(prog, 5, options);
    size_t log_bytes = 0;
    n.log_size(prog, &log_bytes);
    g_log.assign(log_bytes, '\0');
    if (log_bytes) n.log(prog, &g_log[0]);
    if (rc != 0) {
        n.destroy(&prog);
        return TB200_ERR_UNSUPPORTED;
    }
    size_t bytes = 0;
    n.cubin_size(prog, &bytes);
    Compiled *c = new Compiled();
    c->schedule = S;
    c->cubin.resize(bytes);
    n.cubin(prog, c->cubin.data());
    n.destroy(&prog);
    g_cache[key] = c;
    *out = c;
    return TB200_OK;
}

unsigned vector_mask_in(const tb200_group_desc *d, const void *const *inputs, int V) {
    unsigned mask = 0;
    for (int i = 0; i < d->n_inputs; i++) {
        const size_t bytes = dtype_size(d->inputs[i].dtype) * V;
        const bool rows_ok = d->inputs[i].shape != TB200_SHAPE_FULL || d->inputs[i].ld % V == 0;
        if ((d->inputs[i].shape == TB200_SHAPE_FULL || d->inputs[i].shape == TB200_SHAPE_ALONG) && rows_ok &&
            aligned_to(inputs[i], bytes > 16 ? 16 : bytes))
            mask |= 1u << i;
    }
    return mask;
}

// ------------------------------------------------ folds over the other axis ----
//
// The same descriptor with every fold running over the rows (the strided axis) instead of along them: the
// bias gradient, the LayerNorm weight gradients, any "sum over the batch" the planner forms
// (ext/cuTileExt/emit.jl:729-753, build.jl:654-696: partial folds + a merge kernel).  One thread owns a column,
// walks the rows of its slab in order evaluating the term DAG, and writes one partial per fold; a second kernel
// merges the slabs in order.  Coalesced (a warp reads 32 neighbouring columns of a row), deterministic, and the
// outputs are rounded once.  Folds: sum, max, min, prod; terms may not read row statistics.

constexpr int kColThreads = 256;
constexpr int kColSlabsMax = 512;
constexpr int kColBlocksWanted = 1536;   // about ten blocks of 256 threads per SM

struct ColParams {
    const void *in[TB200_GROUP_MAX_INPUTS];
    void *out[TB200_GROUP_MAX_OUTPUTS];
    long long ld_in[TB200_GROUP_MAX_INPUTS];
    float *partial;
    long long rows;
    int slabs;
};

int check_cols(const tb200_group_desc *d) {
    if (!d) return TB200_ERR_NULL;
    if (d->n < 0 || d->rows < 0 || d->n > (int64_t(1) << 30)) return TB200_ERR_SHAPE;
    if (d->n_inputs < 0 || d->n_inputs > TB200_GROUP_MAX_INPUTS || d->n_terms < 1 || d->n_terms > TB200_GROUP_MAX_TERMS ||
        d->n_folds < 1 || d->n_folds > TB200_GROUP_MAX_FOLDS || d->n_outputs < 1 || d->n_outputs > TB200_GROUP_MAX_OUTPUTS)
        return TB200_ERR_SHAPE;
    for (int i = 0; i < d->n_inputs; i++) {
        const tb200_group_input &in = d->inputs[i];
        if (in.dtype != TB200_F32 && in.dtype != TB200_BF16) return TB200_ERR_DTYPE;
        if (in.shape < TB200_SHAPE_FULL || in.shape > TB200_SHAPE_SCALAR) return TB200_ERR_SHAPE;
        if (in.shape == TB200_SHAPE_FULL && in.ld < d->n) return TB200_ERR_SHAPE;
    }
    for (int k = 0; k < d->n_terms; k++) {
        const tb200_term &T = d->terms[k];
        if (T.op < TB200_T_LOAD || T.op > TB200_T_ROUND_BF16) return TB200_ERR_UNSUPPORTED;
        if (T.op == TB200_T_STAT || T.op == TB200_T_STAT2) return TB200_ERR_UNSUPPORTED;
        if (T.op == TB200_T_LOAD && (T.a < 0 || T.a >= d->n_inputs)) return TB200_ERR_SHAPE;
        const int ar = term_arity(T.op);
        if ((ar > 0 && (T.a < 0 || T.a >= k)) || (ar > 1 && (T.b < 0 || T.b >= k)) || (ar > 2 && (T.c < 0 || T.c >= k)))
            return TB200_ERR_SHAPE;
    }
    for (int j = 0; j < d->n_folds; j++) {
        const int kind = d->folds[j].kind;
        if (kind < TB200_FOLD_SUM || kind > TB200_FOLD_MEANVAR) return TB200_ERR_UNSUPPORTED;
        if (d->folds[j].term < 0 || d->folds[j].term >= d->n_terms) return TB200_ERR_SHAPE;
    }
    for (int o = 0; o < d->n_outputs; o++) {
        const tb200_group_output &out = d->outputs[o];
        if ((out.from != 1 && out.from != 2) || out.index < 0 || out.index >= d->n_folds) return TB200_ERR_UNSUPPORTED;
        if (out.from == 2 && d->folds[out.index].kind != TB200_FOLD_MEANVAR) return TB200_ERR_SHAPE;
        if (out.dtype != TB200_F32 && out.dtype != TB200_BF16) return TB200_ERR_DTYPE;
    }
    return TB200_OK;
}

// Float32 words of a fold's state: one, two for the log-sum-exp's (maximum, rebased sum), three for the
// (count, mean, centred sum of squares) of mean and variance
int state_words(int kind) { return kind == TB200_FOLD_LOGSUMEXP ? 2 : kind == TB200_FOLD_MEANVAR ? 3 : 1; }
int total_state_words(const tb200_group_desc &d) {
    int words = 0;
    for (int j = 0; j < d.n_folds; j++) words += state_words(d.folds[j].kind);
    return words;
}

std::string col_load(const tb200_group_desc &d, int i, const std::string &index) {
    const std::string at = "[" + index + "]";
    return d.inputs[i].dtype == TB200_BF16 ? "bf2f(((const u16 *)p.in[" + num(i) + "])" + at + ")"
                                           : "((const float *)p.in[" + num(i) + "])" + at;
}

// declares `float c<i>[V]` holding V consecutive columns of input i starting at element `index`
void col_load_chunk(Emitter &E, int ind, const tb200_group_desc &d, int i, const std::string &index, int V, bool streaming) {
    const std::string c = "c" + num(i);
    if (V == 1) {
        E.line(ind, "const float " + c + "[1] = {" + col_load(d, i, index) + "};");
        return;
    }
    const std::string ld = streaming ? "__ldcs" : "__ldg";
    const std::string q = "q" + num(i);
    if (d.inputs[i].dtype == TB200_BF16 && V == 8) {
        E.line(ind, "const uint4 " + q + " = " + ld + "((const uint4 *)((const u16 *)p.in[" + num(i) + "] + " + index + "));");
        E.line(ind, "const float " + c + "[8] = {bf_lo(" + q + ".x), bf_hi(" + q + ".x), bf_lo(" + q + ".y), bf_hi(" + q + ".y), bf_lo(" + q +
                        ".z), bf_hi(" + q + ".z), bf_lo(" + q + ".w), bf_hi(" + q + ".w)};");
    } else if (d.inputs[i].dtype == TB200_BF16) {
        E.line(ind, "const uint2 q" + num(i) + " = " + ld + "((const uint2 *)((const u16 *)p.in[" + num(i) + "] + " + index + "));");
        E.line(ind, "const float " + c + "[4] = {bf_lo(q" + num(i) + ".x), bf_hi(q" + num(i) + ".x), bf_lo(q" + num(i) + ".y), bf_hi(q" + num(i) + ".y)};");
    } else {
        E.line(ind, "const float4 q" + num(i) + " = " + ld + "((const float4 *)((const float *)p.in[" + num(i) + "] + " + index + "));");
        E.line(ind, "const float " + c + "[4] = {q" + num(i) + ".x, q" + num(i) + ".y, q" + num(i) + ".z, q" + num(i) + ".w};");
    }
}

// V = 4 (8 when every array input is BFloat16): a thread owns that many neighbouring columns (128-bit accesses
// of the narrowest type; needs n, the row pitches and the addresses to allow it); V = 1: one column, any alignment
std::string generate_cols(const tb200_group_desc &d, int V) {
    Emitter E;
    E.line(0, "typedef unsigned short u16; typedef unsigned int u32; typedef long long i64;");
    E.line(0, "struct Params { const void *in[8]; void *out[8]; i64 ld_in[8]; float *partial; i64 rows; int slabs; };");
    E.line(0, "#define NEG_INF __uint_as_float(0xff800000u)");
    E.line(0, "#define POS_INF __uint_as_float(0x7f800000u)");
    E.line(0, "#define LOG2E 1.4426950408889634f");
    E.line(0, "static __device__ __forceinline__ float ex2(float x) { float y; asm(\"ex2.approx.ftz.f32 %0, %1;\" : \"=f\"(y) : \"f\"(x)); return y; }");
    E.line(0, "static __device__ __forceinline__ float exp_diff(float a, float b) { return ex2(fmaf(a, LOG2E, -(b * LOG2E))); }");
    E.line(0, "static __device__ __forceinline__ float bf2f(u32 h) { return __uint_as_float(h << 16); }");
    E.line(0, "static __device__ __forceinline__ float bf_lo(u32 w) { return __uint_as_float(w << 16); }");
    E.line(0, "static __device__ __forceinline__ float bf_hi(u32 w) { return __uint_as_float(w & 0xffff0000u); }");
    E.line(0, "static __device__ __forceinline__ u32 f2bf(float f) { u16 r; asm(\"cvt.rn.bf16.f32 %0, %1;\" : \"=h\"(r) : \"f\"(f)); return r; }");
    // NF: Float32 words of all the folds' states (a fold's words lie one after another in the partial rows)
    E.line(0, "constexpr int N = " + num(d.n) + ", NF = " + num(total_state_words(d)) + ", V = " + num(V) + ";");
    int word0[TB200_GROUP_MAX_FOLDS];
    for (int j = 0, w = 0; j < d.n_folds; j++) { word0[j] = w; w += state_words(d.folds[j].kind); }
    // names of fold j's state words, and of the state an element lifts to
    auto word = [](int j, int w, const std::string &at) { return std::string(w == 0 ? "f" : w == 1 ? "g" : "h") + num(j) + at; };
    auto lift = [&](int j, int w) -> std::string {
        const int kind = d.folds[j].kind;
        const std::string t = "t" + num(d.folds[j].term);
        if (kind == TB200_FOLD_LOGSUMEXP) return w == 0 ? t : "1.0f";
        if (kind == TB200_FOLD_MEANVAR) return w == 0 ? "1.0f" : w == 1 ? t : "0.0f";
        return t;
    };
    auto identity = [&](int j, int w) -> std::string { return w == 0 ? fold_identity(d.folds[j].kind) : "0.0f"; };
    bool used[TB200_GROUP_MAX_INPUTS] = {};
    for (int k = 0; k < d.n_terms; k++)
        if (d.terms[k].op == TB200_T_LOAD) used[d.terms[k].a] = true;
    // ---- partial folds
    E.line(0, "extern \"C\" __global__ void __launch_bounds__(" + num(kColThreads) + ") tb200_cols(const Params p) {");
    E.line(1, "const int i0 = (blockIdx.x * " + num(kColThreads) + " + threadIdx.x) * V;");
    E.line(1, "if (i0 >= N) return;");
    E.line(1, "const i64 per = (p.rows + p.slabs - 1) / p.slabs, r0 = blockIdx.y * per, r1 = r0 + per < p.rows ? r0 + per : p.rows;");
    for (int i = 0; i < d.n_inputs; i++) {
        if (!used[i]) continue;
        if (d.inputs[i].shape == TB200_SHAPE_ALONG) col_load_chunk(E, 1, d, i, "i0", V, false);
        if (d.inputs[i].shape == TB200_SHAPE_SCALAR) E.line(1, "const float sc" + num(i) + " = " + col_load(d, i, "0") + ";");
    }
    for (int j = 0; j < d.n_folds; j++)
        for (int w = 0; w < state_words(d.folds[j].kind); w++) {
            E.line(1, "float " + word(j, w, "[V]") + ";");
            E.line(1, "for (int e = 0; e < V; e++) " + word(j, w, "[e]") + " = " + identity(j, w) + ";");
        }
    E.line(1, "#pragma unroll 4");
    E.line(1, "for (i64 r = r0; r < r1; r++) {");
    for (int i = 0; i < d.n_inputs; i++) {
        if (!used[i]) continue;
        if (d.inputs[i].shape == TB200_SHAPE_PER_ROW) E.line(2, "const float pr" + num(i) + " = " + col_load(d, i, "r") + ";");
        if (d.inputs[i].shape == TB200_SHAPE_FULL) col_load_chunk(E, 2, d, i, "r * p.ld_in[" + num(i) + "] + i0", V, true);
    }
    E.line(2, "#pragma unroll");
    E.line(2, "for (int e = 0; e < V; e++) {");
    for (int k = 0; k < d.n_terms; k++) E.line(3, "const float t" + num(k) + " = " + term_expr(d, k, "") + ";");
    for (int j = 0; j < d.n_folds; j++)
        emit_merge(E, 3, d.folds[j].kind, word(j, 0, "[e]"), word(j, 1, "[e]"), word(j, 2, "[e]"), lift(j, 0), lift(j, 1), lift(j, 2));
    E.line(2, "}");
    E.line(1, "}");
    for (int j = 0; j < d.n_folds; j++)
        for (int w = 0; w < state_words(d.folds[j].kind); w++)
            E.line(1, "for (int e = 0; e < V; e++) p.partial[((i64)blockIdx.y * NF + " + num(word0[j] + w) + ") * N + i0 + e] = " +
                          word(j, w, "[e]") + ";");
    E.line(0, "}");
    // ---- merge of the slabs in a fixed order: 32 columns x 8 lanes a block; lane l folds slabs l, l + 8, ... in
    // order, then the eight lane results are folded in lane order
    E.line(0, "extern \"C\" __global__ void __launch_bounds__(" + num(kColThreads) + ") tb200_cols_merge(const Params p) {");
    E.line(1, "__shared__ float sm[NF][8][33];");
    E.line(1, "const int c = threadIdx.x & 31, l = threadIdx.x >> 5, i0 = blockIdx.x * 32 + c;");
    for (int j = 0; j < d.n_folds; j++) {
        const int kind = d.folds[j].kind, words = state_words(kind);
        for (int w = 0; w < words; w++) E.line(1, "float " + word(j, w, "") + " = " + identity(j, w) + ";");
        E.line(1, "if (i0 < N) {");
        E.line(2, "#pragma unroll 4");
        E.line(2, "for (int s = l; s < p.slabs; s += 8) {");
        for (int w = 0; w < words; w++)
            E.line(3, "const float o" + num(w) + " = p.partial[((i64)s * NF + " + num(word0[j] + w) + ") * N + i0];");
        emit_merge(E, 3, kind, word(j, 0, ""), word(j, 1, ""), word(j, 2, ""), "o0", "o1", "o2");
        E.line(2, "}");
        E.line(1, "}");
        for (int w = 0; w < words; w++) E.line(1, "sm[" + num(word0[j] + w) + "][l][c] = " + word(j, w, "") + ";");
    }
    E.line(1, "__syncthreads();");
    E.line(1, "if (l != 0 || i0 >= N) return;");
    for (int j = 0; j < d.n_folds; j++) {
        const int kind = d.folds[j].kind, words = state_words(kind);
        for (int w = 0; w < words; w++) E.line(1, word(j, w, "") + " = sm[" + num(word0[j] + w) + "][0][c];");
        E.line(1, "for (int k = 1; k < 8; k++) {");
        for (int w = 0; w < words; w++) E.line(2, "const float o" + num(w) + " = sm[" + num(word0[j] + w) + "][k][c];");
        emit_merge(E, 2, kind, word(j, 0, ""), word(j, 1, ""), word(j, 2, ""), "o0", "o1", "o2");
        E.line(1, "}");
    }
    for (int o = 0; o < d.n_outputs; o++) {
        // what a fold observes: the log-sum-exp from (maximum, rebased sum); the mean, or as the second value the
        // variance, from (count, mean, centred sum of squares); any other fold its one word
        const int j = d.outputs[o].index, kind = d.folds[j].kind;
        std::string v = word(j, 0, "");
        if (kind == TB200_FOLD_LOGSUMEXP) v = "(" + word(j, 1, "") + " > 0.0f ? " + word(j, 0, "") + " + logf(" + word(j, 1, "") + ") : " + word(j, 0, "") + ")";
        if (kind == TB200_FOLD_MEANVAR)
            v = d.outputs[o].from == 2 ? "(" + word(j, 0, "") + " > 0.0f ? " + word(j, 2, "") + " / " + word(j, 0, "") + " : 0.0f)" : word(j, 1, "");
        if (d.outputs[o].dtype == TB200_BF16) E.line(1, "((u16 *)p.out[" + num(o) + "])[i0] = (u16)f2bf(" + v + ");");
        else E.line(1, "((float *)p.out[" + num(o) + "])[i0] = " + v + ";");
    }
    E.line(0, "}");
    return E.s;
}

struct CompiledCols {
    std::vector<char> cubin;
    CUfunction fold[64] = {}, merge[64] = {};
};
std::map<std::string, CompiledCols *> g_col_cache;   // guarded by g_cache_lock

int compile_cols(const tb200_group_desc *d, int V, CompiledCols **out) {
    int st = check_cols(d);
    if (st) return st;
    std::string key = "cols" + num(V) + ":" + cache_key(d, 0, 0);
    for (int i = 0; i < d->n_inputs; i++) key.push_back(static_cast<char>('0' + d->inputs[i].shape));
    std::lock_guard<std::mutex> hold(g_cache_lock);
    auto it = g_col_cache.find(key);
    if (it != g_col_cache.end()) {
        *out = it->second;
        return TB200_OK;
    }
    Nvrtc &n = nvrtc();
    if (!n.ok) return TB200_ERR_UNSUPPORTED;
    const std::string source = generate_cols(*d, V);
    void *prog = nullptr;
    if (n.create(&prog, source.c_str(), "tb200_cols.cu", 0, nullptr, nullptr) != 0) return TB200_ERR_UNSUPPORTED;
    const char *options[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device", "--disable-warnings"};
    const int rc = n.compile(prog, 4, options);
    size_t log_bytes = 0;
    n.log_size(prog, &log_bytes);
    g_log.assign(log_bytes, '\0');
    if (log_bytes) n.log(prog, &g_log[0]);
    if (rc != 0) {
        n.destroy(&prog);
        return TB200_ERR_UNSUPPORTED;
    }
    size_t bytes = 0;
    n.cubin_size(prog, &bytes);
    CompiledCols *c = new CompiledCols();
    c->cubin.resize(bytes);
    n.cubin(prog, c->cubin.data());
    n.destroy(&prog);
    g_col_cache[key] = c;
    *out = c;
    return TB200_OK;
}

// columns a thread owns when the extents allow vectors (the addresses are checked at launch)
int col_width(const tb200_group_desc *d) {
    int V = 8;
    for (int i = 0; i < d->n_inputs; i++)
        if ((d->inputs[i].shape == TB200_SHAPE_FULL || d->inputs[i].shape == TB200_SHAPE_ALONG) && d->inputs[i].dtype == TB200_F32)
            V = 4;
    if (d->n % V != 0) return 1;
    for (int i = 0; i < d->n_inputs; i++)
        if (d->inputs[i].shape == TB200_SHAPE_FULL && d->inputs[i].ld % V != 0) return 1;
    return V;
}

// row slabs: enough blocks to fill the GPU whatever the row length (a function of the extents only, so that
// the workspace can be sized without a device)
int col_slabs(const tb200_group_desc *d, int V) {
    const int64_t col_blocks = ceil_div(d->n, static_cast<int64_t>(kColThreads) * V);
    int64_t slabs = ceil_div(kColBlocksWanted, col_blocks);
    if (slabs > kColSlabsMax) slabs = kColSlabsMax;
    if (slabs > d->rows) slabs = d->rows;
    return static_cast<int>(slabs < 1 ? 1 : slabs);
}

// ------------------------------------------------ recurrences whose step is a map ----
//
// One thread owns a position and walks the steps in order with the states in registers; the step's terms are
// straight-line Float32 code generated from the descriptor.  The rows of the step inputs are fetched eight steps
// ahead of the arithmetic (the chain through the states is arithmetic only), neighbouring threads read
// neighbouring positions, every member is rounded once where it is stored.

struct RecParams {
    const void *in[TB200_GROUP_MAX_INPUTS];
    void *out[TB200_GROUP_MAX_OUTPUTS];
    long long ld_in[TB200_GROUP_MAX_INPUTS];
    long long ld_out[TB200_GROUP_MAX_OUTPUTS];
    long long n, steps;
};

int check_recurrence(const tb200_recurrence_desc *r) {
    if (!r) return TB200_ERR_NULL;
    const tb200_group_desc *d = &r->body;
    if (d->n < 0 || d->rows < 0 || d->n > (int64_t(1) << 40)) return TB200_ERR_SHAPE;
    if (d->n_inputs < 0 || d->n_inputs > TB200_GROUP_MAX_INPUTS || d->n_terms < 1 || d->n_terms > TB200_GROUP_MAX_TERMS ||
        d->n_folds != 0 || d->n_outputs < 1 || d->n_outputs > TB200_GROUP_MAX_OUTPUTS)
        return TB200_ERR_SHAPE;
    if (r->n_states < 1 || r->n_states > TB200_RECURRENCE_MAX_STATES) return TB200_ERR_SHAPE;
    for (int i = 0; i < d->n_inputs; i++) {
        const tb200_group_input &in = d->inputs[i];
        if (in.dtype != TB200_F32 && in.dtype != TB200_BF16) return TB200_ERR_DTYPE;
        if (in.shape < TB200_SHAPE_FULL || in.shape > TB200_SHAPE_SCALAR) return TB200_ERR_UNSUPPORTED;
        if (in.shape == TB200_SHAPE_FULL && in.ld < d->n) return TB200_ERR_SHAPE;
    }
    for (int k = 0; k < d->n_terms; k++) {
        const tb200_term &T = d->terms[k];
        const bool leaf_ok = T.op == TB200_T_STATE || T.op == TB200_T_ROW_INDEX;
        if (!leaf_ok && (T.op < TB200_T_LOAD || T.op > TB200_T_ROUND_BF16)) return TB200_ERR_UNSUPPORTED;
        if (T.op == TB200_T_STAT || T.op == TB200_T_STAT2) return TB200_ERR_UNSUPPORTED;
        if (T.op == TB200_T_LOAD && (T.a < 0 || T.a >= d->n_inputs)) return TB200_ERR_SHAPE;
        if (T.op == TB200_T_STATE && (T.a < 0 || T.a >= r->n_states)) return TB200_ERR_SHAPE;
        const int ar = term_arity(T.op);
        if ((ar > 0 && (T.a < 0 || T.a >= k)) || (ar > 1 && (T.b < 0 || T.b >= k)) || (ar > 2 && (T.c < 0 || T.c >= k)))
            return TB200_ERR_SHAPE;
    }
    for (int k = 0; k < r->n_states; k++) {
        const tb200_state &S = r->states[k];
        if (S.start < 0 || S.start >= d->n_inputs || S.next < 0 || S.next >= d->n_terms) return TB200_ERR_SHAPE;
        const int shape = d->inputs[S.start].shape;
        if (shape != TB200_SHAPE_ALONG && shape != TB200_SHAPE_SCALAR) return TB200_ERR_SHAPE;
    }
    for (int o = 0; o < d->n_outputs; o++) {
        const tb200_group_output &out = d->outputs[o];
        if (out.dtype != TB200_F32 && out.dtype != TB200_BF16) return TB200_ERR_DTYPE;
        if (out.from == 0) {
            if (out.index < 0 || out.index >= d->n_terms || out.ld < d->n) return TB200_ERR_SHAPE;
        } else if (out.from == 3) {
            if (out.index < 0 || out.index >= r->n_states) return TB200_ERR_SHAPE;
        } else {
            return TB200_ERR_UNSUPPORTED;
        }
    }
    return TB200_OK;
}

std::string generate_recurrence(const tb200_recurrence_desc &r) {
    const tb200_group_desc &d = r.body;
    int streamed = 0;
    for (int i = 0; i < d.n_inputs; i++) streamed += d.inputs[i].shape == TB200_SHAPE_FULL || d.inputs[i].shape == TB200_SHAPE_PER_ROW;
    const int B = streamed > 4 ? 4 : 8;   // steps whose loads are in flight together (two such sets of registers)
    Emitter E;
    E.line(0, "typedef unsigned short u16; typedef unsigned int u32; typedef long long i64;");
    E.line(0, "struct Params { const void *in[8]; void *out[8]; i64 ld_in[8]; i64 ld_out[8]; i64 n, steps; };");
    E.line(0, "#define LOG2E 1.4426950408889634f");
    E.line(0, "static __device__ __forceinline__ float ex2(float x) { float y; asm(\"ex2.approx.ftz.f32 %0, %1;\" : \"=f\"(y) : \"f\"(x)); return y; }");
    E.line(0, "static __device__ __forceinline__ float exp_diff(float a, float b) { return ex2(fmaf(a, LOG2E, -(b * LOG2E))); }");
    E.line(0, "static __device__ __forceinline__ float bf2f(u32 h) { return __uint_as_float(h << 16); }");
    E.line(0, "static __device__ __forceinline__ u32 f2bf(float f) { u16 r; asm(\"cvt.rn.bf16.f32 %0, %1;\" : \"=h\"(r) : \"f\"(f)); return r; }");
    auto load = [&](int i, const std::string &index) {
        const std::string at = "[" + index + "]";
        return d.inputs[i].dtype == TB200_BF16 ? "bf2f(__ldg((const u16 *)p.in[" + num(i) + "] + " + index + "))"
                                               : "__ldg((const float *)p.in[" + num(i) + "] + " + index + ")";
    };
    auto store = [&](int o, const std::string &index, const std::string &value) {
        return d.outputs[o].dtype == TB200_BF16 ? "((u16 *)p.out[" + num(o) + "])[" + index + "] = (u16)f2bf(" + value + ");"
                                                : "((float *)p.out[" + num(o) + "])[" + index + "] = " + value + ";";
    };
    E.line(0, "extern \"C\" __global__ void __launch_bounds__(256) tb200_recurrence(const Params p) {");
    E.line(1, "const i64 col = (i64)blockIdx.x * blockDim.x + threadIdx.x;");
    E.line(1, "if (col >= p.n) return;");
    E.line(1, "const int i0 = (int)col, e = 0; (void)i0; (void)e;");
    // constants of the position, and the states' starts
    for (int i = 0; i < d.n_inputs; i++) {
        if (d.inputs[i].shape == TB200_SHAPE_ALONG) E.line(1, "const float al" + num(i) + " = " + load(i, "col") + ";");
        if (d.inputs[i].shape == TB200_SHAPE_SCALAR) E.line(1, "const float sc" + num(i) + " = " + load(i, "0") + ";");
    }
    for (int k = 0; k < r.n_states; k++) {
        const int i = r.states[k].start;
        E.line(1, "float st" + num(k) + " = " + (d.inputs[i].shape == TB200_SHAPE_ALONG ? "al" : "sc") + num(i) + ";");
    }
    // the loads of a block of steps are in flight while the block before it is computed: two sets of registers
    for (int i = 0; i < d.n_inputs; i++) {
        const std::string size = "[" + num(B) + "]";
        if (d.inputs[i].shape == TB200_SHAPE_FULL) E.line(1, "float x" + num(i) + size + ", nx" + num(i) + size + ";");
        if (d.inputs[i].shape == TB200_SHAPE_PER_ROW) E.line(1, "float pw" + num(i) + size + ", npw" + num(i) + size + ";");
    }
    auto fetch = [&](int level, const std::string &first) {
        E.line(level, "#pragma unroll");
        E.line(level, "for (int j = 0; j < " + num(B) + "; j++) {");
        E.line(level + 1, "const i64 s = " + first + " + j < p.steps ? " + first + " + j : p.steps - 1;");
        E.line(level + 1, std::string("const i64 row = ") + (r.reverse ? "p.steps - 1 - s" : "s") + ";");
        for (int i = 0; i < d.n_inputs; i++) {
            if (d.inputs[i].shape == TB200_SHAPE_FULL)
                E.line(level + 1, "nx" + num(i) + "[j] = " + load(i, "row * p.ld_in[" + num(i) + "] + col") + ";");
            if (d.inputs[i].shape == TB200_SHAPE_PER_ROW) E.line(level + 1, "npw" + num(i) + "[j] = " + load(i, "row") + ";");
        }
        E.line(level, "}");
    };
    E.line(1, "if (p.steps > 0) {");   // no steps: the states leave as they start, nothing is read
    fetch(2, "0");
    E.line(1, "}");
    E.line(1, "for (i64 s0 = 0; s0 < p.steps; s0 += " + num(B) + ") {");
    E.line(2, "#pragma unroll");
    E.line(2, "for (int j = 0; j < " + num(B) + "; j++) {");
    for (int i = 0; i < d.n_inputs; i++) {
        if (d.inputs[i].shape == TB200_SHAPE_FULL) E.line(3, "x" + num(i) + "[j] = nx" + num(i) + "[j];");
        if (d.inputs[i].shape == TB200_SHAPE_PER_ROW) E.line(3, "pw" + num(i) + "[j] = npw" + num(i) + "[j];");
    }
    E.line(2, "}");
    fetch(2, "(s0 + " + num(B) + ")");
    E.line(2, "#pragma unroll");
    E.line(2, "for (int j = 0; j < " + num(B) + "; j++) {");
    E.line(3, "if (s0 + j < p.steps) {");
    E.line(4, std::string("const i64 row = ") + (r.reverse ? "p.steps - 1 - (s0 + j)" : "s0 + j") + ";");
    for (int k = 0; k < d.n_terms; k++) {
        const tb200_term &T = d.terms[k];
        std::string expr;
        if (T.op == TB200_T_LOAD) {
            const int shape = d.inputs[T.a].shape;
            expr = shape == TB200_SHAPE_FULL ? "x" + num(T.a) + "[j]" : shape == TB200_SHAPE_PER_ROW ? "pw" + num(T.a) + "[j]"
                   : shape == TB200_SHAPE_ALONG ? "al" + num(T.a) : "sc" + num(T.a);
        } else {
            expr = term_expr(d, k, "");
        }
        E.line(4, "const float t" + num(k) + " = " + expr + ";");
    }
    for (int o = 0; o < d.n_outputs; o++)
        if (d.outputs[o].from == 0) E.line(4, store(o, "row * p.ld_out[" + num(o) + "] + col", "t" + num(d.outputs[o].index)));
    for (int k = 0; k < r.n_states; k++) E.line(4, "st" + num(k) + " = t" + num(r.states[k].next) + ";");
    E.line(3, "}");
    E.line(2, "}");
    E.line(1, "}");
    for (int o = 0; o < d.n_outputs; o++)
        if (d.outputs[o].from == 3) E.line(1, store(o, "col", "st" + num(d.outputs[o].index)));
    E.line(0, "}");
    return E.s;
}

struct CompiledRec {
    std::vector<char> cubin;
    CUfunction function[64] = {};
};
std::map<std::string, CompiledRec *> g_rec_cache;   // guarded by g_cache_lock

int compile_recurrence(const tb200_recurrence_desc *r, CompiledRec **out) {
    int st = check_recurrence(r);
    if (st) return st;
    std::string key = "rec:" + cache_key(&r->body, 0, 0);
    for (int i = 0; i < r->body.n_inputs; i++) key.push_back(static_cast<char>('0' + r->body.inputs[i].shape));
    for (int k = 0; k < r->body.n_terms; k++)
        if (r->body.terms[k].op == TB200_T_STATE) key += "s" + num(k) + "=" + num(r->body.terms[k].a) + ";";
    for (int k = 0; k < r->n_states; k++) key += "|" + num(r->states[k].start) + "," + num(r->states[k].next);
    key += r->reverse ? "R" : "F";
    std::lock_guard<std::mutex> hold(g_cache_lock);
    auto it = g_rec_cache.find(key);
    if (it != g_rec_cache.end()) {
        *out = it->second;
        return TB200_OK;
    }
    Nvrtc &n = nvrtc();
    if (!n.ok) return TB200_ERR_UNSUPPORTED;
    const std::string source = generate_recurrence(*r);
    void *prog = nullptr;
    if (n.create(&prog, source.c_str(), "tb200_recurrence.cu", 0, nullptr, nullptr) != 0) return TB200_ERR_UNSUPPORTED;
    const char *options[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device", "--disable-warnings"};
    const int rc = n.compile(prog, 4, options);
    size_t log_bytes = 0;
    n.log_size(prog, &log_bytes);
    g_log.assign(log_bytes, '\0');
    if (log_bytes) n.log(prog, &g_log[0]);
    if (rc != 0) {
        n.destroy(&prog);
        return TB200_ERR_UNSUPPORTED;
    }
    size_t bytes = 0;
    n.cubin_size(prog, &bytes);
    CompiledRec *c = new CompiledRec();
    c->cubin.resize(bytes);
    n.cubin(prog, c->cubin.data());
    n.destroy(&prog);
    g_rec_cache[key] = c;
    *out = c;
    return TB200_OK;
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" int tb200_rowreduce_compile(const tb200_group_desc *d, unsigned vector_inputs, unsigned vector_outputs) {
    if (!d) return TB200_ERR_NULL;
    if (d->n == 0) return tb200_rowreduce_generic_check(d);
    Compiled *c = nullptr;
    return compile_group(d, vector_inputs, vector_outputs, &c);
}

extern "C" size_t tb200_rowreduce_source(const tb200_group_desc *d, unsigned vector_inputs, unsigned vector_outputs, char *buffer,
                                         size_t buffer_bytes) {
    Schedule S{};
    if (!d || d->n <= 0 || make_schedule(d, vector_inputs, vector_outputs, &S) != TB200_OK) return 0;
    const std::string source = generate(*d, S);
    if (buffer && buffer_bytes) {
        const size_t take = source.size() < buffer_bytes - 1 ? source.size() : buffer_bytes - 1;
        memcpy(buffer, source.data(), take);
        buffer[take] = '\0';
    }
    return source.size() + 1;
}

extern "C" const char *tb200_rowreduce_compile_log(void) {
    static thread_local std::string copy;
    std::lock_guard<std::mutex> hold(g_cache_lock);
    copy = g_log;
    return copy.c_str();
}

extern "C" int tb200_rowreduce_compiled(const tb200_group_desc *d, const void *const *inputs, void *const *outputs, void *stream_) {
    int st = tb200_rowreduce_generic_check(d);
    if (st) return st;
    if (d->n == 0 || d->rows == 0) return TB200_OK;
    if (!outputs || (d->n_inputs > 0 && !inputs)) return TB200_ERR_NULL;
    LaunchParams P{};
    bool any_f32 = false;
    for (int i = 0; i < d->n_inputs; i++) {
        // with no steps the arrays that have one row per step are empty, and an empty array may have no address
        const bool per_step = d->inputs[i].shape == TB200_SHAPE_FULL || d->inputs[i].shape == TB200_SHAPE_PER_ROW;
        if (!inputs[i] && !(per_step && d->rows == 0)) return TB200_ERR_NULL;
        if (!aligned_to(inputs[i], dtype_size(d->inputs[i].dtype))) return TB200_ERR_ALIGN;
        P.in[i] = inputs[i];
        P.ld_in[i] = d->inputs[i].ld;
        if (d->inputs[i].shape == TB200_SHAPE_FULL || d->inputs[i].shape == TB200_SHAPE_ALONG) any_f32 |= d->inputs[i].dtype == TB200_F32;
    }
    for (int o = 0; o < d->n_outputs; o++) {
        if (!outputs[o] && !(d->outputs[o].from == 0 && d->rows == 0)) return TB200_ERR_NULL;
        if (!aligned_to(outputs[o], dtype_size(d->outputs[o].dtype))) return TB200_ERR_ALIGN;
        P.out[o] = outputs[o];
        P.ld_out[o] = d->outputs[o].ld;
        if (d->outputs[o].from == 0) any_f32 |= d->outputs[o].dtype == TB200_F32;
    }
    P.rows = d->rows;
    const int V = any_f32 ? 4 : 8;
    const unsigned vec_in = vector_mask_in(d, inputs, V);
    unsigned vec_out = 0;
    for (int o = 0; o < d->n_outputs; o++) {
        const size_t bytes = dtype_size(d->outputs[o].dtype) * V;
        if (d->outputs[o].from == 0 && d->outputs[o].ld % V == 0 && aligned_to(outputs[o], bytes > 16 ? 16 : bytes)) vec_out |= 1u << o;
    }
    Compiled *c = nullptr;
    if ((st = compile_group(d, vec_in, vec_out, &c))) return st;
    DeviceInfo dev;
    if ((st = current_device(&dev))) return st;
    Driver *drv = nullptr;
    if ((st = driver(&drv))) return st;
    {
        std::lock_guard<std::mutex> hold(g_cache_lock);
        if (!c->function[dev.device]) {
            TB200_CUDA(cudaFree(nullptr));   // the runtime's context is current before the driver is used
            CUmodule module = nullptr;
            if (drv->module_load(&module, c->cubin.data()) != CUDA_SUCCESS) return TB200_ERR_CUDA;
            CUfunction fn = nullptr;
            if (drv->get_function(&fn, module, "tb200_group") != CUDA_SUCCESS) return TB200_ERR_CUDA;
            int per_sm = 0;
            if (drv->occupancy(&per_sm, fn, kThreads, 0) != CUDA_SUCCESS || per_sm < 1) per_sm = 1;
            c->blocks_per_sm[dev.device] = per_sm;
            c->function[dev.device] = fn;
        }
    }
    const int64_t blocks = ceil_div(d->rows, c->schedule.rpb);
    const int64_t cap = static_cast<int64_t>(dev.sms) * c->blocks_per_sm[dev.device];
    void *args[] = {&P};
    if (drv->launch(c->function[dev.device], static_cast<unsigned>(blocks < cap ? blocks : cap), 1, 1, kThreads, 1, 1, 0,
                    static_cast<CUstream>(stream_), args, nullptr) != CUDA_SUCCESS)
        return TB200_ERR_CUDA;
    return TB200_OK;
}

// ---- folds over the other axis

extern "C" size_t tb200_colreduce_workspace_bytes(const tb200_group_desc *d) {
    if (check_cols(d) != TB200_OK) return 0;
    // the widest form has the fewest column blocks, hence the most slabs
    tb200_group_desc any_rows = *d;
    any_rows.rows = kColSlabsMax;
    return static_cast<size_t>(col_slabs(&any_rows, 8)) * total_state_words(*d) * static_cast<size_t>(d->n) * sizeof(float);
}

extern "C" int tb200_colreduce_compile(const tb200_group_desc *d) {
    if (!d) return TB200_ERR_NULL;
    CompiledCols *c = nullptr;
    int st = compile_cols(d, 1, &c);
    if (st == TB200_OK && col_width(d) > 1) st = compile_cols(d, col_width(d), &c);
    return st;
}

extern "C" size_t tb200_colreduce_source(const tb200_group_desc *d, char *buffer, size_t buffer_bytes) {
    if (check_cols(d) != TB200_OK) return 0;
    const std::string source = generate_cols(*d, col_width(d));
    if (buffer && buffer_bytes) {
        const size_t take = source.size() < buffer_bytes - 1 ? source.size() : buffer_bytes - 1;
        memcpy(buffer, source.data(), take);
        buffer[take] = '\0';
    }
    return source.size() + 1;
}

extern "C" int tb200_colreduce_compiled(const tb200_group_desc *d, const void *const *inputs, void *const *outputs,
                                        void *workspace, size_t workspace_bytes, void *stream_) {
    int st = check_cols(d);
    if (st) return st;
    if (d->n == 0) return TB200_OK;
    if (!outputs || (d->n_inputs > 0 && !inputs)) return TB200_ERR_NULL;
    ColParams P{};
    for (int i = 0; i < d->n_inputs; i++) {
        // with no steps the arrays that have one row per step are empty, and an empty array may have no address
        const bool per_step = d->inputs[i].shape == TB200_SHAPE_FULL || d->inputs[i].shape == TB200_SHAPE_PER_ROW;
        if (!inputs[i] && !(per_step && d->rows == 0)) return TB200_ERR_NULL;
        if (!aligned_to(inputs[i], dtype_size(d->inputs[i].dtype))) return TB200_ERR_ALIGN;
        P.in[i] = inputs[i];
        P.ld_in[i] = d->inputs[i].ld;
    }
    for (int o = 0; o < d->n_outputs; o++) {
        if (!outputs[o]) return TB200_ERR_NULL;
        if (!aligned_to(outputs[o], dtype_size(d->outputs[o].dtype))) return TB200_ERR_ALIGN;
        P.out[o] = outputs[o];
    }
    if (!workspace || workspace_bytes < tb200_colreduce_workspace_bytes(d) || !aligned_to(workspace, 16)) return TB200_ERR_WORKSPACE;
    int V = col_width(d);
    for (int i = 0; i < d->n_inputs && V > 1; i++) {
        const int shape = d->inputs[i].shape;
        if ((shape == TB200_SHAPE_FULL || shape == TB200_SHAPE_ALONG) && !aligned_to(inputs[i], V * dtype_size(d->inputs[i].dtype)))
            V = 1;
    }
    CompiledCols *c = nullptr;
    if ((st = compile_cols(d, V, &c))) return st;
    DeviceInfo dev;
    if ((st = current_device(&dev))) return st;
    Driver *drv = nullptr;
    if ((st = driver(&drv))) return st;
    {
        std::lock_guard<std::mutex> hold(g_cache_lock);
        if (!c->fold[dev.device]) {
            TB200_CUDA(cudaFree(nullptr));   // the runtime's context is current before the driver is used
            CUmodule module = nullptr;
            if (drv->module_load(&module, c->cubin.data()) != CUDA_SUCCESS) return TB200_ERR_CUDA;
            CUfunction fold = nullptr, merge = nullptr;
            if (drv->get_function(&fold, module, "tb200_cols") != CUDA_SUCCESS) return TB200_ERR_CUDA;
            if (drv->get_function(&merge, module, "tb200_cols_merge") != CUDA_SUCCESS) return TB200_ERR_CUDA;
            c->merge[dev.device] = merge;
            c->fold[dev.device] = fold;
        }
    }
    P.partial = static_cast<float *>(workspace);
    P.rows = d->rows;
    P.slabs = col_slabs(d, V);   // rows == 0: one slab of no rows, every fold's identity
    const unsigned col_blocks = static_cast<unsigned>(ceil_div(d->n, static_cast<int64_t>(kColThreads) * V));
    const unsigned merge_blocks = static_cast<unsigned>(ceil_div(d->n, 32));
    void *args[] = {&P};
    if (drv->launch(c->fold[dev.device], col_blocks, static_cast<unsigned>(P.slabs), 1, kColThreads, 1, 1, 0,
                    static_cast<CUstream>(stream_), args, nullptr) != CUDA_SUCCESS)
        return TB200_ERR_CUDA;
    if (drv->launch(c->merge[dev.device], merge_blocks, 1, 1, kColThreads, 1, 1, 0, static_cast<CUstream>(stream_), args,
                    nullptr) != CUDA_SUCCESS)
        return TB200_ERR_CUDA;
    return TB200_OK;
}

extern "C" int tb200_recurrence_compile(const tb200_recurrence_desc *r) {
    CompiledRec *c = nullptr;
    return compile_recurrence(r, &c);
}

extern "C" size_t tb200_recurrence_source(const tb200_recurrence_desc *r, char *buffer, size_t buffer_bytes) {
    if (check_recurrence(r) != TB200_OK) return 0;
    const std::string source = generate_recurrence(*r);
    if (buffer && buffer_bytes > 0) {
        const size_t len = source.size() < buffer_bytes - 1 ? source.size() : buffer_bytes - 1;
        memcpy(buffer, source.data(), len);
        buffer[len] = '\0';
    }
    return source.size() + 1;
}

extern "C" int tb200_recurrence_compiled(const tb200_recurrence_desc *r, const void *const *inputs, void *const *outputs,
                                         void *stream_) {
    int st = check_recurrence(r);
    if (st) return st;
    const tb200_group_desc *d = &r->body;
    if (d->n == 0) return TB200_OK;
    if (!outputs || !inputs) return TB200_ERR_NULL;
    RecParams P{};
    for (int i = 0; i < d->n_inputs; i++) {
        // with no steps the arrays that have one row per step are empty, and an empty array may have no address
        const bool per_step = d->inputs[i].shape == TB200_SHAPE_FULL || d->inputs[i].shape == TB200_SHAPE_PER_ROW;
        if (!inputs[i] && !(per_step && d->rows == 0)) return TB200_ERR_NULL;
        if (!aligned_to(inputs[i], dtype_size(d->inputs[i].dtype))) return TB200_ERR_ALIGN;
        P.in[i] = inputs[i];
        P.ld_in[i] = d->inputs[i].ld;
    }
    for (int o = 0; o < d->n_outputs; o++) {
        if (!outputs[o] && !(d->outputs[o].from == 0 && d->rows == 0)) return TB200_ERR_NULL;
        if (!aligned_to(outputs[o], dtype_size(d->outputs[o].dtype))) return TB200_ERR_ALIGN;
        P.out[o] = outputs[o];
        P.ld_out[o] = d->outputs[o].ld;
    }
    P.n = d->n;
    P.steps = d->rows;
    CompiledRec *c = nullptr;
    if ((st = compile_recurrence(r, &c))) return st;
    DeviceInfo dev;
    if ((st = current_device(&dev))) return st;
    Driver *drv = nullptr;
    if ((st = driver(&drv))) return st;
    {
        std::lock_guard<std::mutex> hold(g_cache_lock);
        if (!c->function[dev.device]) {
            TB200_CUDA(cudaFree(nullptr));   // the runtime's context is current before the driver is used
            CUmodule module = nullptr;
            if (drv->module_load(&module, c->cubin.data()) != CUDA_SUCCESS) return TB200_ERR_CUDA;
            CUfunction fn = nullptr;
            if (drv->get_function(&fn, module, "tb200_recurrence") != CUDA_SUCCESS) return TB200_ERR_CUDA;
            c->function[dev.device] = fn;
        }
    }
    // the steps are a dependent chain per position, so the positions are the only parallelism: blocks as small as it
    // takes to put some on every SM (a warp at the least), 256 threads once there are enough positions for that
    unsigned threads = 256;
    while (threads > 32 && ceil_div(d->n, threads) < 2ll * dev.sms) threads /= 2;
    const long long blocks = ceil_div(d->n, threads);
    if (blocks > 0x7fffffffll) return TB200_ERR_SHAPE;
    void *args[] = {&P};
    if (drv->launch(c->function[dev.device], static_cast<unsigned>(blocks), 1, 1, threads, 1, 1, 0, static_cast<CUstream>(stream_), args,
                    nullptr) != CUDA_SUCCESS)
        return TB200_ERR_CUDA;
    return TB200_OK;
}
