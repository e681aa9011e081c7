// Groups that are not a row fold of scalars: recognised and handed to the kernel that computes them.
//
// The reference describes attention to a backend as ONE reduction group (src/Compiler/Implement/groups.jl:106-125):
// the element folded over the keys is a pair (score, value row), the score is a `Recomputed` term -- a sum over the
// feature axis formed where it is read (src/Compiler/IR/terms.jl:69-87) --, the causal mask is an `ifelse` on two
// positions (`mask_condition`, ext/cuTileExt/mask.jl:54-75), the log-sum-exp of the scores shares the sweep, and
// the output is the weights' sum of the value rows.  tb200_group_desc spells those three things as
// TB200_T_RECOMPUTED, TB200_T_ROW_INDEX beside TB200_T_INDEX under a TB200_T_SELECT, and TB200_FOLD_WEIGHTED.
// The term interpreter and the kernel generator decline such descriptors (they fold scalars along a row);
// this file recognises the attention group among them -- by the structure of its terms, as the reference's
// `claimed` recognises the sketches it has kernels for (ext/cuTileExt/cuTileExt.jl:899-929) -- and runs it on the
// attention kernels.  Host code only.
#include "common.cuh"

namespace tb200 {
namespace {

struct AttentionMatch {
    bool causal;
    float scale;
    int q_input, k_input, v_input;   // inputs of the recomputed scores' two factors and of the weighted rows
    int lse_fold, out_fold;
    int extent;                      // features
};

bool is_lit(const tb200_group_desc *d, int t, float *value) {
    if (t < 0 || t >= d->n_terms || d->terms[t].op != TB200_T_LIT) return false;
    *value = d->terms[t].imm;
    return true;
}

// scale * Recomputed(q, k) in either order of the product, or the bare Recomputed (scale 1)
bool match_scores(const tb200_group_desc *d, int t, AttentionMatch *m) {
    if (t < 0 || t >= d->n_terms) return false;
    const tb200_term &T = d->terms[t];
    int r = t;
    m->scale = 1.0f;
    if (T.op == TB200_T_MUL) {
        float s;
        if (is_lit(d, T.a, &s)) r = T.b;
        else if (is_lit(d, T.b, &s)) r = T.a;
        else return false;
        m->scale = s;
    }
    if (r < 0 || r >= d->n_terms || d->terms[r].op != TB200_T_RECOMPUTED) return false;
    const tb200_term &R = d->terms[r];
    if (R.a < 0 || R.a >= d->n_inputs || R.b < 0 || R.b >= d->n_inputs || R.c <= 0) return false;
    if (d->inputs[R.a].shape != TB200_SHAPE_ROW_VECTORS || d->inputs[R.b].shape != TB200_SHAPE_ALONG_VECTORS) return false;
    m->q_input = R.a; m->k_input = R.b; m->extent = R.c;
    return true;
}

// select(row_index - index + c > 0, scores, -Inf) with 0 < c <= 1: positions up to and including the row's own
bool match_causal(const tb200_group_desc *d, int t, AttentionMatch *m) {
    const tb200_term &T = d->terms[t];
    if (T.op != TB200_T_SELECT) return false;
    float fill;
    if (!is_lit(d, T.c, &fill) || !(fill < 0.0f) || !isinf(fill)) return false;
    if (T.a < 0 || T.a >= d->n_terms || d->terms[T.a].op != TB200_T_ADD) return false;
    const tb200_term &P = d->terms[T.a];
    float c;
    int diff;
    if (is_lit(d, P.b, &c)) diff = P.a;
    else if (is_lit(d, P.a, &c)) diff = P.b;
    else return false;
    if (!(c > 0.0f && c <= 1.0f)) return false;
    if (diff < 0 || diff >= d->n_terms || d->terms[diff].op != TB200_T_SUB) return false;
    const tb200_term &D = d->terms[diff];
    if (D.a < 0 || D.b < 0 || d->terms[D.a].op != TB200_T_ROW_INDEX || d->terms[D.b].op != TB200_T_INDEX) return false;
    return match_scores(d, T.b, m);
}

int match_attention(const tb200_group_desc *d, AttentionMatch *m) {
    if (!d) return TB200_ERR_NULL;
    if (d->n_inputs < 3 || d->n_inputs > TB200_GROUP_MAX_INPUTS || d->n_terms < 3 || d->n_terms > TB200_GROUP_MAX_TERMS ||
        d->n_folds != 2 || d->n_outputs < 1 || d->n_outputs > 2)
        return TB200_ERR_UNSUPPORTED;
    m->lse_fold = m->out_fold = -1;
    for (int f = 0; f < 2; f++) {
        if (d->folds[f].kind == TB200_FOLD_LOGSUMEXP) m->lse_fold = f;
        if (d->folds[f].kind == TB200_FOLD_WEIGHTED) m->out_fold = f;
        if (d->folds[f].term < 0 || d->folds[f].term >= d->n_terms) return TB200_ERR_SHAPE;
    }
    if (m->lse_fold < 0 || m->out_fold < 0) return TB200_ERR_UNSUPPORTED;
    // the scores: masked or not
    const int scores = d->folds[m->lse_fold].term;
    m->causal = match_causal(d, scores, m);
    if (!m->causal && !match_scores(d, scores, m)) return TB200_ERR_UNSUPPORTED;
    // the weights: exp(scores - stat(lse)), folded with the value rows
    const tb200_fold &of = d->folds[m->out_fold];
    const tb200_term &W = d->terms[of.term];
    if (W.op != TB200_T_EXP || W.a < 0 || d->terms[W.a].op != TB200_T_SUB) return TB200_ERR_UNSUPPORTED;
    const tb200_term &S = d->terms[W.a];
    if (S.a != scores || S.b < 0 || d->terms[S.b].op != TB200_T_STAT || d->terms[S.b].a != m->lse_fold) return TB200_ERR_UNSUPPORTED;
    m->v_input = of.payload;
    if (m->v_input < 0 || m->v_input >= d->n_inputs || d->inputs[m->v_input].shape != TB200_SHAPE_ALONG_VECTORS)
        return TB200_ERR_UNSUPPORTED;
    for (int i : {m->q_input, m->k_input, m->v_input})
        if (d->inputs[i].dtype != TB200_BF16 || d->inputs[i].ld != m->extent) return TB200_ERR_UNSUPPORTED;
    // outputs: the weighted rows (BFloat16, one vector per row), and optionally the log-sum-exp (Float32)
    bool has_out = false;
    for (int o = 0; o < d->n_outputs; o++) {
        const tb200_group_output &out = d->outputs[o];
        if (out.from != 1) return TB200_ERR_UNSUPPORTED;
        if (out.index == m->out_fold && out.dtype == TB200_BF16) has_out = true;
        else if (!(out.index == m->lse_fold && out.dtype == TB200_F32)) return TB200_ERR_UNSUPPORTED;
    }
    return has_out ? TB200_OK : TB200_ERR_UNSUPPORTED;
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" int tb200_group_route(const tb200_group_desc *d) {
    AttentionMatch m;
    const int st = match_attention(d, &m);
    if (st == TB200_OK) return m.causal ? TB200_ROUTE_ATTENTION_CAUSAL : TB200_ROUTE_ATTENTION;
    return st == TB200_ERR_UNSUPPORTED ? TB200_ROUTE_NONE : st;
}

extern "C" int tb200_group_attention(const tb200_group_desc *d, int heads, int kv_heads, int batch, const void *const *inputs,
                                     void *const *outputs, void *stream) {
    AttentionMatch m;
    int st = match_attention(d, &m);
    if (st) return st;
    if (heads <= 0 || kv_heads <= 0 || batch < 0 || d->n > INT32_MAX || d->rows > INT32_MAX) return TB200_ERR_SHAPE;
    if (!inputs || !outputs) return TB200_ERR_NULL;
    tb200_attn_desc a{};
    a.batch = batch; a.heads = heads; a.kv_heads = kv_heads;
    a.queries = static_cast<int>(d->rows); a.keys = static_cast<int>(d->n); a.head_dim = m.extent;
    a.causal = m.causal; a.scale = m.scale; a.dtype = TB200_BF16;
    void *o = nullptr;
    float *lse = nullptr;
    for (int i = 0; i < d->n_outputs; i++) {
        if (d->outputs[i].index == m.out_fold) o = outputs[i];
        else lse = static_cast<float *>(outputs[i]);
    }
    return tb200_attention_fwd(&a, inputs[m.q_input], inputs[m.k_input], inputs[m.v_input], o, lse, stream);
}
