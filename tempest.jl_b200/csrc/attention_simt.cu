// Attention for head dimensions other than 128: Float32 arithmetic on CUDA cores, any head dimension up to
// 256, any lengths, grouped heads, causal or not.  It exists so that every geometry of the reference's own
// attention tests (test/cuda/attention.jl:10-16: D = 8, 16, 32 with 70, 133, 200 positions) has a path through
// this library; it is a fallback in the sense of Tempest's floor (src/Compiler/codegen/scalar.jl:200-256), not
// a tuned kernel -- the tensor-core kernels take D = 128.
//
// The same program as the fast path (test/fixtures/operations.jl:21-76): scores in Float32 from the BFloat16
// q, k; causal keeps key <= query; lse = logsumexp over keys (natural log); o = sum_n v exp(s - lse) rounded
// to BFloat16.  Pullback (src/Compiler/program/differentiate.jl:215-218, 461-467): p = exp(s - lse),
// delta = sum_d dO o, ds = p (dp - delta), dq = scale ds k, dk = scale ds' q, dv = p' dO.
//
// One warp per query (forward, dq) or per key (dk, dv): lanes take 32 keys (queries) of a step for the scores,
// then the head dimension for the accumulation.
#include "attention_simt.cuh"
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kMaxD = 256;
constexpr int kWarps = 4;

struct SimtArgs {
    int batch, heads, kv_heads, queries, keys, d, causal;
    int dv;                        // features of the values (v, o, dout, dv); d unless the descriptor says otherwise
    float scale;
    long long qb, qs, qh;          // element strides of q, dq over (batch, position, head)
    long long kb, ks, kh;          // of k, dk
    long long ob, os, oh;          // of o, dout
    long long vb, vs, vh;          // of v, dv
    const int *doc_start;          // [batch][queries]: first key a query sees, or null
    const int *kv_len;             // [batch]: keys from this index on are masked, or null
};

// the keys query i of batch b sees: [first, last]
__device__ __forceinline__ void key_range(const SimtArgs &a, int b, int i, int &first, int &last) {
    first = a.doc_start ? a.doc_start[static_cast<long long>(b) * a.queries + i] : 0;
    last = a.causal ? i : a.keys - 1;
    if (a.kv_len) last = min(last, a.kv_len[b] - 1);
    if (last > a.keys - 1) last = a.keys - 1;
    if (first < 0) first = 0;
}

__device__ __forceinline__ float ldbf(const __nv_bfloat16 *p) { return __bfloat162float(*p); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__global__ void __launch_bounds__(kWarps * 32) attention_simt_fwd_kernel(const __nv_bfloat16 *q, const __nv_bfloat16 *k,
                                                                        const __nv_bfloat16 *v, __nv_bfloat16 *o,
                                                                        float *lse, SimtArgs a) {
    __shared__ float qs[kWarps][kMaxD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i = blockIdx.x * kWarps + warp, h = blockIdx.y, b = blockIdx.z;
    if (i >= a.queries) return;
    const int g = h / (a.heads / a.kv_heads);
    const long long qrow = b * a.qb + i * a.qs + h * a.qh;
    const long long orow = b * a.ob + i * a.os + h * a.oh;
    for (int d = lane; d < a.d; d += 32) qs[warp][d] = ldbf(q + qrow + d) * a.scale;
    __syncwarp();
    int first, last;
    key_range(a, b, i, first, last);
    float m = -INFINITY, l = 0.0f, acc[kMaxD / 32] = {};
    for (int key0 = first; key0 <= last; key0 += 32) {
        const int j = key0 + lane;
        const bool valid = j <= last;
        float s = -INFINITY;
        if (valid) {
            const __nv_bfloat16 *kr = k + b * a.kb + j * a.ks + g * a.kh;
            s = 0.0f;
            for (int d = 0; d < a.d; d++) s = fmaf(qs[warp][d], ldbf(kr + d), s);
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? __expf(s - m_new) : 0.0f;
        const float corr = __expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int c = 0; c < kMaxD / 32; c++) acc[c] *= corr;
        const int count = min(32, last - key0 + 1);
        for (int jj = 0; jj < count; jj++) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const __nv_bfloat16 *vr = v + b * a.vb + (key0 + jj) * a.vs + g * a.vh;
#pragma unroll
            for (int c = 0; c < kMaxD / 32; c++) {
                const int d = lane + 32 * c;
                if (d < a.dv) acc[c] = fmaf(pj, ldbf(vr + d), acc[c]);
            }
        }
        m = m_new;
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;   // a query that sees no key: zero output, log-sum-exp -Inf
#pragma unroll
    for (int c = 0; c < kMaxD / 32; c++) {
        const int d = lane + 32 * c;
        if (d < a.dv) o[orow + d] = __float2bfloat16_rn(acc[c] * inv);
    }
    if (lse && lane == 0) lse[(static_cast<long long>(b) * a.queries + i) * a.heads + h] = l > 0.0f ? m + __logf(l) : -INFINITY;
}

__global__ void __launch_bounds__(kWarps * 32) attention_simt_dq_kernel(const __nv_bfloat16 *q, const __nv_bfloat16 *k,
                                                                       const __nv_bfloat16 *v, const __nv_bfloat16 *o,
                                                                       const float *lse, const __nv_bfloat16 *dout,
                                                                       __nv_bfloat16 *dq, SimtArgs a) {
    __shared__ float qs[kWarps][kMaxD], gs[kWarps][kMaxD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i = blockIdx.x * kWarps + warp, h = blockIdx.y, b = blockIdx.z;
    if (i >= a.queries) return;
    const int g = h / (a.heads / a.kv_heads);
    const long long qrow = b * a.qb + i * a.qs + h * a.qh;
    const long long orow = b * a.ob + i * a.os + h * a.oh;
    float delta = 0.0f;
    for (int d = lane; d < a.d; d += 32) qs[warp][d] = ldbf(q + qrow + d) * a.scale;
    for (int d = lane; d < a.dv; d += 32) {
        const float gd = ldbf(dout + orow + d);
        gs[warp][d] = gd;
        delta = fmaf(gd, ldbf(o + orow + d), delta);
    }
    delta = warp_sum(delta);
    __syncwarp();
    const float L = lse[(static_cast<long long>(b) * a.queries + i) * a.heads + h];
    int first, last;
    key_range(a, b, i, first, last);
    float acc[kMaxD / 32] = {};
    for (int key0 = first; key0 <= last; key0 += 32) {
        const int j = key0 + lane;
        float ds = 0.0f;
        if (j <= last) {
            const long long kv = b * a.kb + j * a.ks + g * a.kh;
            const long long vv = b * a.vb + j * a.vs + g * a.vh;
            float s = 0.0f, dp = 0.0f;
            for (int d = 0; d < a.d; d++) s = fmaf(qs[warp][d], ldbf(k + kv + d), s);
            for (int d = 0; d < a.dv; d++) dp = fmaf(gs[warp][d], ldbf(v + vv + d), dp);
            ds = __expf(s - L) * (dp - delta);
        }
        const int count = min(32, last - key0 + 1);
        for (int jj = 0; jj < count; jj++) {
            const float dsj = __shfl_sync(0xffffffffu, ds, jj);
            const __nv_bfloat16 *kr = k + b * a.kb + (key0 + jj) * a.ks + g * a.kh;
#pragma unroll
            for (int c = 0; c < kMaxD / 32; c++) {
                const int d = lane + 32 * c;
                if (d < a.d) acc[c] = fmaf(dsj, ldbf(kr + d), acc[c]);
            }
        }
    }
#pragma unroll
    for (int c = 0; c < kMaxD / 32; c++) {
        const int d = lane + 32 * c;
        if (d < a.d) dq[qrow + d] = __float2bfloat16_rn(acc[c] * a.scale);
    }
}

__global__ void __launch_bounds__(kWarps * 32) attention_simt_dkdv_kernel(const __nv_bfloat16 *q, const __nv_bfloat16 *k,
                                                                         const __nv_bfloat16 *v, const __nv_bfloat16 *o,
                                                                         const float *lse, const __nv_bfloat16 *dout,
                                                                         __nv_bfloat16 *dk, __nv_bfloat16 *dv, SimtArgs a) {
    __shared__ float ks[kWarps][kMaxD], vs[kWarps][kMaxD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = blockIdx.x * kWarps + warp, g = blockIdx.y, b = blockIdx.z;
    if (j >= a.keys) return;
    const long long krow = b * a.kb + j * a.ks + g * a.kh;
    const long long vrow = b * a.vb + j * a.vs + g * a.vh;
    const bool key_live = !a.kv_len || j < a.kv_len[b];
    for (int d = lane; d < a.d; d += 32) ks[warp][d] = ldbf(k + krow + d) * a.scale;
    for (int d = lane; d < a.dv; d += 32) vs[warp][d] = ldbf(v + vrow + d);
    __syncwarp();
    const int rep = a.heads / a.kv_heads;
    float acck[kMaxD / 32] = {}, accv[kMaxD / 32] = {};
    for (int r = 0; r < rep; r++) {
        const int h = g * rep + r;
        for (int i0 = a.causal ? (j / 32) * 32 : 0; i0 < a.queries; i0 += 32) {
            const int i = i0 + lane;
            float p = 0.0f, ds = 0.0f;
            if (key_live && i < a.queries && (!a.causal || i >= j) &&
                (!a.doc_start || a.doc_start[static_cast<long long>(b) * a.queries + i] <= j)) {
                const long long qr = b * a.qb + i * a.qs + h * a.qh;
                const long long orr = b * a.ob + i * a.os + h * a.oh;
                float s = 0.0f, dp = 0.0f, delta = 0.0f;
                for (int d = 0; d < a.d; d++) s = fmaf(ks[warp][d], ldbf(q + qr + d), s);
                for (int d = 0; d < a.dv; d++) {
                    const float gd = ldbf(dout + orr + d);
                    dp = fmaf(gd, vs[warp][d], dp);
                    delta = fmaf(gd, ldbf(o + orr + d), delta);
                }
                p = __expf(s - lse[(static_cast<long long>(b) * a.queries + i) * a.heads + h]);
                ds = p * (dp - delta);
            }
            const int count = min(32, a.queries - i0);
            for (int ii = 0; ii < count; ii++) {
                const float pi = __shfl_sync(0xffffffffu, p, ii), dsi = __shfl_sync(0xffffffffu, ds, ii);
                if (pi == 0.0f && dsi == 0.0f) continue;   // masked (uniform across the warp)
                const long long qr = b * a.qb + (i0 + ii) * a.qs + h * a.qh;
                const long long orr = b * a.ob + (i0 + ii) * a.os + h * a.oh;
#pragma unroll
                for (int c = 0; c < kMaxD / 32; c++) {
                    const int d = lane + 32 * c;
                    if (d < a.dv) accv[c] = fmaf(pi, ldbf(dout + orr + d), accv[c]);
                    if (d < a.d) acck[c] = fmaf(dsi, ldbf(q + qr + d), acck[c]);
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < kMaxD / 32; c++) {
        const int d = lane + 32 * c;
        if (d < a.d) dk[krow + d] = __float2bfloat16_rn(acck[c] * a.scale);
        if (d < a.dv) dv[vrow + d] = __float2bfloat16_rn(accv[c]);
    }
}

SimtArgs simt_args(const tb200_attn_desc *d, const tb200_attn_mask *m) {
    SimtArgs a{};
    a.batch = d->batch; a.heads = d->heads; a.kv_heads = d->kv_heads; a.queries = d->queries; a.keys = d->keys;
    a.d = d->head_dim; a.causal = d->causal; a.scale = d->scale;
    a.dv = attention_value_dim(d);
    // the dense default: [batch][position][head][feature]
    a.qh = d->head_dim; a.qs = a.qh * d->heads; a.qb = a.qs * d->queries;
    a.kh = d->head_dim; a.ks = a.kh * d->kv_heads; a.kb = a.ks * d->keys;
    a.oh = a.dv; a.os = a.oh * d->heads; a.ob = a.os * d->queries;
    a.vh = a.dv; a.vs = a.vh * d->kv_heads; a.vb = a.vs * d->keys;
    if (m) {
        a.doc_start = m->doc_start;
        a.kv_len = m->kv_len;
        // other strides: the same for the arrays of either kind (refused before this where the values have features
        // of their own)
        if (m->q_stride[0] || m->q_stride[1] || m->q_stride[2]) {
            a.qb = a.ob = m->q_stride[0]; a.qs = a.os = m->q_stride[1]; a.qh = a.oh = m->q_stride[2];
        }
        if (m->kv_stride[0] || m->kv_stride[1] || m->kv_stride[2]) {
            a.kb = a.vb = m->kv_stride[0]; a.ks = a.vs = m->kv_stride[1]; a.kh = a.vh = m->kv_stride[2];
        }
    }
    return a;
}

}  // namespace

bool attention_simt_takes(const tb200_attn_desc *d) {
    return d->head_dim <= kMaxD && attention_value_dim(d) <= kMaxD && d->value_dim >= 0 && d->heads <= 65535 &&
           d->batch <= 65535;
}

int attention_simt_fwd(const tb200_attn_desc *d, const void *q, const void *k, const void *v, void *o, float *lse,
                       cudaStream_t stream, const tb200_attn_mask *mask) {
    dim3 grid(static_cast<unsigned>(ceil_div(d->queries, kWarps)), d->heads, d->batch);
    attention_simt_fwd_kernel<<<grid, kWarps * 32, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(q), static_cast<const __nv_bfloat16 *>(k), static_cast<const __nv_bfloat16 *>(v),
        static_cast<__nv_bfloat16 *>(o), lse, simt_args(d, mask));
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

int attention_simt_bwd(const tb200_attn_desc *d, const void *q, const void *k, const void *v, const void *o,
                       const float *lse, const void *dout, void *dq, void *dk, void *dv, cudaStream_t stream,
                       const tb200_attn_mask *mask) {
    const __nv_bfloat16 *qb = static_cast<const __nv_bfloat16 *>(q), *kb = static_cast<const __nv_bfloat16 *>(k),
                        *vb = static_cast<const __nv_bfloat16 *>(v), *ob = static_cast<const __nv_bfloat16 *>(o),
                        *gb = static_cast<const __nv_bfloat16 *>(dout);
    dim3 gq(static_cast<unsigned>(ceil_div(d->queries, kWarps)), d->heads, d->batch);
    attention_simt_dq_kernel<<<gq, kWarps * 32, 0, stream>>>(qb, kb, vb, ob, lse, gb, static_cast<__nv_bfloat16 *>(dq),
                                                            simt_args(d, mask));
    TB200_CUDA(cudaGetLastError());
    dim3 gk(static_cast<unsigned>(ceil_div(d->keys, kWarps)), d->kv_heads, d->batch);
    attention_simt_dkdv_kernel<<<gk, kWarps * 32, 0, stream>>>(qb, kb, vb, ob, lse, gb, static_cast<__nv_bfloat16 *>(dk),
                                                              static_cast<__nv_bfloat16 *>(dv), simt_args(d, mask));
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

}  // namespace tb200

using namespace tb200;

namespace {
int check_masked(const tb200_attn_desc *d) {
    if (!d) return TB200_ERR_NULL;
    if (d->batch < 0 || d->heads <= 0 || d->kv_heads <= 0 || d->queries < 0 || d->keys < 0 || d->head_dim <= 0) return TB200_ERR_SHAPE;
    if (d->heads % d->kv_heads != 0 || !(d->scale > 0.0f)) return TB200_ERR_SHAPE;
    if (d->causal && d->queries != d->keys) return TB200_ERR_SHAPE;
    if (d->dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (!attention_simt_takes(d)) return TB200_ERR_UNSUPPORTED;
    return TB200_OK;
}
// values with features of their own come as dense arrays
bool strided_values(const tb200_attn_desc *d, const tb200_attn_mask *m) {
    if (!m || attention_value_dim(d) == d->head_dim) return false;
    for (int i = 0; i < 3; i++)
        if (m->q_stride[i] || m->kv_stride[i]) return true;
    return false;
}
}  // namespace

extern "C" int tb200_attention_fwd_masked(const tb200_attn_desc *d, const tb200_attn_mask *mask, const void *q, const void *k,
                                          const void *v, void *o, float *lse, void *stream) {
    int st = check_masked(d);
    if (st) return st;
    if (strided_values(d, mask)) return TB200_ERR_UNSUPPORTED;
    if (d->batch == 0 || d->queries == 0) return TB200_OK;
    if (d->keys == 0) return TB200_ERR_UNSUPPORTED;
    if (!q || !k || !v || !o) return TB200_ERR_NULL;
    // 128 features, 16-byte aligned arrays, strides the TMA unit can describe: the tensor-core kernel
    if (attention_tensor_geometry(d) && d->dtype == TB200_BF16 && aligned_to(q, 16) && aligned_to(k, 16) && aligned_to(v, 16) &&
        aligned_to(o, 16) && d->queries <= (1 << 24) && d->keys <= (1 << 24)) {
        st = attention_tensor_fwd(d, mask, q, k, v, o, lse, static_cast<cudaStream_t>(stream));
        if (st != TB200_ERR_UNSUPPORTED) return st;
    }
    return attention_simt_fwd(d, q, k, v, o, lse, static_cast<cudaStream_t>(stream), mask);
}

extern "C" int tb200_attention_bwd_masked(const tb200_attn_desc *d, const tb200_attn_mask *mask, const void *q, const void *k,
                                          const void *v, const void *o, const float *lse, const void *dout, void *dq, void *dk,
                                          void *dv, void *stream) {
    int st = check_masked(d);
    if (st) return st;
    if (strided_values(d, mask)) return TB200_ERR_UNSUPPORTED;
    if (d->batch == 0 || (d->queries == 0 && d->keys == 0)) return TB200_OK;
    if (d->queries == 0 || d->keys == 0) return TB200_ERR_UNSUPPORTED;
    if (!q || !k || !v || !o || !lse || !dout || !dq || !dk || !dv) return TB200_ERR_NULL;
    return attention_simt_bwd(d, q, k, v, o, lse, dout, dq, dk, dv, static_cast<cudaStream_t>(stream), mask);
}

// Which kernels compute a descriptor: the tests the entries make, in their order, without a device.
extern "C" int tb200_attention_form(const tb200_attn_desc *d, int masked, int pullback) {
    if (!d) return TB200_ERR_NULL;
    if (d->batch < 0 || d->heads <= 0 || d->kv_heads <= 0 || d->queries < 0 || d->keys < 0 || d->head_dim <= 0)
        return TB200_ERR_SHAPE;
    if (d->heads % d->kv_heads != 0 || !(d->scale > 0.0f)) return TB200_ERR_SHAPE;
    if (d->causal && d->queries != d->keys) return TB200_ERR_SHAPE;
    if (d->dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (d->queries > (1 << 24) || d->keys > (1 << 24)) return TB200_ERR_SHAPE;
    if (!attention_tensor_geometry(d)) return attention_simt_takes(d) ? TB200_ATTN_FORM_CUDA_CORES : TB200_ERR_UNSUPPORTED;
    if (pullback) return d->deterministic ? TB200_ATTN_FORM_TWO_KERNELS : TB200_ATTN_FORM_ONE_KERNEL;
    return (d->queries > 128 && !masked) ? TB200_ATTN_FORM_TWO_TILES : TB200_ATTN_FORM_TILE;
}
