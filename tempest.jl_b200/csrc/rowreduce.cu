// Fused row reductions for sm_100a: softmax and LayerNorm, forward and the
// backward the tape's derivative rules produce, over rows whose folded axis is
// contiguous.
//
// Two schedules, chosen from the row length (the counterpart of the
// reference's resident / split sketches, ext/cuTileExt/cuTileExt.jl:438-455):
//
//  * resident: `tpr` threads share a row and hold all of it in registers
//    (up to 32 elements each, fetched as 128-bit loads), so the row crosses
//    HBM once in and once out.  Blocks are persistent: a grid of
//    SMs x resident-blocks walks the row groups, which lets LayerNorm keep
//    gamma/beta and its dgamma/dbeta partial sums in registers across rows.
//  * split: a long row is cut into chunks of 256 threads x 32 elements; a first
//    launch folds every chunk to a partial state in the workspace, a second
//    merges the row's partial states and writes the outputs ("split-K, two
//    passes").
//
// Numerics: Float32 arithmetic for either element type, sums as fixed-order
// trees (deterministic), exp as ex2.approx of a scaled argument, outputs
// rounded once.
#include <cstdio>
#include <cstdlib>
#include <initializer_list>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "sm100.cuh"

namespace tb200 {
namespace {

constexpr int kResidentMaxThreads = 512;
constexpr int kSplitThreads = 256;

struct RowArgs {
    const void *in0;    // x (forward), y or x (softmax backward), x (LayerNorm backward)
    const void *in1;    // dy
    const void *gamma;
    const void *beta;
    void *out0;         // y (forward) or dx (backward)
    void *stat0;        // lse | mean
    void *stat1;        // rstd
    const void *cstat0; // saved lse | mean
    const void *cstat1; // saved rstd
    float *part0;       // dgamma partial sums [parts][n] | split states
    float *part1;       // dbeta partial sums [parts][n]
    float eps;
    int n;              // row length
    int tpr;            // threads per row (resident)
    int rpc;            // rows per block (resident)
    int splits;         // chunks per row (split)
    int stat_bf16;
    int exact;          // every vector slot of every row slot is inside the data: no bounds checks
    long long rows, ld;
};

template <typename T, bool VEC, int VPT>
struct Row {
    using A = Access<T, VEC>;
    static constexpr int EPV = A::EPV;
    static constexpr int E = VPT * EPV;
    static __device__ __forceinline__ int at(int k, int t, int tpr) { return (k * tpr + t) * EPV; }

    template <bool EXACT = false>
    static __device__ __forceinline__ void load(float (&v)[E], const T *row, int n, int t, int tpr, float fill,
                                                bool live) {
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            int idx = at(k, t, tpr);
            if (EXACT || (live && idx < n)) A::load(row + idx, &v[k * EPV]);
            else
#pragma unroll
                for (int e = 0; e < EPV; e++) v[k * EPV + e] = fill;
        }
    }
    static __device__ __forceinline__ void load_cached(float (&v)[E], const T *row, int n, int t, int tpr,
                                                       float fill) {
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            int idx = at(k, t, tpr);
            if (idx < n) A::load_cached(row + idx, &v[k * EPV]);
            else
#pragma unroll
                for (int e = 0; e < EPV; e++) v[k * EPV + e] = fill;
        }
    }
    template <bool EXACT = false>
    static __device__ __forceinline__ void store(const float (&v)[E], T *row, int n, int t, int tpr, bool live) {
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            int idx = at(k, t, tpr);
            if (EXACT || (live && idx < n)) A::store(row + idx, &v[k * EPV]);
        }
    }
    // Float32 partial sums, one row of the workspace
    static __device__ __forceinline__ void store_f32(const float (&v)[E], float *row, int n, int t, int tpr) {
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            int idx = at(k, t, tpr);
            if (idx < n) {
                if constexpr (EPV % 4 == 0) {
#pragma unroll
                    for (int e = 0; e < EPV; e += 4)
                        *reinterpret_cast<float4 *>(row + idx + e) =
                            make_float4(v[k * EPV + e], v[k * EPV + e + 1], v[k * EPV + e + 2], v[k * EPV + e + 3]);
                } else {
#pragma unroll
                    for (int e = 0; e < EPV; e++) row[idx + e] = v[k * EPV + e];
                }
            }
        }
    }
    // whether element slot (k, e) of thread t lies inside the row
    static __device__ __forceinline__ bool inside(int k, int t, int tpr, int n) { return at(k, t, tpr) < n; }
};

// ------------------------------------------------------------ resident ------

template <typename T, bool VEC, int VPT, bool EXACT>
__device__ __forceinline__ void softmax_fwd_resident_body(const RowArgs &a) {
    using R = Row<T, VEC, VPT>;
    __shared__ float red[2 * 32 * kRedWidth];
    RowCtx c = make_row_ctx(a.tpr, red);
    const T *x = static_cast<const T *>(a.in0);
    T *y = static_cast<T *>(a.out0);
    const long long groups = (a.rows + a.rpc - 1) / a.rpc;
    for (long long g = blockIdx.x; g < groups; g += gridDim.x) {
        const long long r = g * a.rpc + c.slot;
        const bool live = EXACT || r < a.rows;
        float v[R::E];
        R::template load<EXACT>(v, x + r * a.ld, a.n, c.t, a.tpr, -INFINITY, live);
        float m = -INFINITY;
#pragma unroll
        for (int e = 0; e < R::E; e++) m = fmaxf(m, v[e]);
        m = row_allreduce1(m, c, MaxOp());
        // exponentials are taken relative to the maximum, or to zero when it
        // is infinite (an empty or all -Inf row sums to zero)
        const float sh = (fabsf(m) <= 3.402823466e38f) ? m : 0.0f;
        const float off = sh * kLog2e;
        float s = 0.0f;
#pragma unroll
        for (int e = 0; e < R::E; e++) {
            v[e] = fast_exp2(fmaf(v[e], kLog2e, -off));
            s += v[e];
        }
        s = row_allreduce1(s, c, SumOp());
        if (live && c.t == 0 && a.stat0) store_stat(a.stat0, r, m + logf(s), a.stat_bf16);
        const float inv = 1.0f / s;
#pragma unroll
        for (int e = 0; e < R::E; e++) v[e] *= inv;
        R::template store<EXACT>(v, y + r * a.ld, a.n, c.t, a.tpr, live);
    }
}

template <typename T, bool VEC, int VPT>
__global__ void __launch_bounds__(kResidentMaxThreads) softmax_fwd_resident(RowArgs a) {
    if (a.exact) softmax_fwd_resident_body<T, VEC, VPT, true>(a);
    else softmax_fwd_resident_body<T, VEC, VPT, false>(a);
}

template <typename T, bool VEC, int VPT, bool EXACT>
__device__ __forceinline__ void softmax_bwd_resident_body(const RowArgs &a) {
    using R = Row<T, VEC, VPT>;
    __shared__ float red[2 * 32 * kRedWidth];
    RowCtx c = make_row_ctx(a.tpr, red);
    const T *yx = static_cast<const T *>(a.in0);
    const T *dy = static_cast<const T *>(a.in1);
    T *dx = static_cast<T *>(a.out0);
    const long long groups = (a.rows + a.rpc - 1) / a.rpc;
    for (long long g = blockIdx.x; g < groups; g += gridDim.x) {
        const long long r = g * a.rpc + c.slot;
        const bool live = EXACT || r < a.rows;
        float y[R::E], d[R::E];
        R::template load<EXACT>(y, yx + r * a.ld, a.n, c.t, a.tpr, a.cstat0 ? -INFINITY : 0.0f, live);
        R::template load<EXACT>(d, dy + r * a.ld, a.n, c.t, a.tpr, 0.0f, live);
        if (a.cstat0) {
            const float off = (live ? load_stat(a.cstat0, r, a.stat_bf16) : 0.0f) * kLog2e;
#pragma unroll
            for (int e = 0; e < R::E; e++) y[e] = fast_exp2(fmaf(y[e], kLog2e, -off));
        }
        float s = 0.0f;
#pragma unroll
        for (int e = 0; e < R::E; e++) s = fmaf(y[e], d[e], s);
        s = row_allreduce1(s, c, SumOp());
#pragma unroll
        for (int e = 0; e < R::E; e++) d[e] = y[e] * (d[e] - s);
        R::template store<EXACT>(d, dx + r * a.ld, a.n, c.t, a.tpr, live);
    }
}

template <typename T, bool VEC, int VPT>
__global__ void __launch_bounds__(kResidentMaxThreads) softmax_bwd_resident(RowArgs a) {
    if (a.exact) softmax_bwd_resident_body<T, VEC, VPT, true>(a);
    else softmax_bwd_resident_body<T, VEC, VPT, false>(a);
}

template <typename T, bool VEC, int VPT, bool EXACT>
__device__ __forceinline__ void layernorm_fwd_resident_body(const RowArgs &a) {
    using R = Row<T, VEC, VPT>;
    __shared__ float red[2 * 32 * kRedWidth];
    RowCtx c = make_row_ctx(a.tpr, red);
    const T *x = static_cast<const T *>(a.in0);
    T *y = static_cast<T *>(a.out0);
    // gamma and beta (a few KB, shared by every row) are re-read through L1 for
    // each row rather than pinned in registers: the registers buy occupancy
    const T *gamma = static_cast<const T *>(a.gamma);
    const T *beta = static_cast<const T *>(a.beta);
    const float fn = static_cast<float>(a.n);
    const long long groups = (a.rows + a.rpc - 1) / a.rpc;
    for (long long g = blockIdx.x; g < groups; g += gridDim.x) {
        const long long r = g * a.rpc + c.slot;
        const bool live = EXACT || r < a.rows;
        float v[R::E];
        R::template load<EXACT>(v, x + r * a.ld, a.n, c.t, a.tpr, 0.0f, live);
        float s = 0.0f;
#pragma unroll
        for (int e = 0; e < R::E; e++) s += v[e];
        const float mean = row_allreduce1(s, c, SumOp()) / fn;
        float q = 0.0f;
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const bool in = EXACT || R::inside(k, c.t, a.tpr, a.n);
#pragma unroll
            for (int e = 0; e < R::EPV; e++) {
                const float d = v[k * R::EPV + e] - mean;
                v[k * R::EPV + e] = d;
                q = in ? fmaf(d, d, q) : q;
            }
        }
        const float var = row_allreduce1(q, c, SumOp()) / fn;
        const float rstd = 1.0f / sqrtf(var + a.eps);
        if (live && c.t == 0) {
            if (a.stat0) static_cast<float *>(a.stat0)[r] = mean;
            if (a.stat1) static_cast<float *>(a.stat1)[r] = rstd;
        }
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int idx = R::at(k, c.t, a.tpr);
            if (EXACT || idx < a.n) {
                float gam[R::EPV], bet[R::EPV];
                R::A::load_cached(gamma + idx, gam);
                if (beta) R::A::load_cached(beta + idx, bet);
#pragma unroll
                for (int e = 0; e < R::EPV; e++)
                    v[k * R::EPV + e] = fmaf(v[k * R::EPV + e] * rstd, gam[e], beta ? bet[e] : 0.0f);
            }
        }
        R::template store<EXACT>(v, y + r * a.ld, a.n, c.t, a.tpr, live);
    }
}

// Rows of at most 16 elements a thread are compiled for three resident blocks of 512 threads (40 registers): at
// 64 registers the 4096-element Float32 rows of the benchmark ran four 256-thread blocks per SM, half the warps
// the SM holds, and the kernel waited on memory latency rather than bandwidth.
template <typename T, bool VEC, int VPT>
__global__ void __launch_bounds__(kResidentMaxThreads, (VPT * Access<T, VEC>::EPV <= 16 ? 3 : 2))
layernorm_fwd_resident(RowArgs a) {
    if (a.exact) layernorm_fwd_resident_body<T, VEC, VPT, true>(a);
    else layernorm_fwd_resident_body<T, VEC, VPT, false>(a);
}

template <typename T, bool VEC, int VPT, bool EXACT>
__device__ __forceinline__ void layernorm_bwd_resident_body(const RowArgs &a) {
    using R = Row<T, VEC, VPT>;
    __shared__ float red[2 * 32 * kRedWidth];
    RowCtx c = make_row_ctx(a.tpr, red);
    const T *x = static_cast<const T *>(a.in0);
    const T *dy = static_cast<const T *>(a.in1);
    T *dx = static_cast<T *>(a.out0);
    float gam[R::E], dg[R::E], db[R::E];
    R::load_cached(gam, static_cast<const T *>(a.gamma), a.n, c.t, a.tpr, 0.0f);
#pragma unroll
    for (int e = 0; e < R::E; e++) dg[e] = db[e] = 0.0f;
    const float fn = static_cast<float>(a.n);
    const long long groups = (a.rows + a.rpc - 1) / a.rpc;
    for (long long g = blockIdx.x; g < groups; g += gridDim.x) {
        const long long r = g * a.rpc + c.slot;
        const bool live = EXACT || r < a.rows;
        float v[R::E], d[R::E];
        R::template load<EXACT>(v, x + r * a.ld, a.n, c.t, a.tpr, 0.0f, live);
        R::template load<EXACT>(d, dy + r * a.ld, a.n, c.t, a.tpr, 0.0f, live);
        float mean, rstd;
        if (a.cstat0 && a.cstat1) {
            mean = live ? static_cast<const float *>(a.cstat0)[r] : 0.0f;
            rstd = live ? static_cast<const float *>(a.cstat1)[r] : 0.0f;
        } else {
            float s = 0.0f;
#pragma unroll
            for (int e = 0; e < R::E; e++) s += v[e];
            mean = row_allreduce1(s, c, SumOp()) / fn;
            float q = 0.0f;
#pragma unroll
            for (int k = 0; k < VPT; k++) {
                const bool in = EXACT || R::inside(k, c.t, a.tpr, a.n);
#pragma unroll
                for (int e = 0; e < R::EPV; e++) {
                    const float t = v[k * R::EPV + e] - mean;
                    q = in ? fmaf(t, t, q) : q;
                }
            }
            rstd = 1.0f / sqrtf(row_allreduce1(q, c, SumOp()) / fn + a.eps);
            // a slot past the last row holds zeros: with eps = 0 its rstd is infinite and 0 * inf would
            // put NaN into the column sums, so it takes the same (0, 0) the saved-statistics branch gives it
            if (!live) { mean = 0.0f; rstd = 0.0f; }
        }
        // xh in v; padded slots have gamma = 0 and dy = 0, so they add nothing.  The arithmetic runs on
        // pairs of Float32 (fma.rn.f32x2 and friends): the kernel is bound by instruction issue for
        // BFloat16 rows, and the packed forms halve its floating-point instructions.
        static_assert(R::E % 2 == 0 || R::E == 1, "pairs");
        float s2[2] = {0.0f, 0.0f};
        if constexpr (R::E % 2 == 0) {
            const float2 rs2 = make_float2(rstd, rstd);
            const float2 off2 = make_float2(-mean * rstd, -mean * rstd);
            float2 sa = make_float2(0.0f, 0.0f), sb = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int e = 0; e < R::E; e += 2) {
                const float2 xh = __ffma2_rn(make_float2(v[e], v[e + 1]), rs2, off2);
                const float2 dy2 = make_float2(d[e], d[e + 1]);
                const float2 gh = __fmul2_rn(dy2, make_float2(gam[e], gam[e + 1]));
                sa = __fadd2_rn(sa, gh);
                sb = __ffma2_rn(gh, xh, sb);
                const float2 g2 = __ffma2_rn(dy2, xh, make_float2(dg[e], dg[e + 1]));
                const float2 b2 = __fadd2_rn(make_float2(db[e], db[e + 1]), dy2);
                dg[e] = g2.x; dg[e + 1] = g2.y;
                db[e] = b2.x; db[e + 1] = b2.y;
                v[e] = xh.x; v[e + 1] = xh.y;
                d[e] = gh.x; d[e + 1] = gh.y;      // dy is not needed again: keep gh in its place
            }
            s2[0] = sa.x + sa.y;
            s2[1] = sb.x + sb.y;
        } else {
            const float xh = (v[0] - mean) * rstd;
            const float gh = d[0] * gam[0];
            s2[0] = gh;
            s2[1] = gh * xh;
            dg[0] = fmaf(d[0], xh, dg[0]);
            db[0] += d[0];
            v[0] = xh;
            d[0] = gh;
        }
        row_allreduce<2>(s2, c, SumOp());
        const float c1 = s2[0] / fn, c2 = s2[1] / fn;
        if constexpr (R::E % 2 == 0) {
            const float2 nc1 = make_float2(-c1, -c1), nc2 = make_float2(-c2, -c2), rs2 = make_float2(rstd, rstd);
#pragma unroll
            for (int e = 0; e < R::E; e += 2) {
                // (gh - c1) first: exact when they are equal (a row of one element), then - xh c2, then * rstd
                const float2 t = __fadd2_rn(make_float2(d[e], d[e + 1]), nc1);
                const float2 u = __fmul2_rn(__ffma2_rn(make_float2(v[e], v[e + 1]), nc2, t), rs2);
                d[e] = u.x; d[e + 1] = u.y;
            }
        } else {
            d[0] = rstd * ((d[0] - c1) - v[0] * c2);
        }
        R::template store<EXACT>(d, dx + r * a.ld, a.n, c.t, a.tpr, live);
    }
    if (a.part0) {
        const long long p = static_cast<long long>(blockIdx.x) * a.rpc + c.slot;
        R::store_f32(dg, a.part0 + p * a.n, a.n, c.t, a.tpr);
        R::store_f32(db, a.part1 + p * a.n, a.n, c.t, a.tpr);
    }
}

template <typename T, bool VEC, int VPT>
__global__ void __launch_bounds__(kResidentMaxThreads) layernorm_bwd_resident(RowArgs a) {
    if (a.exact) layernorm_bwd_resident_body<T, VEC, VPT, true>(a);
    else layernorm_bwd_resident_body<T, VEC, VPT, false>(a);
}

// The BFloat16 LayerNorm backward again for the common case (128-bit accesses, rows that fill every slot,
// mean and rstd saved by the forward), arranged for occupancy (the same arrangement for Float32 rows was measured
// slower than the general kernel, 5490 against 5750 GB/s, and is not kept): the general kernel above holds x, dy and gamma
// widened to Float32 beside its two sets of accumulators (127 registers, two blocks of 256 threads per SM),
// and at that occupancy it waits on issue slots rather than on HBM.  Here x and dy stay packed as they were
// loaded (eight registers per array instead of sixteen), gamma is re-read from L1, the dgamma / dbeta
// accumulators live in shared memory (each thread's own slots, one 128-bit read-modify-write per four
// elements per row), and the row is unpacked twice -- once for the two row sums and the accumulators, once
// for dx -- which costs a few shifts and buys twice the resident warps.
template <int VPT>
__global__ void __launch_bounds__(256, 4) layernorm_bwd_compact(RowArgs a) {
    using R = Row<__nv_bfloat16, true, VPT>;
    __shared__ float red[2 * 32 * kRedWidth];
    __shared__ float4 acc[2 * 2 * VPT * 256];   // [dgamma | dbeta][chunk][half of the chunk][thread]
    RowCtx c = make_row_ctx(a.tpr, red);
    const int tid = threadIdx.x;
    const __nv_bfloat16 *x = static_cast<const __nv_bfloat16 *>(a.in0);
    const __nv_bfloat16 *dy = static_cast<const __nv_bfloat16 *>(a.in1);
    const __nv_bfloat16 *gamma = static_cast<const __nv_bfloat16 *>(a.gamma);
    __nv_bfloat16 *dx = static_cast<__nv_bfloat16 *>(a.out0);
    const float *mean_in = static_cast<const float *>(a.cstat0), *rstd_in = static_cast<const float *>(a.cstat1);
#pragma unroll
    for (int i = 0; i < 2 * 2 * VPT; i++) acc[i * 256 + tid] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const float inv_n = 1.0f / static_cast<float>(a.n);
    const long long groups = a.rows / a.rpc;
    for (long long g = blockIdx.x; g < groups; g += gridDim.x) {
        const long long r = g * a.rpc + c.slot;
        uint4 rx[VPT], rd[VPT];
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            rx[k] = __ldcs(reinterpret_cast<const uint4 *>(x + r * a.ld + R::at(k, c.t, a.tpr)));
            rd[k] = __ldcs(reinterpret_cast<const uint4 *>(dy + r * a.ld + R::at(k, c.t, a.tpr)));
        }
        const float mean = mean_in[r], rstd = rstd_in[r];
        const float2 rs2 = make_float2(rstd, rstd), off2 = make_float2(-mean * rstd, -mean * rstd);
        float2 sa = make_float2(0.0f, 0.0f), sb = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const uint4 gq = __ldg(reinterpret_cast<const uint4 *>(gamma + R::at(k, c.t, a.tpr)));
            const uint32_t xw[4] = {rx[k].x, rx[k].y, rx[k].z, rx[k].w}, dw[4] = {rd[k].x, rd[k].y, rd[k].z, rd[k].w},
                           gw[4] = {gq.x, gq.y, gq.z, gq.w};
#pragma unroll
            for (int h = 0; h < 2; h++) {   // four elements = one accumulator slot at a time
                float4 *slot_g = &acc[((2 * k + h) * 256) + tid], *slot_b = &acc[((2 * VPT + 2 * k + h) * 256) + tid];
                float4 ag = *slot_g, ab = *slot_b;
                float *pg = &ag.x, *pb = &ab.x;
#pragma unroll
                for (int w = 0; w < 2; w++) {
                    float2 xv, dy2, gm;
                    unpack_bf16x2(xw[2 * h + w], xv.x, xv.y);
                    unpack_bf16x2(dw[2 * h + w], dy2.x, dy2.y);
                    unpack_bf16x2(gw[2 * h + w], gm.x, gm.y);
                    const float2 xh = __ffma2_rn(xv, rs2, off2);
                    const float2 gh = __fmul2_rn(dy2, gm);
                    sa = __fadd2_rn(sa, gh);
                    sb = __ffma2_rn(gh, xh, sb);
                    const float2 g2 = __ffma2_rn(dy2, xh, make_float2(pg[2 * w], pg[2 * w + 1]));
                    const float2 b2 = __fadd2_rn(make_float2(pb[2 * w], pb[2 * w + 1]), dy2);
                    pg[2 * w] = g2.x; pg[2 * w + 1] = g2.y;
                    pb[2 * w] = b2.x; pb[2 * w + 1] = b2.y;
                }
                *slot_g = ag;
                *slot_b = ab;
            }
        }
        float s2[2] = {sa.x + sa.y, sb.x + sb.y};
        row_allreduce<2>(s2, c, SumOp());
        const float c1 = s2[0] * inv_n, c2 = s2[1] * inv_n;
        const float2 nc1 = make_float2(-c1, -c1), nc2 = make_float2(-c2, -c2);
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const uint4 gq = __ldg(reinterpret_cast<const uint4 *>(gamma + R::at(k, c.t, a.tpr)));
            const uint32_t xw[4] = {rx[k].x, rx[k].y, rx[k].z, rx[k].w}, dw[4] = {rd[k].x, rd[k].y, rd[k].z, rd[k].w},
                           gw[4] = {gq.x, gq.y, gq.z, gq.w};
            uint32_t ow[4];
#pragma unroll
            for (int w = 0; w < 4; w++) {
                float2 xv, dy2, gm;
                unpack_bf16x2(xw[w], xv.x, xv.y);
                unpack_bf16x2(dw[w], dy2.x, dy2.y);
                unpack_bf16x2(gw[w], gm.x, gm.y);
                const float2 xh = __ffma2_rn(xv, rs2, off2);
                const float2 gh = __fmul2_rn(dy2, gm);
                const float2 u = __fmul2_rn(__ffma2_rn(xh, nc2, __fadd2_rn(gh, nc1)), rs2);
                ow[w] = pack_bf16x2(u.x, u.y);
            }
            __stcs(reinterpret_cast<uint4 *>(dx + r * a.ld + R::at(k, c.t, a.tpr)), make_uint4(ow[0], ow[1], ow[2], ow[3]));
        }
    }
    if (a.part0) {
        const long long p = static_cast<long long>(blockIdx.x) * a.rpc + c.slot;
#pragma unroll
        for (int k = 0; k < VPT; k++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int col = R::at(k, c.t, a.tpr) + 4 * h;
                *reinterpret_cast<float4 *>(a.part0 + p * a.n + col) = acc[((2 * k + h) * 256) + tid];
                *reinterpret_cast<float4 *>(a.part1 + p * a.n + col) = acc[((2 * VPT + 2 * k + h) * 256) + tid];
            }
    }
}

// The LayerNorm backward for rows of 1024, 2048 or 4096 elements with saved statistics, fed through shared memory:
// one thread issues bulk copies (cp.async.bulk, completion counted on an mbarrier) of whole rows of x and dy into a
// ring of stages, several rows ahead of the arithmetic, so the bytes in flight per SM are set by the ring's depth and
// not by how many registers the resident threads can spare for loads.  512 threads, eight elements each; a thread owns
// the same eight columns of every row, so gamma is widened once per launch and the dgamma / dbeta sums are sixteen
// registers that stay in the thread until the end; x-hat and dy*gamma stay widened across the row's two sums.  A stage
// is free once every thread has passed the barrier inside the row sums' exchange, and is refilled there.
// Every wait on a stage is bounded (about two seconds): a thread that gives up records it in g_rows_error and runs on
// without waiting again, so the launch ends and the host can read the status.
__device__ int g_rows_error = 0;

template <typename T> struct Eight;
template <> struct Eight<__nv_bfloat16> {
    static constexpr int NV = 1;
    static __device__ __forceinline__ int col(int k, int t, int tpr) { return t * 8; }
    static __device__ __forceinline__ void load(const __nv_bfloat16 *row, int t, int tpr, float2 (&v)[4]) {
        const uint4 q = *reinterpret_cast<const uint4 *>(row + t * 8);
        unpack_bf16x2(q.x, v[0].x, v[0].y); unpack_bf16x2(q.y, v[1].x, v[1].y);
        unpack_bf16x2(q.z, v[2].x, v[2].y); unpack_bf16x2(q.w, v[3].x, v[3].y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *row, int t, int tpr, const float2 (&v)[4]) {
        __stcs(reinterpret_cast<uint4 *>(row + t * 8),
               make_uint4(pack_bf16x2(v[0].x, v[0].y), pack_bf16x2(v[1].x, v[1].y), pack_bf16x2(v[2].x, v[2].y),
                          pack_bf16x2(v[3].x, v[3].y)));
    }
};
template <> struct Eight<float> {
    static constexpr int NV = 2;
    static __device__ __forceinline__ int col(int k, int t, int tpr) { return (k * tpr + t) * 4; }
    static __device__ __forceinline__ void load(const float *row, int t, int tpr, float2 (&v)[4]) {
        const float4 p = *reinterpret_cast<const float4 *>(row + t * 4);
        const float4 q = *reinterpret_cast<const float4 *>(row + (tpr + t) * 4);
        v[0] = make_float2(p.x, p.y); v[1] = make_float2(p.z, p.w);
        v[2] = make_float2(q.x, q.y); v[3] = make_float2(q.z, q.w);
    }
    static __device__ __forceinline__ void store(float *row, int t, int tpr, const float2 (&v)[4]) {
        __stcs(reinterpret_cast<float4 *>(row + t * 4), make_float4(v[0].x, v[0].y, v[1].x, v[1].y));
        __stcs(reinterpret_cast<float4 *>(row + (tpr + t) * 4), make_float4(v[2].x, v[2].y, v[3].x, v[3].y));
    }
};
// the eight Float32 partial sums of a thread, at the columns the thread owns
template <typename T>
__device__ __forceinline__ void store_sums(float *row, int t, int tpr, const float2 (&v)[4]) {
    constexpr int half = Eight<T>::NV == 1 ? 4 : 0;   // BFloat16: eight neighbouring columns; Float32: two groups of four
    *reinterpret_cast<float4 *>(row + Eight<T>::col(0, t, tpr)) = make_float4(v[0].x, v[0].y, v[1].x, v[1].y);
    *reinterpret_cast<float4 *>(row + Eight<T>::col(Eight<T>::NV - 1, t, tpr) + half) = make_float4(v[2].x, v[2].y, v[3].x, v[3].y);
}

__device__ __forceinline__ bool stage_wait(uint64_t *bar, uint32_t parity) {
    if (sm100::mbar_wait(bar, parity, 2048)) return true;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    while (true) {
        if (sm100::mbar_wait(bar, parity, 1024)) return true;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > 2000000000ull) return false;
    }
}

// The NV sums of a turn (NV = 2 or 4) over the `wpr` warps that share a row, in two halves around the block's
// barrier.  Inside a warp the values are folded
// butterfly-wise: at the first steps each lane hands half of its values to its partner and keeps the other half, so
// NV values cost  NV/2 + ... + 1 + (5 - log2 NV)  shuffles instead of 5 NV, and each lane ends with the warp's total
// of ONE value; after the exchange through shared memory the same is done over the warps' partial sums, and the
// totals are handed round.  The order of the additions is fixed.  `red`: this phase's [warps of the block][NV].
// BUTTERFLY = false is the plain form (every lane folds every value): measured faster for Float32 rows, which wait
// on HBM and on the chain's latency rather than on issue slots (LayerNorm backward 4096 x 65536: 0.527 ms against 0.548).
template <int NV, bool BUTTERFLY>
__device__ __forceinline__ void turn_sums_put(float (&v)[NV], float (*red)[NV], int lane, int warp) {
    static_assert(NV == 2 || NV == 4, "two or four sums a turn");
    if constexpr (!BUTTERFLY) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int i = 0; i < NV; i++) v[i] += __shfl_xor_sync(0xffffffffu, v[i], o);
        if (lane == 0)
#pragma unroll
            for (int i = 0; i < NV; i++) red[warp][i] = v[i];
    } else if constexpr (NV == 4) {
        const bool up16 = lane & 16, up8 = lane & 8;
        float k0 = up16 ? v[2] : v[0], k1 = up16 ? v[3] : v[1];
        k0 += __shfl_xor_sync(0xffffffffu, up16 ? v[0] : v[2], 16);
        k1 += __shfl_xor_sync(0xffffffffu, up16 ? v[1] : v[3], 16);
        float k = (up8 ? k1 : k0) + __shfl_xor_sync(0xffffffffu, up8 ? k0 : k1, 8);
        k += __shfl_xor_sync(0xffffffffu, k, 4);
        k += __shfl_xor_sync(0xffffffffu, k, 2);
        k += __shfl_xor_sync(0xffffffffu, k, 1);
        if ((lane & 7) == 0) red[warp][lane >> 3] = k;      // lane holds value 2 * bit 4 + bit 3
    } else {
        const bool up16 = lane & 16;
        float k = (up16 ? v[1] : v[0]) + __shfl_xor_sync(0xffffffffu, up16 ? v[0] : v[1], 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) k += __shfl_xor_sync(0xffffffffu, k, o);
        if ((lane & 15) == 0) red[warp][lane >> 4] = k;     // lane holds value bit 4
    }
}
// After the block's barrier: the row's totals from its warps' partial sums.
template <int NV, bool BUTTERFLY>
__device__ __forceinline__ void turn_sums_get(float (&v)[NV], const float (*red)[NV], int lane, int slot, int wpr) {
    const float(*mine)[NV] = red + slot * wpr;
    if (BUTTERFLY && wpr == 16) {
        // lanes 0-15 take one value of the sixteen warps, lanes 16-31 another (two rounds for four values)
        float a = mine[lane & 15][lane >> 4], b = NV == 4 ? mine[lane & 15][2 + (lane >> 4)] : 0.0f;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            a += __shfl_xor_sync(0xffffffffu, a, o);
            if constexpr (NV == 4) b += __shfl_xor_sync(0xffffffffu, b, o);
        }
        v[0] = __shfl_sync(0xffffffffu, a, 0);
        v[1] = __shfl_sync(0xffffffffu, a, 16);
        if constexpr (NV == 4) {
            v[2] = __shfl_sync(0xffffffffu, b, 0);
            v[3] = __shfl_sync(0xffffffffu, b, 16);
        }
    } else {
#pragma unroll
        for (int i = 0; i < NV; i++) v[i] = mine[lane & (wpr - 1)][i];
        for (int o = wpr >> 1; o > 0; o >>= 1)
#pragma unroll
            for (int i = 0; i < NV; i++) v[i] += __shfl_xor_sync(0xffffffffu, v[i], o);
    }
}

constexpr int kStagedThreads = 512;
constexpr int kStagedRowsBf16 = 2;   // BFloat16 rows a block takes per turn

// R rows a turn: the chain  row sums -> shuffles -> exchange -> shuffles  is as long for R rows' sums as for one, and
// with two blocks of 512 threads per SM that chain, not HBM, set the pace of BFloat16 rows (measured: 0.339 ms with it,
// 0.256 ms with the sums left out, 4096 x 65536).  With R > 1 nothing of a row but its sums is kept across the
// exchange: the second pass reads the row from its stage again, so a stage is handed back one turn later.
template <typename T, int R>
__global__ void __launch_bounds__(kStagedThreads, 2) layernorm_bwd_staged(RowArgs a) {
    using E = Eight<T>;
    constexpr bool REREAD = R > 1;
    extern __shared__ __align__(128) unsigned char staged_smem[];
    __shared__ float red[2][kStagedThreads / 32][2 * R];
    uint64_t *full = reinterpret_cast<uint64_t *>(staged_smem);      // one barrier per stage, in the first 128 bytes
    T *ring = reinterpret_cast<T *>(staged_smem + 128);              // [stage][row of the turn][x | dy][row slot][n]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tpr = a.tpr, slot = tid / tpr, t = tid - slot * tpr, wpr = tpr >> 5;
    const int stages = a.splits;
    const T *x = static_cast<const T *>(a.in0);
    const T *dy = static_cast<const T *>(a.in1);
    T *dx = static_cast<T *>(a.out0);
    const float *mean_in = static_cast<const float *>(a.cstat0), *rstd_in = static_cast<const float *>(a.cstat1);
    const long long turn_rows = static_cast<long long>(R) * a.rpc;
    const long long turns = a.rows / turn_rows, step = gridDim.x;
    const size_t row_elems = static_cast<size_t>(2) * a.rpc * a.n;   // one row slot group: x rows, then dy rows
    const size_t stage_elems = R * row_elems;
    const uint32_t row_bytes = static_cast<uint32_t>(a.n * sizeof(T));

    auto fill = [&](int stage, long long turn) {   // one thread: the turn's rows of x and dy
        sm100::mbar_arrive_expect_tx(&full[stage], static_cast<uint32_t>(2 * turn_rows) * row_bytes);
        for (int j = 0; j < R; j++) {
            T *dst = ring + stage * stage_elems + j * row_elems;
            for (int i = 0; i < a.rpc; i++) {
                const long long r = turn * turn_rows + static_cast<long long>(j) * a.rpc + i;
                sm100::bulk_load(dst + static_cast<size_t>(i) * a.n, x + r * a.ld, row_bytes, &full[stage]);
                sm100::bulk_load(dst + static_cast<size_t>(a.rpc + i) * a.n, dy + r * a.ld, row_bytes, &full[stage]);
            }
        }
    };
    if (tid == 0) {
        for (int i = 0; i < stages; i++) sm100::mbar_init(&full[i], 1);
        sm100::fence_barrier_init();
    }
    __syncthreads();
    if (tid == 0)
        for (int i = 0; i < stages; i++)
            if (blockIdx.x + i * step < turns) fill(i, blockIdx.x + i * step);

    float2 gm[4], dg[4], db[4];
    E::load(static_cast<const T *>(a.gamma), t, tpr, gm);
#pragma unroll
    for (int w = 0; w < 4; w++) dg[w] = db[w] = make_float2(0.0f, 0.0f);
    const float inv_n = 1.0f / static_cast<float>(a.n);
    // the rows' saved statistics, fetched a turn ahead
    float mean_next[R], rstd_next[R];
    auto fetch_stats = [&](long long turn) {
#pragma unroll
        for (int j = 0; j < R; j++) {
            const long long r = turn * turn_rows + static_cast<long long>(j) * a.rpc + slot;
            mean_next[j] = turn < turns ? __ldg(mean_in + r) : 0.0f;
            rstd_next[j] = turn < turns ? __ldg(rstd_in + r) : 0.0f;
        }
    };
    fetch_stats(blockIdx.x);
    bool failed = false;
    int stage = 0, phase = 0, last_stage = -1;
    uint32_t parity = 0;
    for (long long g = blockIdx.x; g < turns; g += step) {
        float mean[R], rstd[R];
#pragma unroll
        for (int j = 0; j < R; j++) { mean[j] = mean_next[j]; rstd[j] = rstd_next[j]; }
        fetch_stats(g + step);
        if (!failed && !stage_wait(&full[stage], parity)) {
            failed = true;
            atomicCAS(&g_rows_error, 0, 1);
        }
        const T *sx = ring + stage * stage_elems + static_cast<size_t>(slot) * a.n;
        float2 xh[R][4], gh[R][4];
        float sums[2 * R];
#pragma unroll
        for (int j = 0; j < R; j++) {
            E::load(sx + j * row_elems, t, tpr, xh[j]);
            E::load(sx + j * row_elems + static_cast<size_t>(a.rpc) * a.n, t, tpr, gh[j]);
            const float2 rs2 = make_float2(rstd[j], rstd[j]), off2 = make_float2(-mean[j] * rstd[j], -mean[j] * rstd[j]);
            float2 sa = make_float2(0.0f, 0.0f), sb = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const float2 d2 = gh[j][w];
                xh[j][w] = __ffma2_rn(xh[j][w], rs2, off2);
                gh[j][w] = __fmul2_rn(d2, gm[w]);
                sa = __fadd2_rn(sa, gh[j][w]);
                sb = __ffma2_rn(gh[j][w], xh[j][w], sb);
                dg[w] = __ffma2_rn(d2, xh[j][w], dg[w]);
                db[w] = __fadd2_rn(db[w], d2);
            }
            sums[2 * j] = sa.x + sa.y;
            sums[2 * j + 1] = sb.x + sb.y;
        }
        turn_sums_put<2 * R, sizeof(T) == 2>(sums, red[phase], lane, warp);
        __syncthreads();
        // every thread is past its reads of a stage (this turn's when the rows stay in registers, the turn
        // before's when the second pass reads them again): hand it back
        if (tid == 0) {
            const int back = REREAD ? last_stage : stage;
            const long long ahead = g + (REREAD ? stages - 1 : stages) * step;
            if (back >= 0 && ahead < turns) fill(back, ahead);
        }
        last_stage = stage;
        turn_sums_get<2 * R, sizeof(T) == 2>(sums, red[phase], lane, slot, wpr);
        phase ^= 1;
#pragma unroll
        for (int j = 0; j < R; j++) {
            const long long r = g * turn_rows + static_cast<long long>(j) * a.rpc + slot;
            const float c1 = sums[2 * j] * inv_n, c2 = sums[2 * j + 1] * inv_n;
            const float2 nc1 = make_float2(-c1, -c1), nc2 = make_float2(-c2, -c2), rs2 = make_float2(rstd[j], rstd[j]);
            if constexpr (REREAD) {
                const float2 off2 = make_float2(-mean[j] * rstd[j], -mean[j] * rstd[j]);
                E::load(sx + j * row_elems, t, tpr, xh[j]);
                E::load(sx + j * row_elems + static_cast<size_t>(a.rpc) * a.n, t, tpr, gh[j]);
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    xh[j][w] = __ffma2_rn(xh[j][w], rs2, off2);
                    gh[j][w] = __fmul2_rn(gh[j][w], gm[w]);
                }
            }
#pragma unroll
            for (int w = 0; w < 4; w++)
                xh[j][w] = __fmul2_rn(__ffma2_rn(xh[j][w], nc2, __fadd2_rn(gh[j][w], nc1)), rs2);
            E::store(dx + r * a.ld, t, tpr, xh[j]);
        }
        if (++stage == stages) { stage = 0; parity ^= 1; }
    }
    if (a.part0) {
        const long long p = static_cast<long long>(blockIdx.x) * a.rpc + slot;
        store_sums<T>(a.part0 + p * a.n, t, tpr, dg);
        store_sums<T>(a.part1 + p * a.n, t, tpr, db);
    }
}

// The LayerNorm forward on the same footing: rows arrive through the ring, gamma and beta are widened once per
// launch, R rows share each of the two exchanges (sum, then centred squares: the two-pass variance of the other
// forward kernels), and a stage is handed back as soon as its rows sit in registers.
template <typename T, int R>
__global__ void __launch_bounds__(kStagedThreads, 2) layernorm_fwd_staged(RowArgs a) {
    using E = Eight<T>;
    extern __shared__ __align__(128) unsigned char staged_smem[];
    __shared__ float red[2][kStagedThreads / 32][R];
    uint64_t *full = reinterpret_cast<uint64_t *>(staged_smem);
    T *ring = reinterpret_cast<T *>(staged_smem + 128);              // [stage][row of the turn][row slot][n]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tpr = a.tpr, slot = tid / tpr, t = tid - slot * tpr, wpr = tpr >> 5;
    const int stages = a.splits;
    const T *x = static_cast<const T *>(a.in0);
    T *y = static_cast<T *>(a.out0);
    const long long turn_rows = static_cast<long long>(R) * a.rpc;
    const long long turns = a.rows / turn_rows, step = gridDim.x;
    const size_t stage_elems = static_cast<size_t>(turn_rows) * a.n;
    const uint32_t row_bytes = static_cast<uint32_t>(a.n * sizeof(T));

    auto fill = [&](int stage, long long turn) {
        sm100::mbar_arrive_expect_tx(&full[stage], static_cast<uint32_t>(turn_rows) * row_bytes);
        for (int i = 0; i < turn_rows; i++)
            sm100::bulk_load(ring + stage * stage_elems + static_cast<size_t>(i) * a.n, x + (turn * turn_rows + i) * a.ld,
                             row_bytes, &full[stage]);
    };
    if (tid == 0) {
        for (int i = 0; i < stages; i++) sm100::mbar_init(&full[i], 1);
        sm100::fence_barrier_init();
    }
    __syncthreads();
    if (tid == 0)
        for (int i = 0; i < stages; i++)
            if (blockIdx.x + i * step < turns) fill(i, blockIdx.x + i * step);

    float2 gm[4], bt[4];
    E::load(static_cast<const T *>(a.gamma), t, tpr, gm);
    if (a.beta) E::load(static_cast<const T *>(a.beta), t, tpr, bt);
    else
#pragma unroll
        for (int w = 0; w < 4; w++) bt[w] = make_float2(0.0f, 0.0f);
    const float inv_n = 1.0f / static_cast<float>(a.n);
    bool failed = false;
    int stage = 0, phase = 0;
    uint32_t parity = 0;
    auto exchange = [&](float (&v)[R]) {
        turn_sums_put<R, sizeof(T) == 2>(v, red[phase], lane, warp);
        __syncthreads();
        turn_sums_get<R, sizeof(T) == 2>(v, red[phase], lane, slot, wpr);
        phase ^= 1;
    };
    for (long long g = blockIdx.x; g < turns; g += step) {
        if (!failed && !stage_wait(&full[stage], parity)) {
            failed = true;
            atomicCAS(&g_rows_error, 0, 1);
        }
        const T *sx = ring + stage * stage_elems + static_cast<size_t>(slot) * a.n;
        float2 v[R][4];
        float sums[R];
#pragma unroll
        for (int j = 0; j < R; j++) {
            E::load(sx + static_cast<size_t>(j) * a.rpc * a.n, t, tpr, v[j]);
            const float2 s2 = __fadd2_rn(__fadd2_rn(v[j][0], v[j][1]), __fadd2_rn(v[j][2], v[j][3]));
            sums[j] = s2.x + s2.y;
        }
        exchange(sums);
        // the rows are in registers and every thread is past the barrier: hand the stage back
        if (tid == 0 && g + stages * step < turns) fill(stage, g + stages * step);
        float mean[R];
#pragma unroll
        for (int j = 0; j < R; j++) {
            mean[j] = sums[j] * inv_n;
            const float2 nm = make_float2(-mean[j], -mean[j]);
            float2 q = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int w = 0; w < 4; w++) {
                v[j][w] = __fadd2_rn(v[j][w], nm);
                q = __ffma2_rn(v[j][w], v[j][w], q);
            }
            sums[j] = q.x + q.y;
        }
        exchange(sums);
#pragma unroll
        for (int j = 0; j < R; j++) {
            const long long r = g * turn_rows + static_cast<long long>(j) * a.rpc + slot;
            const float var = sums[j] * inv_n + a.eps;
            float rstd = rsqrtf(var);
            rstd = rstd * fmaf(-0.5f * var * rstd, rstd, 1.5f);   // one Newton step: within an ulp of 1 / sqrt
            if (t == 0) {
                if (a.stat0) static_cast<float *>(a.stat0)[r] = mean[j];
                if (a.stat1) static_cast<float *>(a.stat1)[r] = rstd;
            }
            const float2 rs2 = make_float2(rstd, rstd);
#pragma unroll
            for (int w = 0; w < 4; w++) v[j][w] = __ffma2_rn(__fmul2_rn(v[j][w], rs2), gm[w], bt[w]);
            E::store(y + r * a.ld, t, tpr, v[j]);
        }
        if (++stage == stages) { stage = 0; parity ^= 1; }
    }
}

// ---------------------------------------- LayerNorm backward, rows beyond the resident schedule ----
//
// A row that does not fit one block's registers is streamed instead: one block of 512 threads walks the
// row three times (four when the forward saved no statistics) -- the row sums  sum(dy gamma)  and
// sum(dy gamma xh), then dx -- and the later walks find the row in L2.  dgamma / dbeta are column sums
// over all rows, taken by a second kernel whose threads own one column each: row slabs x column blocks,
// rows in order inside a slab, the slabs merged in order by merge_parts.
constexpr int kLongSlabsMax = 64;

template <typename T, bool VEC>
__global__ void __launch_bounds__(kResidentMaxThreads) layernorm_bwd_long(RowArgs a) {
    using A = Access<T, VEC>;
    constexpr int E = A::EPV;
    __shared__ float red[2 * 32 * kRedWidth];
    RowCtx c = make_row_ctx(kResidentMaxThreads, red);
    const float fn = static_cast<float>(a.n);
    const int stride = kResidentMaxThreads * E;
    const T *gamma = static_cast<const T *>(a.gamma);
    for (long long r = blockIdx.x; r < a.rows; r += gridDim.x) {
        const T *x = static_cast<const T *>(a.in0) + r * a.ld;
        const T *dy = static_cast<const T *>(a.in1) + r * a.ld;
        T *dx = static_cast<T *>(a.out0) + r * a.ld;
        float mean, rstd;
        if (a.cstat0) {
            mean = static_cast<const float *>(a.cstat0)[r];
            rstd = static_cast<const float *>(a.cstat1)[r];
        } else {
            float s = 0.0f;
            for (int i = c.t * E; i < a.n; i += stride) {
                float v[E];
                A::load_cached(x + i, v);
#pragma unroll
                for (int e = 0; e < E; e++) s += v[e];
            }
            mean = row_allreduce1(s, c, SumOp()) / fn;
            float q = 0.0f;
            for (int i = c.t * E; i < a.n; i += stride) {
                float v[E];
                A::load_cached(x + i, v);
#pragma unroll
                for (int e = 0; e < E; e++) q = fmaf(v[e] - mean, v[e] - mean, q);
            }
            rstd = 1.0f / sqrtf(row_allreduce1(q, c, SumOp()) / fn + a.eps);
            if (c.t == 0 && a.stat0) {   // the column sums read them
                static_cast<float *>(a.stat0)[r] = mean;
                static_cast<float *>(a.stat1)[r] = rstd;
            }
        }
        float s2[2] = {0.0f, 0.0f};
        for (int i = c.t * E; i < a.n; i += stride) {
            float v[E], d[E], g[E];
            A::load_cached(x + i, v);
            A::load_cached(dy + i, d);
            A::load_cached(gamma + i, g);
#pragma unroll
            for (int e = 0; e < E; e++) {
                const float gh = d[e] * g[e];
                s2[0] += gh;
                s2[1] = fmaf(gh, (v[e] - mean) * rstd, s2[1]);
            }
        }
        row_allreduce<2>(s2, c, SumOp());
        const float c1 = s2[0] / fn, c2 = s2[1] / fn;
        for (int i = c.t * E; i < a.n; i += stride) {
            float v[E], d[E], g[E];
            A::load(x + i, v);
            A::load(dy + i, d);
            A::load_cached(gamma + i, g);
#pragma unroll
            for (int e = 0; e < E; e++) d[e] = rstd * ((d[e] * g[e] - c1) - (v[e] - mean) * rstd * c2);
            A::store(dx + i, d);
        }
    }
}

// part0[slab][col] = sum over the slab's rows of dy xh, part1[slab][col] = sum of dy
template <typename T>
__global__ void __launch_bounds__(256) layernorm_bwd_colsums(const T *x, const T *dy, const float *mean,
                                                             const float *rstd, float *part0, float *part1, int n,
                                                             long long rows, long long ld, int slabs) {
    const int col = blockIdx.x * 256 + threadIdx.x;
    const long long per = (rows + slabs - 1) / slabs;
    const long long r0 = blockIdx.y * per;
    const long long r1 = r0 + per < rows ? r0 + per : rows;
    if (col >= n) return;
    float dg = 0.0f, db = 0.0f;
    for (long long r = r0; r < r1; r++) {
        float v, d;
        Access<T, false>::load_cached(x + r * ld + col, &v);
        Access<T, false>::load_cached(dy + r * ld + col, &d);
        dg = fmaf(d, (v - mean[r]) * rstd[r], dg);
        db += d;
    }
    part0[static_cast<long long>(blockIdx.y) * n + col] = dg;
    part1[static_cast<long long>(blockIdx.y) * n + col] = db;
}

// Column sums of the partial dgamma / dbeta rows: 32 columns x 8 lanes per
// block; each lane strides over the parts in order, the 8 lanes merge in a
// fixed tree.  Output in the element type, rounded once.
template <typename T>
__global__ void __launch_bounds__(256) merge_parts(const float *part0, const float *part1, T *out0, T *out1,
                                                   int n, int parts) {
    __shared__ float sm[2][8][33];
    const int col = blockIdx.x * 32 + (threadIdx.x & 31);
    const int lane = threadIdx.x >> 5;
    float s0 = 0.0f, s1 = 0.0f;
    if (col < n)
        for (int p = lane; p < parts; p += 8) {
            s0 += part0[static_cast<long long>(p) * n + col];
            s1 += part1[static_cast<long long>(p) * n + col];
        }
    sm[0][lane][threadIdx.x & 31] = s0;
    sm[1][lane][threadIdx.x & 31] = s1;
    __syncthreads();
    if (lane == 0 && col < n) {
        float t0 = 0.0f, t1 = 0.0f;
#pragma unroll
        for (int l = 0; l < 8; l++) {
            t0 += sm[0][l][threadIdx.x];
            t1 += sm[1][l][threadIdx.x];
        }
        float o0[1] = {t0}, o1[1] = {t1};
        if (out0) Access<T, false>::store(out0 + col, o0);
        if (out1) Access<T, false>::store(out1 + col, o1);
    }
}

// The same column sums with 128-bit reads, for row lengths that are a multiple of four: 16 threads side by
// side take 64 columns (256 contiguous bytes of a partial row), 16 such groups stride over the parts, and the
// 16 per-group sums of a column merge in a fixed order.  The narrow kernel above reads 128 bytes per part row
// and block, which left the merge at a fraction of the memory rate once the backward ran 4 blocks per SM.
template <typename T>
__global__ void __launch_bounds__(256) merge_parts_wide(const float *part0, const float *part1, T *out0, T *out1, int n, int parts) {
    __shared__ float4 sm[2][16][17];
    const int cg = threadIdx.x & 15, lane = threadIdx.x >> 4;
    const int col = blockIdx.x * 64 + cg * 4;
    float4 s0 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), s1 = s0;
    if (col < n) {
#pragma unroll 4
        for (int p = lane; p < parts; p += 16) {
            const float4 a = __ldcs(reinterpret_cast<const float4 *>(part0 + static_cast<long long>(p) * n + col));
            const float4 b = __ldcs(reinterpret_cast<const float4 *>(part1 + static_cast<long long>(p) * n + col));
            s0.x += a.x; s0.y += a.y; s0.z += a.z; s0.w += a.w;
            s1.x += b.x; s1.y += b.y; s1.z += b.z; s1.w += b.w;
        }
    }
    sm[0][lane][cg] = s0;
    sm[1][lane][cg] = s1;
    __syncthreads();
    if (lane < 2 && col < n) {   // lane 0 finishes dgamma, lane 1 dbeta
        float4 t = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int l = 0; l < 16; l++) {
            const float4 v = sm[lane][l][cg];
            t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
        }
        T *out = lane == 0 ? out0 : out1;
        if (out) {
            const float r[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int e = 0; e < 4; e++) Access<T, false>::store(out + col + e, &r[e]);
        }
    }
}

__global__ void fill_stat(void *p, long long count, float value, int as_bf16) {
    long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i < count) store_stat(p, i, value, as_bf16);
}

// --------------------------------------------------------------- split ------
// Block b folds chunk (b % splits) of row (b / splits); a chunk is
// kSplitThreads x E elements held in registers.  States live in part0 as
// float4 per (row, chunk).

template <typename T, bool VEC, int VPT>
struct Chunk {
    using R = Row<T, VEC, VPT>;
    static constexpr int LEN = kSplitThreads * R::E;
    long long r;
    int c, base, len;
    __device__ __forceinline__ Chunk(const RowArgs &a) {
        r = blockIdx.x / a.splits;
        c = static_cast<int>(blockIdx.x - r * a.splits);
        base = c * LEN;
        len = min(LEN, a.n - base);
    }
};

// merge of the row's log-sum-exp states (m, s): the maximum first, then each
// sum moved to it once (the reference's RebasedSums, src/Compiler/IR/folds.jl:240-264)
__device__ __forceinline__ float merged_lse(const float4 *states, int splits, RowCtx &c) {
    float m = -INFINITY;
    for (int i = threadIdx.x; i < splits; i += blockDim.x) m = fmaxf(m, states[i].x);
    m = row_allreduce1(m, c, MaxOp());
    const float sh = (fabsf(m) <= 3.402823466e38f) ? m : 0.0f;
    float s = 0.0f;
    for (int i = threadIdx.x; i < splits; i += blockDim.x) {
        const float4 st = states[i];
        const float shi = (fabsf(st.x) <= 3.402823466e38f) ? st.x : 0.0f;
        s += st.y * fast_exp2((shi - sh) * kLog2e);
    }
    s = row_allreduce1(s, c, SumOp());
    return m + logf(s);
}

template <typename T, bool VEC, int VPT>
__global__ void __launch_bounds__(kSplitThreads) softmax_fwd_split_fold(RowArgs a) {
    using R = Row<T, VEC, VPT>;
    __shared__ float red[2 * 32 * kRedWidth];
    RowCtx c = make_row_ctx(kSplitThreads, red);
    Chunk<T, VEC, VPT> ch(a);
    float v[R::E];
    R::load(v, static_cast<const T *>(a.in0) + ch.r * a.ld + ch.base, ch.len, c.t, kSplitThreads, -INFINITY, true);
    float m = -INFINITY;
#pragma unroll
    for (int e = 0; e < R::E; e++) m = fmaxf(m, v[e]);
    m = row_allreduce1(m, c, MaxOp());
    const float sh = (fabsf(m) <= 3.402823466e38f) ? m : 0.0f;
    float s = 0.0f;
#pragma unroll
    for (int e = 0; e < R::E; e++) s += fast_exp2((v[e] - sh) * kLog2e);
    s = row_allreduce1(s, c, SumOp());
    if (threadIdx.x == 0) reinterpret_cast<float4 *>(a.part0)[blockIdx.x] = make_float4(m, s, 0.0f, 0.0f);
}

template <typename T, bool VEC, int VPT>
__global__ void __launch_bounds__(kSplitThreads) softmax_fwd_split_write(RowArgs a) {
    using R = Row<T, VEC, VPT>;
    __shared__ float red[2 * 32 * kRedWidth];
    RowCtx c = make_row_ctx(kSplitThreads, red);
    Chunk<T, VEC, VPT> ch(a);
    const float lse = merged_lse(reinterpret_cast<const float4 *>(a.part0) + ch.r * a.splits, a.splits, c);
    if (ch.c == 0 && threadIdx.x == 0 && a.stat0) store_stat(a.stat0, ch.r, lse, a.stat_bf16);
    float v[R::E];
    R::load(v, static_cast<const T *>(a.in0) + ch.r * a.ld + ch.base, ch.len, c.t, kSplitThreads, 0.0f, true);
    const float off = lse * kLog2e;
#pragma unroll
    for (int e = 0; e < R::E; e++) v[e] = fast_exp2(fmaf(v[e], kLog2e, -off));
    R::store(v, static_cast<T *>(a.out0) + ch.r * a.ld + ch.base, ch.len, c.t, kSplitThreads, true);
}

template <typename T, bool VEC, int VPT>
__global__ void __launch_bounds__(kSplitThreads) softmax_bwd_split_fold(RowArgs a) {
    using R = Row<T, VEC, VPT>;
    __shared__ float red[2 * 32 * kRedWidth];
    RowCtx c = make_row_ctx(kSplitThreads, red);
    Chunk<T, VEC, VPT> ch(a);
    float y[R::E], d[R::E];
    R::load(y, static_cast<const T *>(a.in0) + ch.r * a.ld + ch.base, ch.len, c.t, kSplitThreads,
            a.cstat0 ? -INFINITY : 0.0f, true);
    R::load(d, static_cast<const T *>(a.in1) + ch.r * a.ld + ch.base, ch.len, c.t, kSplitThreads, 0.0f, true);
    if (a.cstat0) {
        const float off = load_stat(a.cstat0, ch.r, a.stat_bf16) * kLog2e;
#pragma unroll
        for (int e = 0; e < R::E; e++) y[e] = fast_exp2(fmaf(y[e], kLog2e, -off));
    }
    float s = 0.0f;
#pragma unroll
    for (int e = 0; e < R::E; e++) s = fmaf(y[e], d[e], s);
    s = row_allreduce1(s, c, SumOp());
    if (threadIdx.x == 0) reinterpret_cast<float4 *>(a.part0)[blockIdx.x] = make_float4(s, 0.0f, 0.0f, 0.0f);
}

template <typename T, bool VEC, int VPT>
__global__ void __launch_bounds__(kSplitThreads) softmax_bwd_split_write(RowArgs a) {
    using R = Row<T, VEC, VPT>;
    __shared__ float red[2 * 32 * kRedWidth];
    RowCtx c = make_row_ctx(kSplitThreads, red);
    Chunk<T, VEC, VPT> ch(a);
    const float4 *states = reinterpret_cast<const float4 *>(a.part0) + ch.r * a.splits;
    float s = 0.0f;
    for (int i = threadIdx.x; i < a.splits; i += blockDim.x) s += states[i].x;
    s = row_allreduce1(s, c, SumOp());
    float y[R::E], d[R::E];
    R::load(y, static_cast<const T *>(a.in0) + ch.r * a.ld + ch.base, ch.len, c.t, kSplitThreads,
            a.cstat0 ? -INFINITY : 0.0f, true);
    R::load(d, static_cast<const T *>(a.in1) + ch.r * a.ld + ch.base, ch.len, c.t, kSplitThreads, 0.0f, true);
    if (a.cstat0) {
        const float off = load_stat(a.cstat0, ch.r, a.stat_bf16) * kLog2e;
#pragma unroll
        for (int e = 0; e < R::E; e++) y[e] = fast_exp2(fmaf(y[e], kLog2e, -off));
    }
#pragma unroll
    for (int e = 0; e < R::E; e++) d[e] = y[e] * (d[e] - s);
    R::store(d, static_cast<T *>(a.out0) + ch.r * a.ld + ch.base, ch.len, c.t, kSplitThreads, true);
}

// LayerNorm: chunk states (count, mean, M2) merged as Chan combines them
// (src/Compiler/IR/folds.jl:166-182).
template <typename T, bool VEC, int VPT>
__global__ void __launch_bounds__(kSplitThreads) layernorm_split_fold(RowArgs a) {
    using R = Row<T, VEC, VPT>;
    __shared__ float red[2 * 32 * kRedWidth];
    RowCtx c = make_row_ctx(kSplitThreads, red);
    Chunk<T, VEC, VPT> ch(a);
    float v[R::E];
    R::load(v, static_cast<const T *>(a.in0) + ch.r * a.ld + ch.base, ch.len, c.t, kSplitThreads, 0.0f, true);
    float s = 0.0f;
#pragma unroll
    for (int e = 0; e < R::E; e++) s += v[e];
    const float cnt = static_cast<float>(ch.len);
    const float mean = row_allreduce1(s, c, SumOp()) / cnt;
    float q = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const bool in = R::inside(k, c.t, kSplitThreads, ch.len);
#pragma unroll
        for (int e = 0; e < R::EPV; e++) {
            const float d = v[k * R::EPV + e] - mean;
            q = in ? fmaf(d, d, q) : q;
        }
    }
    q = row_allreduce1(q, c, SumOp());
    if (threadIdx.x == 0) reinterpret_cast<float4 *>(a.part0)[blockIdx.x] = make_float4(cnt, mean, q, 0.0f);
}

__device__ __forceinline__ void merged_moments(const float4 *states, int splits, float fn, float eps, RowCtx &c,
                                               float &mean, float &rstd) {
    float s = 0.0f;
    for (int i = threadIdx.x; i < splits; i += blockDim.x) s = fmaf(states[i].x, states[i].y, s);
    mean = row_allreduce1(s, c, SumOp()) / fn;
    float q = 0.0f;
    for (int i = threadIdx.x; i < splits; i += blockDim.x) {
        const float4 st = states[i];
        const float d = st.y - mean;
        q += st.z + st.x * d * d;
    }
    rstd = 1.0f / sqrtf(row_allreduce1(q, c, SumOp()) / fn + eps);
}

template <typename T, bool VEC, int VPT>
__global__ void __launch_bounds__(kSplitThreads) layernorm_fwd_split_write(RowArgs a) {
    using R = Row<T, VEC, VPT>;
    __shared__ float red[2 * 32 * kRedWidth];
    RowCtx c = make_row_ctx(kSplitThreads, red);
    Chunk<T, VEC, VPT> ch(a);
    float mean, rstd;
    merged_moments(reinterpret_cast<const float4 *>(a.part0) + ch.r * a.splits, a.splits, static_cast<float>(a.n),
                   a.eps, c, mean, rstd);
    if (ch.c == 0 && threadIdx.x == 0) {
        if (a.stat0) static_cast<float *>(a.stat0)[ch.r] = mean;
        if (a.stat1) static_cast<float *>(a.stat1)[ch.r] = rstd;
    }
    float v[R::E], gam[R::E], bet[R::E];
    R::load(v, static_cast<const T *>(a.in0) + ch.r * a.ld + ch.base, ch.len, c.t, kSplitThreads, 0.0f, true);
    R::load_cached(gam, static_cast<const T *>(a.gamma) + ch.base, ch.len, c.t, kSplitThreads, 0.0f);
    if (a.beta) R::load_cached(bet, static_cast<const T *>(a.beta) + ch.base, ch.len, c.t, kSplitThreads, 0.0f);
    else
#pragma unroll
        for (int e = 0; e < R::E; e++) bet[e] = 0.0f;
#pragma unroll
    for (int e = 0; e < R::E; e++) v[e] = fmaf((v[e] - mean) * rstd, gam[e], bet[e]);
    R::store(v, static_cast<T *>(a.out0) + ch.r * a.ld + ch.base, ch.len, c.t, kSplitThreads, true);
}

// ------------------------------------------------------------- dispatch -----

enum RowOp { OP_SOFTMAX_FWD, OP_SOFTMAX_BWD, OP_LN_FWD, OP_LN_BWD };

// elements a thread holds in the resident schedule, by how many row-sized
// register arrays the kernel keeps
inline int resident_elems(RowOp op) { return op == OP_LN_BWD ? 16 : 32; }

struct Schedule {
    bool vec;     // 128-bit accesses
    bool split;   // two-pass schedule
    int vpt;      // vectors per thread
    int tpr, rpc; // resident geometry
    int threads;
    int splits;
    long long blocks; // grid (resident: an upper bound before occupancy)
    bool exact;       // the rows fill every vector slot of every row slot of every block
    bool staged;      // LayerNorm kernels fed through a ring in shared memory (`splits` = its stages)
    int turn, arrays; // staged: rows a row slot takes per turn, row-sized arrays a stage holds per row
};

inline int round_vpt(int64_t v) { return v <= 1 ? 1 : v <= 2 ? 2 : v <= 4 ? 4 : 8; }

Schedule plan_rows(RowOp op, int64_t n, int64_t rows, int64_t ld, int dtype, bool aligned16) {
    Schedule s{};
    const int es = static_cast<int>(dtype_size(dtype));
    const int epv_vec = 16 / es;
    s.vec = aligned16 && n % epv_vec == 0 && ld % epv_vec == 0;
    const int epv = s.vec ? epv_vec : 1;
    const int max_e = resident_elems(op);
    int max_vpt = s.vec ? max_e / epv : 8;
    const int64_t nvec = n / epv;
    // the forward kernels hold one row-sized array: four vectors a thread over twice the threads keep more warps
    // resident than eight (measured on 4096-long Float32 rows); longer rows still take eight
    // (BFloat16 rows keep 32 elements a thread: at 16, over twice the threads, the LayerNorm forward fell from 5018
    // to 3999 GB/s)
    if (s.vec && max_vpt > 4 && (op == OP_SOFTMAX_FWD || op == OP_LN_FWD) && nvec <= 4 * kResidentMaxThreads) max_vpt = 4;
    const int tpr = next_pow2(ceil_div(nvec, max_vpt));
    if (tpr <= kResidentMaxThreads) {
        s.split = false;
        s.tpr = tpr;
        s.vpt = round_vpt(ceil_div(nvec, tpr));
        s.threads = tpr >= 128 ? tpr : 128;
        s.rpc = s.threads / tpr;
        s.splits = 1;
        s.blocks = ceil_div(rows, s.rpc);
        s.exact = s.vec && nvec == static_cast<int64_t>(s.tpr) * s.vpt && rows % s.rpc == 0;
    } else {
        s.split = true;
        s.vpt = s.vec ? 32 / epv : 8;  // split chunks hold 32 elements per thread (8 when scalar)
        s.tpr = kSplitThreads;
        s.rpc = 1;
        s.threads = kSplitThreads;
        const int64_t chunk = static_cast<int64_t>(kSplitThreads) * s.vpt * epv;
        s.splits = static_cast<int>(ceil_div(n, chunk));
        s.blocks = rows * s.splits;
    }
    return s;
}

using RowKernel = void (*)(RowArgs);

// One struct per kernel family, so a family can be named as a type and
// instantiated for the schedule's (element type, access width, vectors per thread).
// ELEMS: the most elements a thread holds in any schedule of the family (`resident_elems`; split chunks hold 32);
// wider instantiations are never launched and are not compiled.
#define TB200_FAMILY(NAME, KERNEL, ELEMS)                                  \
    struct NAME {                                                          \
        static constexpr int kMaxElems = ELEMS;                            \
        template <typename T, bool VEC, int VPT>                           \
        static RowKernel get() { return KERNEL<T, VEC, VPT>; }             \
    }
TB200_FAMILY(SoftmaxFwdResident, softmax_fwd_resident, 32);
TB200_FAMILY(SoftmaxBwdResident, softmax_bwd_resident, 32);
TB200_FAMILY(LayernormFwdResident, layernorm_fwd_resident, 32);
TB200_FAMILY(LayernormBwdResident, layernorm_bwd_resident, 16);
TB200_FAMILY(SoftmaxFwdSplitFold, softmax_fwd_split_fold, 32);
TB200_FAMILY(SoftmaxFwdSplitWrite, softmax_fwd_split_write, 32);
TB200_FAMILY(SoftmaxBwdSplitFold, softmax_bwd_split_fold, 32);
TB200_FAMILY(SoftmaxBwdSplitWrite, softmax_bwd_split_write, 32);
TB200_FAMILY(LayernormSplitFold, layernorm_split_fold, 32);
TB200_FAMILY(LayernormFwdSplitWrite, layernorm_fwd_split_write, 32);
#undef TB200_FAMILY

template <typename Fam, typename T, bool VEC>
RowKernel pick_vpt(int vpt) {
    constexpr int EPV = Access<T, VEC>::EPV;
    switch (vpt) {
        case 1: return Fam::template get<T, VEC, 1>();
        case 2: return Fam::template get<T, VEC, 2>();
        case 4:
            if constexpr (4 * EPV <= Fam::kMaxElems) return Fam::template get<T, VEC, 4>();
            else return nullptr;
        case 8:
            // (8 vectors of 8 BFloat16 would be 64 elements a thread: never scheduled by any family)
            if constexpr (8 * EPV <= Fam::kMaxElems) return Fam::template get<T, VEC, 8>();
            else return nullptr;
        default: return nullptr;
    }
}

template <typename Fam>
RowKernel pick(int dtype, const Schedule &s) {
    if (dtype == TB200_F32) return s.vec ? pick_vpt<Fam, float, true>(s.vpt) : pick_vpt<Fam, float, false>(s.vpt);
    return s.vec ? pick_vpt<Fam, __nv_bfloat16, true>(s.vpt) : pick_vpt<Fam, __nv_bfloat16, false>(s.vpt);
}

// Resident blocks per SM of a kernel at a block size, asked of the runtime once
// per (kernel, block size, device).
int blocks_per_sm(RowKernel kernel, int threads, int device, int *out) {
    static std::mutex lock;
    static std::map<std::tuple<const void *, int, int>, int> memo;
    const auto key = std::make_tuple(reinterpret_cast<const void *>(kernel), threads, device);
    {
        std::lock_guard<std::mutex> hold(lock);
        auto it = memo.find(key);
        if (it != memo.end()) {
            *out = it->second;
            return TB200_OK;
        }
    }
    int per_sm = 0;
    TB200_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0));
    if (per_sm < 1) per_sm = 1;
    std::lock_guard<std::mutex> hold(lock);
    memo[key] = per_sm;
    *out = per_sm;
    return TB200_OK;
}

// Persistent grid of a resident kernel: every SM full, never more blocks than row groups.
int resident_grid(RowKernel kernel, const Schedule &s, const DeviceInfo &dev, long long *grid) {
    if (!kernel) return TB200_ERR_UNSUPPORTED;
    int per_sm = 0;
    int st = blocks_per_sm(kernel, s.threads, dev.device, &per_sm);
    if (st) return st;
    long long g = static_cast<long long>(dev.sms) * per_sm;
    *grid = g < s.blocks ? g : s.blocks;
    return TB200_OK;
}

int launch_resident(RowKernel kernel, const Schedule &s, const DeviceInfo &dev, const RowArgs &a,
                    cudaStream_t stream) {
    long long grid = 0;
    int st = resident_grid(kernel, s, dev, &grid);
    if (st) return st;
    kernel<<<static_cast<unsigned>(grid), s.threads, 0, stream>>>(a);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

int launch_split(RowKernel kernel, const Schedule &s, const RowArgs &a, cudaStream_t stream) {
    if (!kernel) return TB200_ERR_UNSUPPORTED;
    kernel<<<static_cast<unsigned>(s.blocks), s.threads, 0, stream>>>(a);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

int check_rows(int64_t n, int64_t rows, int64_t ld, int dtype) {
    if (dtype != TB200_F32 && dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (n < 0 || rows < 0 || ld < n) return TB200_ERR_SHAPE;
    if (n > (int64_t(1) << 30) || rows > (int64_t(1) << 40)) return TB200_ERR_SHAPE;
    return TB200_OK;
}

bool all_aligned(size_t a, std::initializer_list<const void *> ps) {
    for (const void *p : ps)
        if (p && !aligned_to(p, a)) return false;
    return true;
}

int fill(void *p, int64_t count, float value, int as_bf16, cudaStream_t stream) {
    if (!p || count == 0) return TB200_OK;
    fill_stat<<<static_cast<unsigned>(ceil_div(count, 256)), 256, 0, stream>>>(p, count, value, as_bf16);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

size_t split_state_bytes(const Schedule &s, int64_t rows) {
    return static_cast<size_t>(rows) * s.splits * sizeof(float4);
}

}  // namespace
}  // namespace tb200

using namespace tb200;

namespace {

// The LayerNorm backward's kernel for a schedule: the compact BFloat16 form where it applies (128-bit accesses,
// every slot filled, 256-thread blocks, statistics saved by the forward), else the general family.
RowKernel ln_bwd_kernel(int dtype, const Schedule &s, bool saved_stats) {
    if (s.staged) return dtype == TB200_F32 ? layernorm_bwd_staged<float, 1> : layernorm_bwd_staged<__nv_bfloat16, kStagedRowsBf16>;
    if (dtype == TB200_BF16 && s.vec && s.exact && saved_stats && s.threads == 256) {
        if (s.vpt == 1) return layernorm_bwd_compact<1>;
        if (s.vpt == 2) return layernorm_bwd_compact<2>;
    }

    return pick<LayernormBwdResident>(dtype, s);
}

// The schedule the LayerNorm backward runs: rows of 1024, 2048 or 4096 elements that allow 128-bit accesses, with
// the statistics saved and whole groups of rows, take the form fed through shared memory (eight elements a thread,
// 512 threads, `splits` = stages of the ring); everything else keeps the plan.
constexpr size_t kStagedRingBytes = 96 * 1024;
constexpr int kStagedRowsFwd = 4;    // rows a block of the forward takes per turn
// `arrays`: row-sized arrays a stage holds per row (x; x and dy); `turn`: rows per turn per row slot.
Schedule staged_schedule(const Schedule &s, int64_t n, int64_t rows, int dtype, int arrays, int turn) {
    if (!s.vec || s.split || (n != 1024 && n != 2048 && n != 4096)) return s;
    Schedule w = s;
    w.staged = true;
    w.threads = kStagedThreads;
    w.tpr = static_cast<int>(n / 8);
    w.rpc = kStagedThreads / w.tpr;
    w.turn = turn;
    w.arrays = arrays;
    if (rows % (turn * w.rpc) != 0) return s;
    w.vpt = dtype == TB200_F32 ? 2 : 1;
    w.exact = true;
    w.blocks = rows / (turn * w.rpc);
    const size_t stage = static_cast<size_t>(arrays) * turn * w.rpc * n * dtype_size(dtype);
    w.splits = static_cast<int>(kStagedRingBytes / stage);
    if (w.splits > 8) w.splits = 8;
    return w;
}
Schedule ln_bwd_schedule(const Schedule &s, int64_t n, int64_t rows, int dtype, bool saved_stats) {
    if (!saved_stats) return s;
    return staged_schedule(s, n, rows, dtype, 2, dtype == TB200_F32 ? 1 : kStagedRowsBf16);
}
size_t staged_smem_bytes(const Schedule &s, int64_t n, int dtype) {
    return 128 + static_cast<size_t>(s.splits) * s.arrays * s.turn * s.rpc * n * dtype_size(dtype);
}
// Grid of a staged kernel: as many blocks per SM as its ring allows (asked of the runtime once per kernel and
// device), never more than there are turns.
int staged_grid(RowKernel kernel, const Schedule &s, const DeviceInfo &dev, int64_t n, int dtype, long long *grid) {
    static std::mutex lock;
    static std::map<std::tuple<const void *, int, size_t>, int> memo;
    const size_t smem = staged_smem_bytes(s, n, dtype);
    const auto key = std::make_tuple(reinterpret_cast<const void *>(kernel), dev.device, smem);
    int per_sm = 0;
    {
        std::lock_guard<std::mutex> hold(lock);
        auto it = memo.find(key);
        if (it != memo.end()) per_sm = it->second;
    }
    if (!per_sm) {
        TB200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(128 + kStagedRingBytes)));
        TB200_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kStagedThreads, smem));
        if (per_sm < 1) return TB200_ERR_UNSUPPORTED;
        std::lock_guard<std::mutex> hold(lock);
        memo[key] = per_sm;
    }
    const long long g = static_cast<long long>(per_sm) * dev.sms;
    *grid = g < s.blocks ? g : s.blocks;
    return TB200_OK;
}
int ln_bwd_grid(RowKernel kernel, const Schedule &s, const DeviceInfo &dev, int64_t n, int dtype, long long *grid) {
    return s.staged ? staged_grid(kernel, s, dev, n, dtype, grid) : resident_grid(kernel, s, dev, grid);
}

// Scratch layout of the streamed LayerNorm backward: mean and rstd of every row (used when the forward saved
// none), then the column sums' partial rows.
int ln_long_slabs(int64_t n, int64_t rows, int sms) {
    const int64_t col_blocks = ceil_div(n, 256);
    int64_t slabs = ceil_div(static_cast<int64_t>(sms) * 8, col_blocks);
    if (slabs > kLongSlabsMax) slabs = kLongSlabsMax;
    if (slabs > rows) slabs = rows;
    return static_cast<int>(slabs < 1 ? 1 : slabs);
}
size_t ln_long_stat_bytes(int64_t rows) { return (static_cast<size_t>(rows) * 2 * sizeof(float) + 15) / 16 * 16; }
size_t ln_long_bytes(int64_t n, int64_t rows) {
    return ln_long_stat_bytes(rows) + static_cast<size_t>(kLongSlabsMax) * n * 2 * sizeof(float);
}

// Bytes of scratch one schedule of an operator needs.
int schedule_workspace(RowOp op, const Schedule &s, const DeviceInfo &dev, int64_t n, int64_t rows, int dtype,
                       size_t *bytes) {
    *bytes = 0;
    if (s.split) {
        *bytes = op == OP_LN_BWD ? ln_long_bytes(n, rows) : split_state_bytes(s, rows);
        return TB200_OK;
    }
    if (op == OP_LN_BWD) {
        // either form may run (the call decides by its arguments): room for the larger grid
        long long grid = 0, compact = 0;
        int st = resident_grid(ln_bwd_kernel(dtype, s, false), s, dev, &grid);
        if (st) return st;
        const Schedule saved = ln_bwd_schedule(s, n, rows, dtype, true);
        if ((st = ln_bwd_grid(ln_bwd_kernel(dtype, saved, true), saved, dev, n, dtype, &compact))) return st;
        long long parts = grid * s.rpc;
        if (compact * saved.rpc > parts) parts = compact * saved.rpc;
        *bytes = static_cast<size_t>(parts) * static_cast<size_t>(n) * 2 * sizeof(float);
    }
    return TB200_OK;
}

bool workspace_ok(const void *workspace, size_t have, size_t need) {
    return need == 0 || (workspace && have >= need && aligned_to(workspace, 16));
}

}  // namespace

extern "C" size_t tb200_rowop_workspace_bytes(int op, int64_t n, int64_t rows, int dtype) {
    if (op < OP_SOFTMAX_FWD || op > OP_LN_BWD) return 0;
    if (check_rows(n, rows, n, dtype) != TB200_OK || n == 0 || rows == 0) return 0;
    DeviceInfo dev;
    if (current_device(&dev) != TB200_OK) return 0;
    // the call picks 128-bit or scalar accesses from its pointers and ld: cover both
    size_t most = 0;
    for (int vec = 0; vec < 2; vec++) {
        const Schedule s = plan_rows(static_cast<RowOp>(op), n, rows, vec ? n : n + 1, dtype, vec != 0);
        size_t bytes = 0;
        if (schedule_workspace(static_cast<RowOp>(op), s, dev, n, rows, dtype, &bytes) != TB200_OK) return 0;
        if (bytes > most) most = bytes;
    }
    return most;
}

extern "C" int tb200_softmax_fwd(const void *x, void *y, void *lse, int64_t n, int64_t rows, int64_t ld, int dtype,
                                 int stat_dtype, void *workspace, size_t workspace_bytes, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int st = check_rows(n, rows, ld, dtype);
    if (st) return st;
    if (stat_dtype != TB200_F32 && stat_dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (rows == 0) return TB200_OK;
    if (n == 0) return fill(lse, rows, -INFINITY, stat_dtype == TB200_BF16, stream);
    if (!x || !y) return TB200_ERR_NULL;
    if (!all_aligned(dtype_size(dtype), {x, y}) || !all_aligned(dtype_size(stat_dtype), {lse})) return TB200_ERR_ALIGN;
    DeviceInfo dev;
    if ((st = current_device(&dev))) return st;
    const Schedule s = plan_rows(OP_SOFTMAX_FWD, n, rows, ld, dtype, all_aligned(16, {x, y}));
    RowArgs a{};
    a.in0 = x; a.out0 = y; a.stat0 = lse; a.n = static_cast<int>(n); a.rows = rows; a.ld = ld;
    a.tpr = s.tpr; a.rpc = s.rpc; a.splits = s.splits; a.stat_bf16 = stat_dtype == TB200_BF16; a.exact = s.exact;
    if (!s.split) return launch_resident(pick<SoftmaxFwdResident>(dtype, s), s, dev, a, stream);
    if (!workspace_ok(workspace, workspace_bytes, split_state_bytes(s, rows))) return TB200_ERR_WORKSPACE;
    a.part0 = static_cast<float *>(workspace);
    if ((st = launch_split(pick<SoftmaxFwdSplitFold>(dtype, s), s, a, stream))) return st;
    return launch_split(pick<SoftmaxFwdSplitWrite>(dtype, s), s, a, stream);
}

extern "C" int tb200_softmax_bwd(const void *y_or_x, const void *lse, const void *dy, void *dx, int64_t n,
                                 int64_t rows, int64_t ld, int dtype, int stat_dtype, void *workspace,
                                 size_t workspace_bytes, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int st = check_rows(n, rows, ld, dtype);
    if (st) return st;
    if (stat_dtype != TB200_F32 && stat_dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (rows == 0 || n == 0) return TB200_OK;
    if (!y_or_x || !dy || !dx) return TB200_ERR_NULL;
    if (!all_aligned(dtype_size(dtype), {y_or_x, dy, dx}) || !all_aligned(dtype_size(stat_dtype), {lse}))
        return TB200_ERR_ALIGN;
    DeviceInfo dev;
    if ((st = current_device(&dev))) return st;
    const Schedule s = plan_rows(OP_SOFTMAX_BWD, n, rows, ld, dtype, all_aligned(16, {y_or_x, dy, dx}));
    RowArgs a{};
    a.in0 = y_or_x; a.in1 = dy; a.out0 = dx; a.cstat0 = lse; a.n = static_cast<int>(n); a.rows = rows; a.ld = ld;
    a.tpr = s.tpr; a.rpc = s.rpc; a.splits = s.splits; a.stat_bf16 = stat_dtype == TB200_BF16; a.exact = s.exact;
    if (!s.split) return launch_resident(pick<SoftmaxBwdResident>(dtype, s), s, dev, a, stream);
    if (!workspace_ok(workspace, workspace_bytes, split_state_bytes(s, rows))) return TB200_ERR_WORKSPACE;
    a.part0 = static_cast<float *>(workspace);
    if ((st = launch_split(pick<SoftmaxBwdSplitFold>(dtype, s), s, a, stream))) return st;
    return launch_split(pick<SoftmaxBwdSplitWrite>(dtype, s), s, a, stream);
}

extern "C" int tb200_layernorm_fwd(const void *x, const void *gamma, const void *beta, void *y, float *mean,
                                   float *rstd, float eps, int64_t n, int64_t rows, int64_t ld, int dtype,
                                   void *workspace, size_t workspace_bytes, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int st = check_rows(n, rows, ld, dtype);
    if (st) return st;
    if (rows == 0 || n == 0) return TB200_OK;
    if (!x || !y || !gamma) return TB200_ERR_NULL;
    if (!all_aligned(dtype_size(dtype), {x, y, gamma, beta}) || !all_aligned(4, {mean, rstd})) return TB200_ERR_ALIGN;
    DeviceInfo dev;
    if ((st = current_device(&dev))) return st;
    const Schedule s = plan_rows(OP_LN_FWD, n, rows, ld, dtype, all_aligned(16, {x, y, gamma, beta}));
    RowArgs a{};
    a.in0 = x; a.gamma = gamma; a.beta = beta; a.out0 = y; a.stat0 = mean; a.stat1 = rstd; a.eps = eps;
    a.n = static_cast<int>(n); a.rows = rows; a.ld = ld; a.tpr = s.tpr; a.rpc = s.rpc; a.splits = s.splits;
    a.exact = s.exact;
    // BFloat16 rows of 1024, 2048 or 4096 elements: the form fed through shared memory (for Float32 rows the resident
    // kernel is the faster one, 0.356 against 0.379 ms on 4096 x 65536)
    const Schedule staged = dtype == TB200_BF16 ? staged_schedule(s, n, rows, dtype, 1, kStagedRowsFwd) : s;
    if (staged.staged) {
        const RowKernel kernel = layernorm_fwd_staged<__nv_bfloat16, kStagedRowsFwd>;
        long long grid = 0;
        if ((st = staged_grid(kernel, staged, dev, n, dtype, &grid))) return st;
        a.tpr = staged.tpr; a.rpc = staged.rpc; a.splits = staged.splits; a.exact = 1;
        kernel<<<static_cast<unsigned>(grid), staged.threads, staged_smem_bytes(staged, n, dtype), stream>>>(a);
        TB200_CUDA(cudaGetLastError());
        return TB200_OK;
    }
    if (!s.split) return launch_resident(pick<LayernormFwdResident>(dtype, s), s, dev, a, stream);
    if (!workspace_ok(workspace, workspace_bytes, split_state_bytes(s, rows))) return TB200_ERR_WORKSPACE;
    a.part0 = static_cast<float *>(workspace);
    if ((st = launch_split(pick<LayernormSplitFold>(dtype, s), s, a, stream))) return st;
    return launch_split(pick<LayernormFwdSplitWrite>(dtype, s), s, a, stream);
}

extern "C" int tb200_layernorm_bwd(const void *x, const void *gamma, const void *dy, const float *mean,
                                   const float *rstd, void *dx, void *dgamma, void *dbeta, float eps, int64_t n,
                                   int64_t rows, int64_t ld, int dtype, void *workspace, size_t workspace_bytes,
                                   void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int st = check_rows(n, rows, ld, dtype);
    if (st) return st;
    if (n == 0) return TB200_OK;
    if (rows == 0) {  // sums over no rows are zero
        if (dgamma) TB200_CUDA(cudaMemsetAsync(dgamma, 0, n * dtype_size(dtype), stream));
        if (dbeta) TB200_CUDA(cudaMemsetAsync(dbeta, 0, n * dtype_size(dtype), stream));
        return TB200_OK;
    }
    if (!x || !gamma || !dy || !dx) return TB200_ERR_NULL;
    if (!all_aligned(dtype_size(dtype), {x, gamma, dy, dx, dgamma, dbeta}) || !all_aligned(4, {mean, rstd}))
        return TB200_ERR_ALIGN;
    DeviceInfo dev;
    if ((st = current_device(&dev))) return st;
    const Schedule s = ln_bwd_schedule(plan_rows(OP_LN_BWD, n, rows, ld, dtype, all_aligned(16, {x, gamma, dy, dx})), n,
                                       rows, dtype, mean && rstd);
    RowArgs a{};
    a.in0 = x; a.in1 = dy; a.gamma = gamma; a.out0 = dx; a.cstat0 = mean; a.cstat1 = rstd; a.eps = eps;
    a.n = static_cast<int>(n); a.rows = rows; a.ld = ld; a.tpr = s.tpr; a.rpc = s.rpc; a.splits = 1;
    a.exact = s.exact;
    if (s.split) {   // rows beyond the resident schedule: streamed, column sums by a kernel of their own
        const bool sums = dgamma || dbeta;
        const bool saved = mean && rstd;
        if ((sums || !saved) && !workspace_ok(workspace, workspace_bytes, ln_long_bytes(n, rows)))
            return TB200_ERR_WORKSPACE;
        float *own_stats = static_cast<float *>(workspace);
        if (!saved) {
            a.cstat0 = a.cstat1 = nullptr;
            if (sums) { a.stat0 = own_stats; a.stat1 = own_stats + rows; }
        }
        const unsigned grid = static_cast<unsigned>(rows < 4LL * dev.sms ? rows : 4LL * dev.sms);
        if (dtype == TB200_F32) {
            if (s.vec) layernorm_bwd_long<float, true><<<grid, kResidentMaxThreads, 0, stream>>>(a);
            else layernorm_bwd_long<float, false><<<grid, kResidentMaxThreads, 0, stream>>>(a);
        } else {
            if (s.vec) layernorm_bwd_long<__nv_bfloat16, true><<<grid, kResidentMaxThreads, 0, stream>>>(a);
            else layernorm_bwd_long<__nv_bfloat16, false><<<grid, kResidentMaxThreads, 0, stream>>>(a);
        }
        TB200_CUDA(cudaGetLastError());
        if (!sums) return TB200_OK;
        const float *mean_at = saved ? mean : own_stats, *rstd_at = saved ? rstd : own_stats + rows;
        float *part0 = reinterpret_cast<float *>(static_cast<char *>(workspace) + ln_long_stat_bytes(rows));
        const int slabs = ln_long_slabs(n, rows, dev.sms);
        float *part1 = part0 + static_cast<size_t>(slabs) * n;
        const dim3 cgrid(static_cast<unsigned>(ceil_div(n, 256)), static_cast<unsigned>(slabs));
        const unsigned mblocks = static_cast<unsigned>(ceil_div(n, 32));
        if (dtype == TB200_F32) {
            layernorm_bwd_colsums<float><<<cgrid, 256, 0, stream>>>(static_cast<const float *>(x), static_cast<const float *>(dy),
                                                                   mean_at, rstd_at, part0, part1, a.n, rows, ld, slabs);
            merge_parts<float><<<mblocks, 256, 0, stream>>>(part0, part1, static_cast<float *>(dgamma),
                                                            static_cast<float *>(dbeta), a.n, slabs);
        } else {
            layernorm_bwd_colsums<__nv_bfloat16><<<cgrid, 256, 0, stream>>>(
                static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(dy), mean_at, rstd_at, part0, part1,
                a.n, rows, ld, slabs);
            merge_parts<__nv_bfloat16><<<mblocks, 256, 0, stream>>>(part0, part1, static_cast<__nv_bfloat16 *>(dgamma),
                                                                    static_cast<__nv_bfloat16 *>(dbeta), a.n, slabs);
        }
        TB200_CUDA(cudaGetLastError());
        return TB200_OK;
    }
    const RowKernel kernel = ln_bwd_kernel(dtype, s, mean && rstd);
    long long grid = 0;
    if ((st = ln_bwd_grid(kernel, s, dev, n, dtype, &grid))) return st;
    if (s.staged) a.splits = s.splits;
    const bool sums = dgamma || dbeta;
    const size_t part_len = static_cast<size_t>(grid) * s.rpc * static_cast<size_t>(n);
    if (sums) {
        if (!workspace_ok(workspace, workspace_bytes, part_len * 2 * sizeof(float))) return TB200_ERR_WORKSPACE;
        a.part0 = static_cast<float *>(workspace);
        a.part1 = a.part0 + part_len;
    }
    kernel<<<static_cast<unsigned>(grid), s.threads, s.staged ? staged_smem_bytes(s, n, dtype) : 0, stream>>>(a);
    TB200_CUDA(cudaGetLastError());
    if (sums) {
        const int parts = static_cast<int>(grid * s.rpc);
        if (n % 4 == 0) {
            const unsigned blocks = static_cast<unsigned>(ceil_div(n, 64));
            if (dtype == TB200_F32)
                merge_parts_wide<float><<<blocks, 256, 0, stream>>>(a.part0, a.part1, static_cast<float *>(dgamma),
                                                                    static_cast<float *>(dbeta), a.n, parts);
            else
                merge_parts_wide<__nv_bfloat16><<<blocks, 256, 0, stream>>>(a.part0, a.part1, static_cast<__nv_bfloat16 *>(dgamma),
                                                                            static_cast<__nv_bfloat16 *>(dbeta), a.n, parts);
        } else {
            const unsigned blocks = static_cast<unsigned>(ceil_div(n, 32));
            if (dtype == TB200_F32)
                merge_parts<float><<<blocks, 256, 0, stream>>>(a.part0, a.part1, static_cast<float *>(dgamma),
                                                               static_cast<float *>(dbeta), a.n, parts);
            else
                merge_parts<__nv_bfloat16><<<blocks, 256, 0, stream>>>(a.part0, a.part1, static_cast<__nv_bfloat16 *>(dgamma),
                                                                       static_cast<__nv_bfloat16 *>(dbeta), a.n, parts);
        }
        TB200_CUDA(cudaGetLastError());
    }
    return TB200_OK;
}

// ------------------------------------------------- LayerNorm backward, no allocation ----
//
// tb200_layernorm_bwd_noalloc is tb200_layernorm_bwd for callers that have no way to hand
// over scratch memory: a host program that fixed all of its device buffers before it knew
// which kernels it would run and has no allocator to ask afterwards (a plugin called from a
// runtime that owns every byte of device memory, an embedded or real-time loop that must
// not reach the driver's allocator, which takes a process-wide lock and may synchronise the
// device).  The dgamma / dbeta partial sums then live in the fixed array below, which is
// part of the library's image: every GPU that loads the library holds these 8 MiB until the
// process exits.
//
// The array's name is a host-side handle in host code, not an address a kernel can use; the
// device address comes from cudaGetSymbolAddress, asked once per device (with that device
// current) by the first call on it, which is why that first call should be made outside any
// stream capture.  All calls on a device share the array and nothing is kept between calls:
// each launch overwrites the partial rows it later merges, so nothing needs clearing, but two
// calls whose kernels overlap on the GPU (different streams) would overwrite each other's
// partial sums.  Calls must be ordered by the caller.
namespace {

constexpr size_t kNoAllocScratchBytes = size_t(8) << 20;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchBytes / sizeof(float)];

// Device address of the scratch on the current device, looked up on first use.
int noalloc_scratch(const tb200::DeviceInfo &dev, float **out) {
    static std::mutex lock;
    static float *known[64] = {};
    std::lock_guard<std::mutex> hold(lock);
    if (!known[dev.device]) {
        float *ptr = nullptr;
        TB200_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_noalloc_scratch));
        if (!ptr) return TB200_ERR_CUDA;
        known[dev.device] = ptr;
    }
    *out = known[dev.device];
    return TB200_OK;
}

}  // namespace

extern "C" size_t tb200_layernorm_bwd_noalloc_max_row(void) {
    // the longest row the resident schedule of the LayerNorm backward takes; one block's
    // partial sums for it (2 x 8192 Float32) fit the scratch 128 times over
    return 8192;
}

extern "C" int tb200_layernorm_bwd_noalloc(const void *x, const void *gamma, const void *dy, const float *mean,
                                           const float *rstd, void *dx, void *dgamma, void *dbeta, float eps,
                                           int64_t n, int64_t rows, int64_t ld, int dtype, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int st = check_rows(n, rows, ld, dtype);
    if (st) return st;
    if (n == 0) return TB200_OK;
    // beyond the built-in scratch: say so instead of running with too little
    if (static_cast<size_t>(n) > tb200_layernorm_bwd_noalloc_max_row()) return TB200_ERR_WORKSPACE;
    if (rows == 0) {
        if (dgamma) TB200_CUDA(cudaMemsetAsync(dgamma, 0, n * dtype_size(dtype), stream));
        if (dbeta) TB200_CUDA(cudaMemsetAsync(dbeta, 0, n * dtype_size(dtype), stream));
        return TB200_OK;
    }
    if (!x || !gamma || !dy || !dx) return TB200_ERR_NULL;
    if (!all_aligned(dtype_size(dtype), {x, gamma, dy, dx, dgamma, dbeta}) || !all_aligned(4, {mean, rstd}))
        return TB200_ERR_ALIGN;
    DeviceInfo dev;
    if ((st = current_device(&dev))) return st;
    const Schedule s = plan_rows(OP_LN_BWD, n, rows, ld, dtype, all_aligned(16, {x, gamma, dy, dx}));
    if (s.split) return TB200_ERR_WORKSPACE;
    const RowKernel kernel = pick<LayernormBwdResident>(dtype, s);
    long long grid = 0;
    if ((st = resident_grid(kernel, s, dev, &grid))) return st;
    // as many blocks as the scratch has partial rows for
    const long long room = static_cast<long long>(kNoAllocScratchBytes / (2 * sizeof(float) * static_cast<size_t>(n))) /
                           s.rpc;
    if (room < 1) return TB200_ERR_WORKSPACE;
    if (grid > room) grid = room;
    float *scratch = nullptr;
    if ((st = noalloc_scratch(dev, &scratch))) return st;
    RowArgs a{};
    a.in0 = x; a.in1 = dy; a.gamma = gamma; a.out0 = dx; a.cstat0 = mean; a.cstat1 = rstd; a.eps = eps;
    a.n = static_cast<int>(n); a.rows = rows; a.ld = ld; a.tpr = s.tpr; a.rpc = s.rpc; a.splits = 1;
    a.exact = s.exact;
    const bool sums = dgamma || dbeta;
    const size_t part_len = static_cast<size_t>(grid) * s.rpc * static_cast<size_t>(n);
    if (sums) {
        a.part0 = scratch;
        a.part1 = scratch + part_len;
    }
    kernel<<<static_cast<unsigned>(grid), s.threads, 0, stream>>>(a);
    TB200_CUDA(cudaGetLastError());
    if (sums) {
        const int parts = static_cast<int>(grid * s.rpc);
        const unsigned blocks = static_cast<unsigned>(ceil_div(n, 32));
        if (dtype == TB200_F32)
            merge_parts<float><<<blocks, 256, 0, stream>>>(a.part0, a.part1, static_cast<float *>(dgamma),
                                                           static_cast<float *>(dbeta), a.n, parts);
        else
            merge_parts<__nv_bfloat16><<<blocks, 256, 0, stream>>>(a.part0, a.part1,
                                                                   static_cast<__nv_bfloat16 *>(dgamma),
                                                                   static_cast<__nv_bfloat16 *>(dbeta), a.n, parts);
        TB200_CUDA(cudaGetLastError());
    }
    return TB200_OK;
}

// As tb200_device_error, for the row kernels that wait on copies into shared memory: 0, or 1 when a wait gave up.
extern "C" int tb200_rows_device_error(void) {
    int code = 0, zero = 0;
    TB200_CUDA(cudaDeviceSynchronize());
    TB200_CUDA(cudaMemcpyFromSymbol(&code, tb200::g_rows_error, sizeof(int)));
    if (code) TB200_CUDA(cudaMemcpyToSymbol(tb200::g_rows_error, &zero, sizeof(int)));
    return code;
}
