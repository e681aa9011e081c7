// Chunked gated DeltaNet forward (delta-rule linear attention) for sm_100a.
//
// The rule  S_t = exp(a_t) (S_{t-1} - beta_t k_t (k_t' S_{t-1})) + beta_t k_t v_t',  o_t = S_t' q_t  in the
// chunked WY form of examples/deltanet.jl:58-85 (chunks of C = 64 positions):
//   within a chunk   ca = cumsum(a);  A = beta .* decay(t > s) .* (K K');  (I + A) [W | Ut] = [beta e^ca K | beta V];
//                    P = decay(t >= s) .* (Q K')
//   across chunks    U = Ut - W S;   o = (e^ca Q) S + P U;   S <- e^{ca_C} S + (e^{ca_C - ca} K)' U
// Arrays: q, k (dk, T, heads) = memory [head][t][dk]; v (dv, T, heads); a, beta (T, heads) Float32;
// the result (T, dv, heads) = memory [head][dv][t] (examples/deltanet.jl:56-57, 85).
//
// Two launches.  `deltanet_chunk_kernel` does everything inside a chunk, one block per (head, chunk):
// the two 64 x 64 x 128 products on CUDA cores in Float32 and, instead of forming (I + A)^-1 by blocks as
// the reference's `blocks` does (examples/deltanet.jl:39-54), a forward substitution on the 256 right-hand
// columns at once, one column per thread with the solution held in registers -- the same numbers, no
// inverse.  `deltanet_scan_kernel` carries the state, one block per (head, 32 value features): the state
// slice (128 x 32 Float32) lives in shared memory for all 128 chunks and each chunk costs three small
// products.  The path is bound by the chain of chunks and by HBM, not by the tensor cores (about 0.1 TFLOP
// in all), which is why this first version keeps to Float32 CUDA-core arithmetic; W, Ut and P are rounded
// to BFloat16 when they cross from one launch to the other.
#include <mutex>

#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kC = 64;        // chunk length
constexpr int kDK = 128;
constexpr int kDV = 128;
constexpr int kDVP = 32;      // value features per scan block
constexpr int kPadF = 132;    // Float32 row pitch of a 128-wide tile in shared memory
constexpr int kPadH = 136;    // BFloat16 row pitch of a 128-wide tile
constexpr int kPadP = 72;     // BFloat16 row pitch of a 64-wide tile

__device__ __forceinline__ float bf16_bits_to_float(unsigned short h) { return __uint_as_float(static_cast<uint32_t>(h) << 16); }

// ---------------------------------------------------------------- within a chunk ----

__global__ void __launch_bounds__(256) deltanet_chunk_kernel(const __nv_bfloat16 *q, const __nv_bfloat16 *k,
                                                             const __nv_bfloat16 *v, const float *a, const float *beta,
                                                             __nv_bfloat16 *w_out, __nv_bfloat16 *u_out,
                                                             __nv_bfloat16 *p_out, int T) {
    extern __shared__ float sm[];
    float *Kf = sm;                       // [64][132]
    float *Qf = Kf + kC * kPadF;          // [64][132]
    float *A = Qf + kC * kPadF;           // [64][64]
    float *ca = A + kC * kC;              // [64]
    float *be = ca + kC;                  // [64]
    const int chunks = T / kC;
    const int head = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const long long row0 = static_cast<long long>(head) * T + static_cast<long long>(chunk) * kC;
    const int tid = threadIdx.x;

    for (int i = tid; i < kC * kDK / 8; i += 256) {
        const int r = i / (kDK / 8), c = (i % (kDK / 8)) * 8;
        float kv[8], qv[8];
        Access<__nv_bfloat16, true>::load_cached(k + (row0 + r) * kDK + c, kv);
        Access<__nv_bfloat16, true>::load_cached(q + (row0 + r) * kDK + c, qv);
#pragma unroll
        for (int e = 0; e < 8; e++) { Kf[r * kPadF + c + e] = kv[e]; Qf[r * kPadF + c + e] = qv[e]; }
    }
    if (tid < kC) be[tid] = beta[row0 + tid];
    if (tid == 0) {
        float s = 0.0f;
        for (int t = 0; t < kC; t++) { s += a[row0 + t]; ca[t] = s; }
    }
    __syncthreads();

    // A = beta .* decay(t > s) .* (K K'), P = decay(t >= s) .* (Q K'): 4 x 4 outputs per thread
    {
        const int ty = tid >> 4, tx = tid & 15;
        float kk[4][4] = {}, qk[4][4] = {};
        if (tx <= ty) {   // blocks above the diagonal are zero
            for (int d = 0; d < kDK; d += 4) {
                float4 kt[4], qt[4], ks[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    kt[i] = *reinterpret_cast<const float4 *>(Kf + (ty * 4 + i) * kPadF + d);
                    qt[i] = *reinterpret_cast<const float4 *>(Qf + (ty * 4 + i) * kPadF + d);
                    ks[i] = *reinterpret_cast<const float4 *>(Kf + (tx * 4 + i) * kPadF + d);
                }
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        kk[i][j] += kt[i].x * ks[j].x + kt[i].y * ks[j].y + kt[i].z * ks[j].z + kt[i].w * ks[j].w;
                        qk[i][j] += qt[i].x * ks[j].x + qt[i].y * ks[j].y + qt[i].z * ks[j].z + qt[i].w * ks[j].w;
                    }
            }
        }
        __nv_bfloat16 *pc = p_out + (static_cast<long long>(head) * chunks + chunk) * kC * kC;
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int t = ty * 4 + i, s = tx * 4 + j;
                const float dec = t >= s ? __expf(ca[t] - ca[s]) : 0.0f;
                A[t * kC + s] = t > s ? be[t] * dec * kk[i][j] : 0.0f;
                pc[t * kC + s] = __float2bfloat16_rn(t >= s ? dec * qk[i][j] : 0.0f);
            }
    }
    __syncthreads();

    // (I + A) x = rhs by forward substitution, one right-hand column per thread, x in registers
    {
        const int c = tid;   // 0..127: W, 128..255: Ut
        float x[kC];
#pragma unroll
        for (int t = 0; t < kC; t++) {
            float rhs;
            if (c < kDK) rhs = be[t] * __expf(ca[t]) * Kf[t * kPadF + c];
            else rhs = be[t] * bf16_bits_to_float(__ldg(reinterpret_cast<const unsigned short *>(v) + (row0 + t) * kDV + (c - kDK)));
            float acc = rhs;
#pragma unroll
            for (int s = 0; s < t; s++) acc = fmaf(-A[t * kC + s], x[s], acc);
            x[t] = acc;
        }
        __nv_bfloat16 *dst = (c < kDK ? w_out : u_out) + row0 * 128 + (c & 127);
#pragma unroll
        for (int t = 0; t < kC; t++) dst[t * 128] = __float2bfloat16_rn(x[t]);
    }
}

// ----------------------------------------------------------------- across chunks ----

__device__ __forceinline__ void unpack8(const __nv_bfloat16 *p, float *v) {
    Access<__nv_bfloat16, true>::unpack(*reinterpret_cast<const uint4 *>(p), v);
}

__global__ void __launch_bounds__(256) deltanet_scan_kernel(const __nv_bfloat16 *q, const __nv_bfloat16 *k,
                                                            const float *a, const __nv_bfloat16 *w_in,
                                                            const __nv_bfloat16 *u_in, const __nv_bfloat16 *p_in,
                                                            __nv_bfloat16 *o, int T) {
    extern __shared__ float sm[];
    float *S = sm;                                      // [128][32] the state slice
    float *Ut = S + kDK * kDVP;                         // [64][32]
    float *U = Ut + kC * kDVP;                          // [64][32]
    float *eca = U + kC * kDVP;                         // [64] exp(ca)
    float *ekd = eca + kC;                              // [64] exp(ca_C - ca)
    __nv_bfloat16 *Wh = reinterpret_cast<__nv_bfloat16 *>(ekd + kC);   // [64][136]
    __nv_bfloat16 *Qh = Wh + kC * kPadH;
    __nv_bfloat16 *Kh = Qh + kC * kPadH;
    __nv_bfloat16 *Ph = Kh + kC * kPadH;                // [64][72]
    __nv_bfloat16 *Oh = Ph + kC * kPadP;                // [32][72] output staging, [feature][position]
    __shared__ float gamma_sm;

    const int head = blockIdx.x, part = blockIdx.y;
    const int tid = threadIdx.x;
    const int chunks = T / kC;
    for (int i = tid; i < kDK * kDVP; i += 256) S[i] = 0.0f;

    const int ty = tid >> 3, tx = tid & 7;   // outputs [64][32]: rows 2ty, 2ty+1; columns 4tx..4tx+3
    for (int chunk = 0; chunk < chunks; chunk++) {
        const long long row0 = static_cast<long long>(head) * T + static_cast<long long>(chunk) * kC;
        __syncthreads();   // the previous chunk's readers are done with the tiles
        for (int i = tid; i < kC * kDK / 8; i += 256) {
            const int r = i / (kDK / 8), c = (i % (kDK / 8)) * 8;
            *reinterpret_cast<uint4 *>(Wh + r * kPadH + c) = __ldg(reinterpret_cast<const uint4 *>(w_in + (row0 + r) * kDK + c));
            *reinterpret_cast<uint4 *>(Qh + r * kPadH + c) = __ldg(reinterpret_cast<const uint4 *>(q + (row0 + r) * kDK + c));
            *reinterpret_cast<uint4 *>(Kh + r * kPadH + c) = __ldg(reinterpret_cast<const uint4 *>(k + (row0 + r) * kDK + c));
        }
        for (int i = tid; i < kC * kC / 8; i += 256) {
            const int r = i / (kC / 8), c = (i % (kC / 8)) * 8;
            *reinterpret_cast<uint4 *>(Ph + r * kPadP + c) =
                __ldg(reinterpret_cast<const uint4 *>(p_in + (static_cast<long long>(head) * chunks + chunk) * kC * kC + r * kC + c));
        }
        for (int i = tid; i < kC * kDVP / 8; i += 256) {
            const int r = i / (kDVP / 8), c = (i % (kDVP / 8)) * 8;
            float uv[8];
            Access<__nv_bfloat16, true>::load_cached(u_in + (row0 + r) * kDV + part * kDVP + c, uv);
#pragma unroll
            for (int e = 0; e < 8; e++) Ut[r * kDVP + c + e] = uv[e];
        }
        if (tid == 0) {
            float s = 0.0f;
            for (int t = 0; t < kC; t++) { s += a[row0 + t]; eca[t] = s; }
            const float last = s;
            for (int t = 0; t < kC; t++) { const float c = eca[t]; ekd[t] = __expf(last - c); eca[t] = __expf(c); }
            gamma_sm = __expf(last);
        }
        __syncthreads();

        // U = Ut - W S
        float acc[2][4];
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[r][j] = Ut[(2 * ty + r) * kDVP + 4 * tx + j];
        for (int i = 0; i < kDK; i += 8) {
            float w0[8], w1[8];
            unpack8(Wh + (2 * ty) * kPadH + i, w0);
            unpack8(Wh + (2 * ty + 1) * kPadH + i, w1);
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const float4 s4 = *reinterpret_cast<const float4 *>(S + (i + e) * kDVP + 4 * tx);
                acc[0][0] = fmaf(-w0[e], s4.x, acc[0][0]); acc[0][1] = fmaf(-w0[e], s4.y, acc[0][1]);
                acc[0][2] = fmaf(-w0[e], s4.z, acc[0][2]); acc[0][3] = fmaf(-w0[e], s4.w, acc[0][3]);
                acc[1][0] = fmaf(-w1[e], s4.x, acc[1][0]); acc[1][1] = fmaf(-w1[e], s4.y, acc[1][1]);
                acc[1][2] = fmaf(-w1[e], s4.z, acc[1][2]); acc[1][3] = fmaf(-w1[e], s4.w, acc[1][3]);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; r++)
            *reinterpret_cast<float4 *>(U + (2 * ty + r) * kDVP + 4 * tx) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
        __syncthreads();

        // o = (e^ca Q) S + P U
        float oa[2][4] = {};
        for (int i = 0; i < kDK; i += 8) {
            float q0[8], q1[8];
            unpack8(Qh + (2 * ty) * kPadH + i, q0);
            unpack8(Qh + (2 * ty + 1) * kPadH + i, q1);
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const float4 s4 = *reinterpret_cast<const float4 *>(S + (i + e) * kDVP + 4 * tx);
                oa[0][0] = fmaf(q0[e], s4.x, oa[0][0]); oa[0][1] = fmaf(q0[e], s4.y, oa[0][1]);
                oa[0][2] = fmaf(q0[e], s4.z, oa[0][2]); oa[0][3] = fmaf(q0[e], s4.w, oa[0][3]);
                oa[1][0] = fmaf(q1[e], s4.x, oa[1][0]); oa[1][1] = fmaf(q1[e], s4.y, oa[1][1]);
                oa[1][2] = fmaf(q1[e], s4.z, oa[1][2]); oa[1][3] = fmaf(q1[e], s4.w, oa[1][3]);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const float g = eca[2 * ty + r];
#pragma unroll
            for (int j = 0; j < 4; j++) oa[r][j] *= g;
        }
        for (int s = 0; s < kC; s += 8) {
            float p0[8], p1[8];
            unpack8(Ph + (2 * ty) * kPadP + s, p0);
            unpack8(Ph + (2 * ty + 1) * kPadP + s, p1);
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const float4 u4 = *reinterpret_cast<const float4 *>(U + (s + e) * kDVP + 4 * tx);
                oa[0][0] = fmaf(p0[e], u4.x, oa[0][0]); oa[0][1] = fmaf(p0[e], u4.y, oa[0][1]);
                oa[0][2] = fmaf(p0[e], u4.z, oa[0][2]); oa[0][3] = fmaf(p0[e], u4.w, oa[0][3]);
                oa[1][0] = fmaf(p1[e], u4.x, oa[1][0]); oa[1][1] = fmaf(p1[e], u4.y, oa[1][1]);
                oa[1][2] = fmaf(p1[e], u4.z, oa[1][2]); oa[1][3] = fmaf(p1[e], u4.w, oa[1][3]);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int j = 0; j < 4; j++) Oh[(4 * tx + j) * kPadP + 2 * ty + r] = __float2bfloat16_rn(oa[r][j]);
        __syncthreads();   // every reader of S is done; the staged output is complete

        // the result is (positions, features): 128 contiguous bytes per feature
        {
            const int f = tid >> 3, c = (tid & 7) * 8;
            *reinterpret_cast<uint4 *>(o + (static_cast<long long>(head) * kDV + part * kDVP + f) * T +
                                       static_cast<long long>(chunk) * kC + c) =
                *reinterpret_cast<const uint4 *>(Oh + f * kPadP + c);
        }
        // S <- e^{ca_C} S + (e^{ca_C - ca} K)' U : rows 4 ty2 .. +3 of S, columns 4 tx .. +3
        {
            const float gamma = gamma_sm;
            float sa[4][4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float4 s4 = *reinterpret_cast<const float4 *>(S + (4 * ty + i) * kDVP + 4 * tx);
                sa[i][0] = gamma * s4.x; sa[i][1] = gamma * s4.y; sa[i][2] = gamma * s4.z; sa[i][3] = gamma * s4.w;
            }
            for (int t = 0; t < kC; t++) {
                const float e = ekd[t];
                const uint2 kb = *reinterpret_cast<const uint2 *>(Kh + t * kPadH + 4 * ty);
                float kv[4];
                unpack_bf16x2(kb.x, kv[0], kv[1]);
                unpack_bf16x2(kb.y, kv[2], kv[3]);
                const float4 u4 = *reinterpret_cast<const float4 *>(U + t * kDVP + 4 * tx);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float kd = kv[i] * e;
                    sa[i][0] = fmaf(kd, u4.x, sa[i][0]); sa[i][1] = fmaf(kd, u4.y, sa[i][1]);
                    sa[i][2] = fmaf(kd, u4.z, sa[i][2]); sa[i][3] = fmaf(kd, u4.w, sa[i][3]);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
                *reinterpret_cast<float4 *>(S + (4 * ty + i) * kDVP + 4 * tx) = make_float4(sa[i][0], sa[i][1], sa[i][2], sa[i][3]);
        }
    }
}

constexpr size_t kChunkSmem = (2 * kC * kPadF + kC * kC + 2 * kC) * sizeof(float);
constexpr size_t kScanSmem = (kDK * kDVP + 2 * kC * kDVP + 2 * kC) * sizeof(float) +
                             (3 * kC * kPadH + kC * kPadP + kDVP * kPadP) * sizeof(__nv_bfloat16);

}  // namespace
}  // namespace tb200

using namespace tb200;

namespace {
int check_deltanet(const tb200_deltanet_desc *d) {
    if (!d) return TB200_ERR_NULL;
    if (d->heads < 0 || d->positions < 0) return TB200_ERR_SHAPE;
    if (d->dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (d->dk != kDK || d->dv != kDV || d->chunk != kC || d->positions % kC != 0) return TB200_ERR_UNSUPPORTED;
    return TB200_OK;
}
}  // namespace

extern "C" size_t tb200_deltanet_workspace_bytes(const tb200_deltanet_desc *d) {
    if (check_deltanet(d) != TB200_OK) return 0;
    const size_t rows = static_cast<size_t>(d->heads) * d->positions;
    return rows * (kDK + kDV + kC) * sizeof(__nv_bfloat16);
}

extern "C" int tb200_deltanet_fwd(const tb200_deltanet_desc *d, const void *q, const void *k, const void *v,
                                  const float *a, const float *beta, void *o, void *workspace, size_t workspace_bytes,
                                  void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int st = check_deltanet(d);
    if (st) return st;
    if (d->heads == 0 || d->positions == 0) return TB200_OK;
    if (!q || !k || !v || !a || !beta || !o) return TB200_ERR_NULL;
    if (!aligned_to(q, 16) || !aligned_to(k, 16) || !aligned_to(v, 16) || !aligned_to(o, 16) || !aligned_to(a, 4) ||
        !aligned_to(beta, 4))
        return TB200_ERR_ALIGN;
    const size_t need = tb200_deltanet_workspace_bytes(d);
    if (!workspace || workspace_bytes < need || !aligned_to(workspace, 16)) return TB200_ERR_WORKSPACE;
    DeviceInfo dev;
    if ((st = current_device(&dev))) return st;
    static std::mutex lock;
    static bool configured[64] = {};
    {
        std::lock_guard<std::mutex> hold(lock);
        if (!configured[dev.device]) {
            TB200_CUDA(cudaFuncSetAttribute(deltanet_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(kChunkSmem)));
            TB200_CUDA(cudaFuncSetAttribute(deltanet_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(kScanSmem)));
            configured[dev.device] = true;
        }
    }
    const size_t rows = static_cast<size_t>(d->heads) * d->positions;
    __nv_bfloat16 *w = static_cast<__nv_bfloat16 *>(workspace);
    __nv_bfloat16 *u = w + rows * kDK;
    __nv_bfloat16 *pw = u + rows * kDV;
    const int T = d->positions;
    const unsigned chunks = static_cast<unsigned>(d->heads) * (T / kC);
    deltanet_chunk_kernel<<<chunks, 256, kChunkSmem, stream>>>(
        static_cast<const __nv_bfloat16 *>(q), static_cast<const __nv_bfloat16 *>(k),
        static_cast<const __nv_bfloat16 *>(v), a, beta, w, u, pw, T);
    TB200_CUDA(cudaGetLastError());
    dim3 grid(static_cast<unsigned>(d->heads), kDV / kDVP);
    deltanet_scan_kernel<<<grid, 256, kScanSmem, stream>>>(static_cast<const __nv_bfloat16 *>(q),
                                                          static_cast<const __nv_bfloat16 *>(k), a, w, u, pw,
                                                          static_cast<__nv_bfloat16 *>(o), T);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}
