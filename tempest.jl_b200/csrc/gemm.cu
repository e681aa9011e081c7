// GEMM with fused epilogues for sm_100a.
//
// Fast path (BFloat16 in, Float32 accumulate): a persistent, warp-specialised
// kernel, one CTA per SM.  One thread issues TMA tile loads into a ring of
// 128-byte-swizzled shared-memory stages; one thread issues tcgen05.mma
// (128 x BN x 16 per instruction) accumulating in tensor memory; eight warps
// drain finished accumulators with tcgen05.ld, apply the epilogue in
// registers and store whole lines through a staging buffer.  Tensor memory
// holds two accumulator tiles, so the epilogue of tile i overlaps the main
// loop of tile i + 1; what is not hidden is the last tile's drain, which is
// why it is spread over eight warps.  Either operand may
// be K-major or MN-major in memory (all of NN / NT / TN / TT), which is what
// lets the backward products dX = dY * W' and dW = X' * dY read the forward's
// arrays in place.  No load uses cluster multicast.  A launch may hold a batch
// of alike products (the batch is the third coordinate of every tensor map)
// and may cut the sum over k into ranges (split-K): each (range, member, tile)
// is one work item of the persistent loop, the ranges' Float32 partial tiles
// go to a workspace and a second kernel merges them in range order and applies
// the epilogue.  BFloat16 or Float16 operands.
//
// Generic path: a shared-memory tiled SIMT kernel for Float32 operands, odd
// leading dimensions and anything else the TMA path cannot address.
//
// Every wait on an mbarrier is bounded: after about two seconds the kernel
// records an error code, stops issuing work and drains, so a pipeline bug ends
// as a status, not as a hung device.
#include <cuda.h>

#include <mutex>
#include <vector>

#include "common.cuh"
#include "sm100.cuh"

namespace tb200 {
namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;          // 64 BFloat16 = one 128-byte swizzle line
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 320;   // warp 0 loads, warp 1 issues MMAs, warps 2-9 run the epilogue
constexpr int kEpilogueWarps = 8;    // two per quarter of the accumulator's lanes, half of the tile's columns each
constexpr int kAccumStages = 2;

__device__ int g_gemm_error = 0;

struct GemmArgs {
    CUtensorMap tmap_a;
    CUtensorMap tmap_b;
    CUtensorMap tmap_aux;
    int staged_epilogue;     // results leave through the staging buffers in whole lines (aux arrives by TMA)
    void *c;
    const void *bias;
    const void *aux;
    void *aux_out;
    long long ldc, ld_aux, ld_aux_out;
    long long stride_c, stride_bias, stride_aux, stride_aux_out;   // between batch members, elements
    float alpha;
    int m, n, k;
    int epilogue;
    int in_f16;           // operands (and the bias) are Float16, not BFloat16
    int a_mn, b_mn;       // operand is MN-major in memory
    int a_batched, b_batched;   // 0: every member reads the same array
    int tiles_m, tiles_n;
    int batch;            // members
    int splits;           // ranges of the sum over k (1 = unsplit)
    int kb_per_split;     // 64-wide k blocks per range
    int stages;
    int debug;            // bit 0: the loader withholds its tiles (test hook)
    unsigned long long wait_ns;   // after which a bounded wait gives up
    int *schedule;        // null: work items dealt round-robin by block index.  Else two counters (next item,
                          // blocks finished), zero before the launch and left zero by it: every block takes
                          // its next item from the first, so a block that reaches its SM late (another kernel
                          // held it) takes fewer items instead of making the launch wait for its share
};

// ------------------------------------------------------------- epilogues ----

__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool PRECISE>
__device__ __forceinline__ float tanh_of(float x) {
    if constexpr (PRECISE) return tanhf(x);
    else return tanh_fast(x);
}

// gelu(x) = x/2 * (1 + tanh(0.7978846 (x + 0.044715 x^3)))   (test/fixtures/programs.jl:19 of the reference)
template <bool PRECISE>
__device__ __forceinline__ float gelu_tanh(float x) {
    const float u = 0.7978846f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanh_of<PRECISE>(u));
}
template <bool PRECISE>
__device__ __forceinline__ float gelu_tanh_grad(float x) {
    const float u = 0.7978846f * (x + 0.044715f * x * x * x);
    const float t = tanh_of<PRECISE>(u);
    const float du = 0.7978846f * (1.0f + 0.134145f * x * x);
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
}

// value written for accumulator `acc` (already scaled by alpha); `pre` receives what the activation saw
template <bool PRECISE>
__device__ __forceinline__ float epilogue_value(int kind, float acc, float bias, float aux, float &pre) {
    switch (kind) {
        case TB200_EPI_BIAS: return acc + bias;
        case TB200_EPI_BIAS_GELU: pre = acc + bias; return gelu_tanh<PRECISE>(pre);
        case TB200_EPI_BIAS_TANH: pre = acc + bias; return tanh_of<PRECISE>(pre);
        case TB200_EPI_MUL_GELU_GRAD: return acc * gelu_tanh_grad<PRECISE>(aux);
        case TB200_EPI_MUL_TANH_GRAD: return acc * (1.0f - aux * aux);
        case TB200_EPI_AXPY: return aux + acc;
        default: return acc;
    }
}

// The same with the kind known at compile time: the tensor-core kernel is instantiated per epilogue,
// which keeps its drain loop a few hundred instructions (a run-time switch inlined for each of a
// chunk's 32 values made the loop outgrow the instruction cache and the drain, not the MMAs, set the pace).
template <int EPI>
__device__ __forceinline__ float epilogue_fixed(float acc, float bias, float aux, float &pre) {
    if constexpr (EPI == TB200_EPI_BIAS) return acc + bias;
    else if constexpr (EPI == TB200_EPI_BIAS_GELU) { pre = acc + bias; return gelu_tanh<false>(pre); }
    else if constexpr (EPI == TB200_EPI_BIAS_TANH) { pre = acc + bias; return tanh_of<false>(pre); }
    else if constexpr (EPI == TB200_EPI_MUL_GELU_GRAD) return acc * gelu_tanh_grad<false>(aux);
    else if constexpr (EPI == TB200_EPI_MUL_TANH_GRAD) return acc * (1.0f - aux * aux);
    else if constexpr (EPI == TB200_EPI_AXPY) return aux + acc;
    else return acc;
}

__host__ __device__ constexpr bool epilogue_reads_bias(int kind) {
    return kind == TB200_EPI_BIAS || kind == TB200_EPI_BIAS_GELU || kind == TB200_EPI_BIAS_TANH;
}
__host__ __device__ constexpr bool epilogue_reads_aux(int kind) {
    return kind == TB200_EPI_MUL_GELU_GRAD || kind == TB200_EPI_MUL_TANH_GRAD || kind == TB200_EPI_AXPY;
}

__device__ __forceinline__ bool aligned_dev(const void *p, uintptr_t a) {
    return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

// Output element kinds of the tensor-core kernel.
constexpr int OUT_F32 = 0, OUT_BF16 = 1, OUT_F16 = 2;

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ void unpack_f16x2(uint32_t w, float &lo, float &hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w));
    lo = f.x; hi = f.y;
}
// two values rounded to the 16-bit output type OUT
template <int OUT>
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    if constexpr (OUT == OUT_F16) return pack_f16x2(lo, hi);
    else return pack_bf16x2(lo, hi);
}
// eight 16-bit values (Float16 when `f16`, else BFloat16) widened to Float32
__device__ __forceinline__ void unpack_half8(uint4 q, float *v, bool f16) {
    if (f16) {
        unpack_f16x2(q.x, v[0], v[1]); unpack_f16x2(q.y, v[2], v[3]);
        unpack_f16x2(q.z, v[4], v[5]); unpack_f16x2(q.w, v[6], v[7]);
    } else {
        Access<__nv_bfloat16, true>::unpack(q, v);
    }
}
__device__ __forceinline__ float half_to_f32(const void *p, long long i, bool f16) {
    return f16 ? __half2float(static_cast<const __half *>(p)[i])
               : __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
}

// `count` (<= 32) consecutive values of one output row, as Float32 or rounded to the 16-bit type;
// 128-bit stores when the whole chunk is there and the address allows.
template <int OUT>
__device__ __forceinline__ void store_row32(void *base, long long offset, const float (&v)[32], int count) {
    if constexpr (OUT == OUT_F32) {
        float *o = static_cast<float *>(base) + offset;
        if (count == 32 && aligned_dev(o, 16)) {
#pragma unroll
            for (int j = 0; j < 8; j++)
                reinterpret_cast<float4 *>(o)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (j < count) o[j] = v[j];
        }
    } else {
        uint16_t *o = static_cast<uint16_t *>(base) + offset;
        if (count == 32 && aligned_dev(o, 16)) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint4 q;
                q.x = pack_half2<OUT>(v[8 * j], v[8 * j + 1]);
                q.y = pack_half2<OUT>(v[8 * j + 2], v[8 * j + 3]);
                q.z = pack_half2<OUT>(v[8 * j + 4], v[8 * j + 5]);
                q.w = pack_half2<OUT>(v[8 * j + 6], v[8 * j + 7]);
                reinterpret_cast<uint4 *>(o)[j] = q;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (j < count) o[j] = static_cast<uint16_t>(pack_half2<OUT>(v[j], 0.0f) & 0xffffu);
        }
    }
}

// ------------------------------------------------------- tcgen05 kernel ----

__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait: false once `*failed` is set by anyone or `limit_ns` have passed.  PEER: a thread of the pair's
// other CTA arrives, after writing what this thread reads next.
template <bool PEER = false>
__device__ __forceinline__ bool wait_or_fail(uint64_t *bar, uint32_t parity, volatile int *failed, int code,
                                             unsigned long long limit_ns) {
    if (PEER ? mbar_wait_cluster(bar, parity, 4096) : mbar_wait(bar, parity, 4096)) return true;
    const uint64_t t0 = global_ns();
    while (true) {
        if (PEER ? mbar_wait_cluster(bar, parity, 1024) : mbar_wait(bar, parity, 1024)) return true;
        if (*failed) return false;
        if (global_ns() - t0 > limit_ns) {
            *failed = code;
            atomicCAS(&g_gemm_error, 0, code);
            return false;
        }
    }
}

constexpr int kStageLine = 128;                   // bytes per staged row: one 128-byte swizzle line
constexpr int kEpilogueStage = 32 * kStageLine;   // 32 rows of one warp

// One work item of the persistent loop: which range of the sum, which batch member, which tile.
struct WorkItem {
    int zc;        // third coordinate of the output (member, or range * batch + member when the sum is split)
    int member;
    int tm, tn;
    int kb0, kb1;  // 64-wide blocks of k
};
__device__ __forceinline__ WorkItem work_item(const GemmArgs &p, int item, int num_kb) {
    const int tiles = p.tiles_m * p.tiles_n;
    WorkItem w;
    w.zc = item / tiles;
    const int t = item - w.zc * tiles;
    w.tm = t / p.tiles_n;
    w.tn = t - w.tm * p.tiles_n;
    const int range = w.zc / p.batch;
    w.member = w.zc - range * p.batch;
    w.kb0 = range * p.kb_per_split;
    w.kb1 = w.kb0 + p.kb_per_split < num_kb ? w.kb0 + p.kb_per_split : num_kb;
    return w;
}

// 32 staged rows of 128 bytes (swizzled as the threads wrote them) to global memory: eight lanes a row, a
// 16-byte piece each, so a warp instruction writes four whole 128-byte lines.  `ES` bytes per element.
template <int ES>
__device__ __forceinline__ void flush_stage(const uint8_t *stage, uint8_t *base, long long pitch_bytes, int row0, int m,
                                            int col0, int n, int lane) {
    constexpr int PER = 16 / ES;
    const int piece = lane & 7, sub = lane >> 3;
    uint4 q[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int r = 4 * i + sub;
        q[i] = *reinterpret_cast<const uint4 *>(stage + r * kStageLine + ((piece ^ (r & 7)) << 4));
    }
    const int col = col0 + piece * PER;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int row = row0 + 4 * i + sub;
        if (row >= m || col >= n) continue;
        uint8_t *dst = base + row * pitch_bytes + static_cast<long long>(col) * ES;
        if (col + PER <= n) {
            *reinterpret_cast<uint4 *>(dst) = q[i];
        } else {
            // the row's last piece, cut by the edge of the array
            const uint32_t w[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
#pragma unroll
            for (int e = 0; e < PER; e++)
                if (col + e < n) {
                    if constexpr (ES == 4) reinterpret_cast<uint32_t *>(dst)[e] = w[e];
                    else reinterpret_cast<uint16_t *>(dst)[e] = static_cast<uint16_t>(w[e >> 1] >> ((e & 1) * 16));
                }
        }
    }
}

// 32 values of one row through the epilogue: acc -> v (what is stored), pre (what the activation saw).  Bias + GELU,
// the forward's epilogue, runs as packed pairs: gelu(x) = x/2 + x/2 tanh(x (c + 0.044715 c x^2)), c = 0.7978846.
template <int EPI>
__device__ __forceinline__ void epilogue_values(const uint32_t (&r)[32], float alpha, const float (&bv)[32],
                                                const float (&auxv)[32], float (&v)[32], float (&pre)[32]) {
    if constexpr (EPI == TB200_EPI_BIAS_GELU) {
        const float2 al = make_float2(alpha, alpha), c1 = make_float2(0.7978846f, 0.7978846f),
                     c2 = make_float2(0.7978846f * 0.044715f, 0.7978846f * 0.044715f), half = make_float2(0.5f, 0.5f);
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), al,
                                        make_float2(bv[j], bv[j + 1]));
            const float2 u = __fmul2_rn(x, __ffma2_rn(__fmul2_rn(x, x), c2, c1));
            const float2 hx = __fmul2_rn(x, half);
            const float2 y = __ffma2_rn(hx, make_float2(tanh_fast(u.x), tanh_fast(u.y)), hx);
            pre[j] = x.x; pre[j + 1] = x.y;
            v[j] = y.x; v[j + 1] = y.y;
        }
    } else if constexpr (EPI == TB200_EPI_MUL_GELU_GRAD) {
        // acc * gelu'(x), x the saved pre-activation: gelu'(x) = (1 + t) / 2 + x / 2 (1 - t^2) c (1 + 3 * 0.044715 x^2),
        // t = tanh(x c (1 + 0.044715 x^2)), c = 0.7978846; as packed pairs
        const float2 al = make_float2(alpha, alpha), c1 = make_float2(0.7978846f, 0.7978846f),
                     c2 = make_float2(0.7978846f * 0.044715f, 0.7978846f * 0.044715f),
                     c3 = make_float2(0.7978846f * 0.134145f, 0.7978846f * 0.134145f), half = make_float2(0.5f, 0.5f),
                     one = make_float2(1.0f, 1.0f), minus = make_float2(-1.0f, -1.0f);
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
            const float2 x = make_float2(auxv[j], auxv[j + 1]);
            const float2 x2 = __fmul2_rn(x, x);
            const float2 u = __fmul2_rn(x, __ffma2_rn(x2, c2, c1));
            const float2 t = make_float2(tanh_fast(u.x), tanh_fast(u.y));
            const float2 du = __ffma2_rn(x2, c3, c1);
            const float2 h = __ffma2_rn(t, half, half);
            const float2 omt2 = __ffma2_rn(__fmul2_rn(t, t), minus, one);
            const float2 grad = __ffma2_rn(__fmul2_rn(__fmul2_rn(x, half), omt2), du, h);
            const float2 a = __fmul2_rn(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), al);
            const float2 y = __fmul2_rn(a, grad);
            pre[j] = a.x; pre[j + 1] = a.y;
            v[j] = y.x; v[j + 1] = y.y;
        }
    } else {
        constexpr bool reads_bias = epilogue_reads_bias(EPI), reads_aux = epilogue_reads_aux(EPI);
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const float a = __uint_as_float(r[j]) * alpha;
            pre[j] = a;
            v[j] = epilogue_fixed<EPI>(a, reads_bias ? bv[j] : 0.0f, reads_aux ? auxv[j] : 0.0f, pre[j]);
        }
    }
}

// One epilogue warp's share of a finished accumulator tile -- 32 rows by `COLS` columns from column `c_off` of the
// tile -- through shared memory: the threads (one accumulator row each) write 32 rows x 128 bytes at a time into the
// warp's staging buffer (128-byte swizzled, so that a thread writing its own row does not collide with its
// neighbours), and the warp reads the buffer back a line at a time and stores whole 128-byte lines.  The operand an
// epilogue reads (aux) arrives in the same buffer by a TMA load and is taken into registers before the results go
// over it; a second result (the pre-activation values) goes through the buffer after the first.  `bias_q`: the tile's
// bias, eight columns a lane.  Returns false if a bounded wait gave up.
template <int COLS, int EPI, int OUT>
__device__ __forceinline__ bool epilogue_tile_staged(const GemmArgs &p, uint32_t tmem_acc, int row0, int n0, int c_off,
                                                     int zc, int member, int lane, uint8_t *stage, uint64_t *aux_bar,
                                                     uint32_t &aux_phase, volatile int *failed, uint4 bias_q) {
    constexpr int EPL = OUT == OUT_F32 ? 32 : 64;   // elements per 128-byte line
    constexpr int HALVES = EPL / 32;
    constexpr int ES = OUT == OUT_F32 ? 4 : 2;
    constexpr bool reads_bias = epilogue_reads_bias(EPI), reads_aux = epilogue_reads_aux(EPI);
    const bool has_aux_out = EPI == TB200_EPI_BIAS_GELU && p.aux_out != nullptr;
    const int sw = lane & 7;
    const bool in_f16 = p.in_f16 != 0;
    uint8_t *mine = stage + lane * kStageLine;
#pragma unroll 1
    for (int g = 0; g < COLS / EPL; g++) {
        const int col0 = n0 + c_off + g * EPL;
        if (col0 >= p.n) break;
        uint4 ax[8];
        if (reads_aux) {
            __syncwarp();   // every lane has read the previous group out of the buffer
            if (lane == 0) {
                mbar_arrive_expect_tx(aux_bar, kEpilogueStage);
                tma_load_3d(stage, &p.tmap_aux, aux_bar, col0, row0, member);
            }
            if (!wait_or_fail(aux_bar, aux_phase, failed, 5, p.wait_ns)) return false;
            aux_phase ^= 1;
#pragma unroll
            for (int j = 0; j < 8; j++) ax[j] = *reinterpret_cast<const uint4 *>(mine + ((j ^ sw) << 4));
        }
        __syncwarp();   // the buffer is free: the results may go over it
        uint4 zq[8];
#pragma unroll
        for (int h = 0; h < HALVES; h++) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_acc + c_off + g * EPL + h * 32, r);
            tmem_ld_wait();
            float auxv[32], bv[32];
            if (reads_aux) {
                if constexpr (OUT == OUT_F32) {
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        auxv[4 * j] = __uint_as_float(ax[j].x); auxv[4 * j + 1] = __uint_as_float(ax[j].y);
                        auxv[4 * j + 2] = __uint_as_float(ax[j].z); auxv[4 * j + 3] = __uint_as_float(ax[j].w);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++) unpack_half8(ax[4 * h + j], &auxv[8 * j], OUT == OUT_F16);
                }
            }
            if (reads_bias) {
                const int src = (c_off + g * EPL + h * 32) >> 3;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint4 q;
                    q.x = __shfl_sync(0xffffffffu, bias_q.x, src + j);
                    q.y = __shfl_sync(0xffffffffu, bias_q.y, src + j);
                    q.z = __shfl_sync(0xffffffffu, bias_q.z, src + j);
                    q.w = __shfl_sync(0xffffffffu, bias_q.w, src + j);
                    unpack_half8(q, &bv[8 * j], in_f16);
                }
            }
            float v[32], pre[32];
            epilogue_values<EPI>(r, p.alpha, bv, auxv, v, pre);
            if constexpr (OUT == OUT_F32) {
#pragma unroll
                for (int j = 0; j < 8; j++)
                    *reinterpret_cast<float4 *>(mine + ((j ^ sw) << 4)) =
                        make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint4 q;
                    q.x = pack_half2<OUT>(v[8 * j], v[8 * j + 1]);
                    q.y = pack_half2<OUT>(v[8 * j + 2], v[8 * j + 3]);
                    q.z = pack_half2<OUT>(v[8 * j + 4], v[8 * j + 5]);
                    q.w = pack_half2<OUT>(v[8 * j + 6], v[8 * j + 7]);
                    *reinterpret_cast<uint4 *>(mine + (((4 * h + j) ^ sw) << 4)) = q;
                    if (has_aux_out) {
                        zq[4 * h + j].x = pack_half2<OUT>(pre[8 * j], pre[8 * j + 1]);
                        zq[4 * h + j].y = pack_half2<OUT>(pre[8 * j + 2], pre[8 * j + 3]);
                        zq[4 * h + j].z = pack_half2<OUT>(pre[8 * j + 4], pre[8 * j + 5]);
                        zq[4 * h + j].w = pack_half2<OUT>(pre[8 * j + 6], pre[8 * j + 7]);
                    }
                }
            }
        }
        __syncwarp();
        flush_stage<ES>(stage, static_cast<uint8_t *>(p.c) + static_cast<long long>(zc) * p.stride_c * ES, p.ldc * ES, row0,
                        p.m, col0, p.n, lane);
        if constexpr (OUT != OUT_F32) {
            if (has_aux_out) {
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 8; j++) *reinterpret_cast<uint4 *>(mine + ((j ^ sw) << 4)) = zq[j];
                __syncwarp();
                flush_stage<2>(stage, static_cast<uint8_t *>(p.aux_out) + static_cast<long long>(member) * p.stride_aux_out * 2,
                               p.ld_aux_out * 2, row0, p.m, col0, p.n, lane);
            }
        }
    }
    return true;
}

// PAIR: launched as clusters of two CTAs that share tiles of 256 x BN -- each CTA loads its 128 rows of A and its
// half of B's columns, the first CTA's MMA thread issues 256-row instructions that read both, each CTA drains its own
// 128 rows.  Per CTA and 64 of k that is 32 KB from L2 instead of 48 KB for the same 128 x 256 x 64 of work, and the
// ring is six stages deep.  Both CTAs' loads count on the first CTA's barrier, where the MMA thread waits (plain
// loads with one destination each: no multicast); the MMAs' completion arrives on both CTAs' barriers.
template <int BN, int EPI, int OUT, bool PAIR = false>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_tcgen05(const __grid_constant__ GemmArgs p) {
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzle atoms are 1024 bytes: align the ring
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int ROWS = PAIR ? 2 * BM : BM;     // rows of a tile
    constexpr int BNL = PAIR ? BN / 2 : BN;      // columns of B this CTA loads
    constexpr uint32_t A_BYTES = BM * BK * 2;
    constexpr uint32_t B_BYTES = BNL * BK * 2;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int MAX_STAGES = 8;

    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t tmem_full_bar[kAccumStages];
    __shared__ __align__(8) uint64_t tmem_empty_bar[kAccumStages];
    __shared__ __align__(8) uint64_t aux_bar[kEpilogueWarps];
    // the work items of this block, handed from the loading thread to the MMA thread and the epilogue warps
    constexpr int kItemSlots = 4;
    __shared__ __align__(8) uint64_t item_full[kItemSlots];
    __shared__ __align__(8) uint64_t item_empty[kItemSlots];
    __shared__ int item_slot[kItemSlots];
    // pair with a tile counter: the first CTA's loading thread draws the items and writes them into the second's ring
    __shared__ __align__(8) uint64_t mail_full[kItemSlots];    // used in the second CTA: an item has arrived
    __shared__ __align__(8) uint64_t mail_empty[kItemSlots];   // used in the first CTA: the second has read it
    __shared__ int mail_item[kItemSlots];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int failed_smem;
    volatile int *failed = &failed_smem;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int stages = p.stages;
    const int num_kb = (p.k + BK - 1) / BK;
    const int num_items = p.tiles_m * p.tiles_n * p.batch * p.splits;
    const unsigned long long wait_ns = p.wait_ns;
    const uint32_t rank = PAIR ? cluster_rank() : 0u;

    if (threadIdx.x == 0) {
        failed_smem = 0;
        for (int s = 0; s < stages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < kAccumStages; s++) {
            mbar_init(&tmem_full_bar[s], 1);
            mbar_init(&tmem_empty_bar[s], PAIR ? 2 * kEpilogueWarps : kEpilogueWarps);   // pair: both CTAs' warps
        }
        for (int s = 0; s < kEpilogueWarps; s++) mbar_init(&aux_bar[s], 1);
        for (int s = 0; s < kItemSlots; s++) {
            mbar_init(&mail_full[s], 1);
            mbar_init(&mail_empty[s], 1);
            mbar_init(&item_full[s], 1);
            mbar_init(&item_empty[s], 1 + kEpilogueWarps);   // the MMA thread and one lane of each epilogue warp
        }
        fence_barrier_init();
        prefetch_tensormap(&p.tmap_a);
        prefetch_tensormap(&p.tmap_b);
        if (p.staged_epilogue && epilogue_reads_aux(EPI)) prefetch_tensormap(&p.tmap_aux);
    }
    if (warp == 1) {
        // each CTA of a pair allocates its own tensor memory: all of it, so both get the same (first) column
        tmem_alloc(&tmem_base_smem, kAccumStages * BN);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    if constexpr (PAIR) cluster_sync_all();   // the other CTA's barriers are initialised before anything arrives on them
    else __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_smem;
    // barriers, tensor memory and descriptors are ready; global memory is touched from here on
    grid_dependency_wait();

    if (warp == 0) {
        // ---- TMA producer; it also draws the block's work items and passes them on (with the test hook set it
        // passes the items on but loads nothing: every consumer's wait for operands then runs out)
        if (elect_one()) {
            int stage = 0, slot = 0;
            uint32_t phase = 0, slot_phase = 0;
            const bool withhold = (p.debug & 1) != 0;
            // a pair takes its tiles by the cluster's index: both CTAs walk the same list
            const int first = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
            const int step = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
            const bool drawn = p.schedule != nullptr;          // items come from the plan's counter
            const bool draws = drawn && rank == 0;             // ... which this thread reads
            const bool told = PAIR && drawn && rank != 0;      // ... or the first CTA's loading thread tells it
            int item = draws ? atomicAdd(p.schedule, 1) : first;
            int mslot = 0;
            uint32_t mphase = 0;
            while (true) {
                if (!wait_or_fail(&item_empty[slot], slot_phase ^ 1, failed, 6, wait_ns)) break;
                if (told) {
                    if (!wait_or_fail<true>(&mail_full[mslot], mphase, failed, 10, wait_ns)) break;
                    item = mail_item[mslot];
                    mbar_arrive_cluster(cluster_map(&mail_empty[mslot], 0));
                    if (++mslot == kItemSlots) { mslot = 0; mphase ^= 1; }
                }
                const bool live = item >= 0 && item < num_items && !*failed;
                if (PAIR && draws) {
                    if (!wait_or_fail(&mail_empty[mslot], mphase ^ 1, failed, 11, wait_ns)) break;
                    st_cluster_u32(cluster_map(&mail_item[mslot], 1), static_cast<uint32_t>(live ? item : -1));
                    mbar_arrive_cluster(cluster_map(&mail_full[mslot], 1));
                    if (++mslot == kItemSlots) { mslot = 0; mphase ^= 1; }
                }
                item_slot[slot] = live ? item : -1;
                mbar_arrive(&item_full[slot]);
                if (++slot == kItemSlots) { slot = 0; slot_phase ^= 1; }
                if (!live) break;
                // the next item is drawn now, so that the answer is there when this one's loads are out
                const int next = draws ? atomicAdd(p.schedule, 1) : item + step;
                const WorkItem w = work_item(p, item, num_kb);
                item = next;
                if (withhold) continue;
                const int m0 = w.tm * ROWS + static_cast<int>(rank) * BM, n0 = w.tn * BN + static_cast<int>(rank) * (BN - BNL);
                const int za = p.a_batched ? w.member : 0, zb = p.b_batched ? w.member : 0;
                for (int kb = w.kb0; kb < w.kb1; kb++) {
                    if (!wait_or_fail(&empty_bar[stage], phase ^ 1, failed, 1, wait_ns)) break;

                    uint8_t *sa = smem + stage * STAGE_BYTES;
                    uint8_t *sb = sa + A_BYTES;
                    const int k0 = kb * BK;
                    if constexpr (PAIR) {
                        // both CTAs' operands are counted on the first CTA's barrier, where the MMA thread waits
                        if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
                        const uint32_t bar = cluster_map(&full_bar[stage], 0);
                        if (p.a_mn) {
                            for (int j = 0; j < BM / 64; j++)
                                tma_load_3d_pair(sa + j * (BK * 128), &p.tmap_a, bar, m0 + j * 64, k0, za);
                        } else {
                            tma_load_3d_pair(sa, &p.tmap_a, bar, k0, m0, za);
                        }
                        if (p.b_mn) {
                            for (int j = 0; j < BNL / 64; j++)
                                tma_load_3d_pair(sb + j * (BK * 128), &p.tmap_b, bar, n0 + j * 64, k0, zb);
                        } else {
                            tma_load_3d_pair(sb, &p.tmap_b, bar, k0, n0, zb);
                        }
                    } else {
                        mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
                        if (p.a_mn) {   // [K][M]: slabs of 64 along M, each 64 K-lines of 128 bytes
                            for (int j = 0; j < BM / 64; j++)
                                tma_load_3d(sa + j * (BK * 128), &p.tmap_a, &full_bar[stage], m0 + j * 64, k0, za);
                        } else {        // [M][K]: 128 rows of 128 bytes
                            tma_load_3d(sa, &p.tmap_a, &full_bar[stage], k0, m0, za);
                        }
                        if (p.b_mn) {
                            for (int j = 0; j < BNL / 64; j++)
                                tma_load_3d(sb + j * (BK * 128), &p.tmap_b, &full_bar[stage], n0 + j * 64, k0, zb);
                        } else {
                            tma_load_3d(sb, &p.tmap_b, &full_bar[stage], k0, n0, zb);
                        }
                    }
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1 && PAIR && rank != 0) {
        // ---- second CTA of a pair: no MMAs are issued here; the items are taken and let go
        if (elect_one()) {
            int slot = 0;
            uint32_t slot_phase = 0;
            for (;;) {
                if (!wait_or_fail(&item_full[slot], slot_phase, failed, 7, wait_ns)) break;
                const int item = item_slot[slot];
                mbar_arrive(&item_empty[slot]);
                if (++slot == kItemSlots) { slot = 0; slot_phase ^= 1; }
                if (item < 0 || *failed) break;
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (elect_one()) {
            const uint32_t idesc = p.in_f16 ? umma_idesc_f16(ROWS, BN, p.a_mn != 0, p.b_mn != 0)
                                            : umma_idesc_bf16(ROWS, BN, p.a_mn != 0, p.b_mn != 0);
            // K-major: 8-row groups 1024 bytes apart, 32 bytes per 16 K; MN-major: slabs BK*128 bytes
            // apart, 8-line groups 1024 bytes apart, 2048 bytes per 16 K
            const uint32_t a_lead = p.a_mn ? BK * 128 : 16, b_lead = p.b_mn ? BK * 128 : 16;
            const uint32_t a_step = (p.a_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4;
            const uint32_t b_step = (p.b_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4;
            int stage = 0, it = 0, slot = 0;
            uint32_t phase = 0, slot_phase = 0;
            for (;; it++) {
                if (!wait_or_fail(&item_full[slot], slot_phase, failed, 7, wait_ns)) break;
                const int item = item_slot[slot];
                mbar_arrive(&item_empty[slot]);
                if (++slot == kItemSlots) { slot = 0; slot_phase ^= 1; }
                if (item < 0 || *failed) break;
                const WorkItem w = work_item(p, item, num_kb);
                const int acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!wait_or_fail(&tmem_empty_bar[acc], acc_phase ^ 1, failed, 2, wait_ns)) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = w.kb0; kb < w.kb1; kb++) {
                    if (!wait_or_fail(&full_bar[stage], phase, failed, 3, wait_ns)) break;
                    tcgen05_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    const uint64_t a_desc = umma_smem_desc(sa, a_lead, 1024);
                    const uint64_t b_desc = umma_smem_desc(sa + A_BYTES, b_lead, 1024);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        if constexpr (PAIR)
                            tcgen05_mma_f16_pair(d_tmem, a_desc + k * a_step, b_desc + k * b_step, idesc,
                                                 ((kb - w.kb0) | k) != 0);
                        else
                            tcgen05_mma_f16(d_tmem, a_desc + k * a_step, b_desc + k * b_step, idesc,
                                            ((kb - w.kb0) | k) != 0);
                    }
                    // the stage is free (in both CTAs of a pair) once these MMAs have read it
                    if constexpr (PAIR) tcgen05_commit_pair(&empty_bar[stage]);
                    else tcgen05_commit(&empty_bar[stage]);
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
                if (*failed) break;
                // the accumulator is complete (in both CTAs of a pair)
                if constexpr (PAIR) tcgen05_commit_pair(&tmem_full_bar[acc]);
                else tcgen05_commit(&tmem_full_bar[acc]);
            }
        }
    } else {
        // ---- epilogue: warps q and q + 4 own tensor-memory lanes [32 q, 32 q + 32), half of the tile's columns each
        const int q = warp & 3;
        const int c_off = ((warp - 2) >> 2) * (BN / 2);
        int it = 0;
        // staging for the epilogue sits behind the operand ring: one buffer of 32 lines per warp
        uint8_t *stage = smem + stages * STAGE_BYTES + (warp - 2) * kEpilogueStage;
        uint32_t aux_phase = 0;
        const bool in_f16 = p.in_f16 != 0;
        int slot = 0;
        uint32_t slot_phase = 0;
        for (;; it++) {
            if (!wait_or_fail(&item_full[slot], slot_phase, failed, 7, wait_ns)) break;
            const int item = item_slot[slot];
            __syncwarp();
            if (lane == 0) mbar_arrive(&item_empty[slot]);
            if (++slot == kItemSlots) { slot = 0; slot_phase ^= 1; }
            if (item < 0) break;
            const WorkItem w = work_item(p, item, num_kb);
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            // the tile's bias, eight columns a lane, fetched while the accumulator is still being summed
            uint4 bias_q = make_uint4(0u, 0u, 0u, 0u);
            if (epilogue_reads_bias(EPI) && p.staged_epilogue && lane < BN / 8) {
                const int col = w.tn * BN + lane * 8;
                const uint16_t *bp = static_cast<const uint16_t *>(p.bias) + w.member * p.stride_bias + col;
                if (col + 8 <= p.n && aligned_dev(bp, 16)) {
                    bias_q = __ldg(reinterpret_cast<const uint4 *>(bp));
                } else {
                    uint32_t h[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) h[e] = col + e < p.n ? bp[e] : 0u;
                    bias_q = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
                }
            }
            if (!wait_or_fail(&tmem_full_bar[acc], acc_phase, failed, 4, wait_ns)) break;
            tcgen05_fence_after();
            if (p.staged_epilogue) {
                const int row0 = w.tm * ROWS + static_cast<int>(rank) * BM + q * 32;
                const uint32_t tmem_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
                bool ok = true;
                if (row0 < p.m)
                    ok = epilogue_tile_staged<BN / 2, EPI, OUT>(p, tmem_acc, row0, w.tn * BN, c_off, w.zc, w.member, lane,
                                                                stage, &aux_bar[warp - 2], aux_phase, failed, bias_q);
                if (!ok) break;
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (PAIR) mbar_arrive_cluster(cluster_map(&tmem_empty_bar[acc], 0));
                    else mbar_arrive(&tmem_empty_bar[acc]);
                }
                continue;
            }
            const int m = w.tm * ROWS + static_cast<int>(rank) * BM + q * 32 + lane;
            const int n0 = w.tn * BN;
            const bool row_ok = m < p.m;
            constexpr bool reads_bias = epilogue_reads_bias(EPI), reads_aux = epilogue_reads_aux(EPI);
            const long long c_base = static_cast<long long>(w.zc) * p.stride_c + static_cast<long long>(m) * p.ldc;
            const long long x_base = static_cast<long long>(w.member) * p.stride_aux + static_cast<long long>(m) * p.ld_aux;
            const long long o_base =
                static_cast<long long>(w.member) * p.stride_aux_out + static_cast<long long>(m) * p.ld_aux_out;
            const void *bias = static_cast<const uint16_t *>(p.bias) + w.member * p.stride_bias;
#pragma unroll 1
            for (int c = c_off / 32; c < (c_off + BN / 2) / 32; c++) {
                uint32_t r[32];
                __syncwarp();   // rows past the edge skip the stores below: rejoin before the warp-wide load
                tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32, r);
                tmem_ld_wait();
                const int col0 = n0 + c * 32;
                if (!row_ok || col0 >= p.n) continue;
                const bool whole = col0 + 32 <= p.n;
                float v[32], pre[32];
#pragma unroll
                for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]) * p.alpha;
                float auxv[32];
                if (reads_aux) {
                    if (OUT == OUT_F32 && EPI == TB200_EPI_AXPY) {
                        const float *ap = static_cast<const float *>(p.aux) + x_base + col0;
#pragma unroll
                        for (int j = 0; j < 32; j++) auxv[j] = (whole || col0 + j < p.n) ? ap[j] : 0.0f;
                    } else {
                        // the activation pullbacks read the operands' type, the accumulating epilogue the result's
                        const bool aux_f16 = EPI == TB200_EPI_AXPY ? OUT == OUT_F16 : in_f16;
                        const uint16_t *ap = static_cast<const uint16_t *>(p.aux) + x_base + col0;
                        if (whole && aligned_dev(ap, 16)) {
#pragma unroll
                            for (int j = 0; j < 4; j++)
                                unpack_half8(__ldg(reinterpret_cast<const uint4 *>(ap) + j), &auxv[j * 8], aux_f16);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++) auxv[j] = (col0 + j < p.n) ? half_to_f32(ap, j, aux_f16) : 0.0f;
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    float b = 0.0f;
                    if (reads_bias && (whole || col0 + j < p.n)) b = half_to_f32(bias, col0 + j, in_f16);
                    pre[j] = v[j];
                    v[j] = epilogue_fixed<EPI>(v[j], b, reads_aux ? auxv[j] : 0.0f, pre[j]);
                }
                store_row32<OUT>(p.c, c_base + col0, v, whole ? 32 : p.n - col0);
                if (p.aux_out) {
                    if (in_f16) store_row32<OUT_F16>(p.aux_out, o_base + col0, pre, whole ? 32 : p.n - col0);
                    else store_row32<OUT_BF16>(p.aux_out, o_base + col0, pre, whole ? 32 : p.n - col0);
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR) mbar_arrive_cluster(cluster_map(&tmem_empty_bar[acc], 0));
                else mbar_arrive(&tmem_empty_bar[acc]);
            }
        }
    }

    tcgen05_fence_before();
    // neither CTA of a pair leaves (or frees tensor memory) while the other may still arrive on its barriers
    if constexpr (PAIR) cluster_sync_all();
    else __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kAccumStages * BN);
    }
    // the last block out leaves the two counters as it found them, for the next launch
    if (p.schedule && threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(p.schedule + 1, 1) == static_cast<int>(gridDim.x) - 1) {
            p.schedule[0] = 0;
            p.schedule[1] = 0;
            __threadfence();
        }
    }
}

// Split-K, second launch: C = epilogue(alpha * sum over ranges of the partial tiles), ranges added in order.
struct MergeArgs {
    const float *partial;   // [range][member][m][ld_partial]
    void *c;
    const void *bias, *aux;
    void *aux_out;
    long long ld_partial, ldc, ld_aux, ld_aux_out;
    long long stride_c, stride_bias, stride_aux, stride_aux_out;
    float alpha;
    int m, n, batch, splits;
    int epilogue;
    int in_dtype, out_dtype;
};

__global__ void __launch_bounds__(256) gemm_splitk_merge(const MergeArgs q) {
    const long long per_member = static_cast<long long>(q.m) * q.n;
    const long long total = per_member * q.batch;
    const bool reads_bias = epilogue_reads_bias(q.epilogue), reads_aux = epilogue_reads_aux(q.epilogue);
    const int aux_dtype = q.epilogue == TB200_EPI_AXPY ? q.out_dtype : q.in_dtype;
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
        const int member = static_cast<int>(i / per_member);
        const long long r = i - member * per_member;
        const int row = static_cast<int>(r / q.n), col = static_cast<int>(r - static_cast<long long>(row) * q.n);
        float acc = 0.0f;
        for (int s = 0; s < q.splits; s++)
            acc += q.partial[((static_cast<long long>(s) * q.batch + member) * q.m + row) * q.ld_partial + col];
        const float b = reads_bias ? load_elem(q.bias, member * q.stride_bias + col, q.in_dtype) : 0.0f;
        const float x = reads_aux ? load_elem(q.aux, member * q.stride_aux + row * q.ld_aux + col, aux_dtype) : 0.0f;
        float pre = acc * q.alpha;
        const float v = epilogue_value<false>(q.epilogue, pre, b, x, pre);
        store_elem(q.c, member * q.stride_c + row * q.ldc + col, v, q.out_dtype);
        if (q.aux_out) store_elem(q.aux_out, member * q.stride_aux_out + row * q.ld_aux_out + col, pre, q.in_dtype);
    }
}

// --------------------------------------------------------- SIMT kernel ----
// C[M][N] = epilogue(alpha * A * B): 64 x 64 tile per block of 256 threads, 4 x 4 outputs per thread,
// operands through shared memory in Float32.  Any layout, any leading dimension, any element type;
// batch members along the grid's third axis.

struct SimtArgs {
    const void *a, *b;
    void *c;
    const void *bias, *aux;
    void *aux_out;
    long long lda, ldb, ldc, ld_aux, ld_aux_out;
    long long stride_a, stride_b, stride_c, stride_bias, stride_aux, stride_aux_out;
    float alpha;
    int m, n, k, batch;
    int epilogue;
    int in_dtype, out_dtype;
    int a_mn, b_mn;
};

__global__ void __launch_bounds__(256) gemm_simt(const SimtArgs p) {
    __shared__ float sa[16][65];
    __shared__ float sb[16][65];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const bool reads_bias = epilogue_reads_bias(p.epilogue), reads_aux = epilogue_reads_aux(p.epilogue);
    const int aux_dtype = p.epilogue == TB200_EPI_AXPY ? p.out_dtype : p.in_dtype;
    for (int member = blockIdx.z; member < p.batch; member += gridDim.z) {
        const long long a0 = member * p.stride_a, b0 = member * p.stride_b;
        float acc[4][4] = {};
        for (int k0 = 0; k0 < p.k; k0 += 16) {
            for (int i = threadIdx.x; i < 64 * 16; i += 256) {
                // consecutive threads walk the operand's contiguous axis
                int mm, kk;
                if (p.a_mn) { mm = i & 63; kk = i >> 6; } else { kk = i & 15; mm = i >> 4; }
                const int gm = m0 + mm, gk = k0 + kk;
                float v = 0.0f;
                if (gm < p.m && gk < p.k)
                    v = load_elem(p.a, a0 + (p.a_mn ? static_cast<long long>(gk) * p.lda + gm
                                                    : static_cast<long long>(gm) * p.lda + gk), p.in_dtype);
                sa[kk][mm] = v;
                int nn;
                if (p.b_mn) { nn = i & 63; kk = i >> 6; } else { kk = i & 15; nn = i >> 4; }
                const int gn = n0 + nn;
                const int gk2 = k0 + kk;
                v = 0.0f;
                if (gn < p.n && gk2 < p.k)
                    v = load_elem(p.b, b0 + (p.b_mn ? static_cast<long long>(gk2) * p.ldb + gn
                                                    : static_cast<long long>(gn) * p.ldb + gk2), p.in_dtype);
                sb[kk][nn] = v;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < 16; kk++) {
                float av[4], bv[4];
#pragma unroll
                for (int i = 0; i < 4; i++) { av[i] = sa[kk][ty * 4 + i]; bv[i] = sb[kk][tx * 4 + i]; }
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
            }
            __syncthreads();
        }
        for (int i = 0; i < 4; i++)
            for (int j = 0; j < 4; j++) {
                const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
                if (m >= p.m || n >= p.n) continue;
                const float b = reads_bias ? load_elem(p.bias, member * p.stride_bias + n, p.in_dtype) : 0.0f;
                const float x = reads_aux ? load_elem(p.aux, member * p.stride_aux + static_cast<long long>(m) * p.ld_aux + n, aux_dtype)
                                          : 0.0f;
                float pre = acc[i][j] * p.alpha;
                const float v = epilogue_value<true>(p.epilogue, pre, b, x, pre);
                store_elem(p.c, member * p.stride_c + static_cast<long long>(m) * p.ldc + n, v, p.out_dtype);
                if (p.aux_out)
                    store_elem(p.aux_out, member * p.stride_aux_out + static_cast<long long>(m) * p.ld_aux_out + n, pre,
                               p.in_dtype);
            }
    }
}

// ------------------------------------------------------------ host side ----

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_fn(EncodeTiledFn *out) {
    static std::mutex lock;
    static EncodeTiledFn fn = nullptr;
    std::lock_guard<std::mutex> hold(lock);
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        TB200_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres));
        if (!sym || qres != cudaDriverEntryPointSuccess) return TB200_ERR_UNSUPPORTED;
        fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    *out = fn;
    return TB200_OK;
}

// `members` 2-D arrays of `rows` x `cols` (cols contiguous, row pitch ld elements, `member_stride` elements from
// one array to the next) as 128-byte-swizzled boxes of box_rows rows x 128 bytes (64 16-bit or 32 Float32
// elements) of one member.
int make_tmap(CUtensorMap *map, const void *base, int64_t cols, int64_t rows, int64_t ld, int box_rows, int dtype,
              int64_t members = 1, int64_t member_stride = 0) {
    EncodeTiledFn fn;
    int st = encode_fn(&fn);
    if (st) return st;
    const cuuint64_t es = dtype == TB200_F32 ? 4 : 2;
    if (members < 1) members = 1;
    // an axis of one element still needs a legal pitch: any multiple of 16 bytes that covers the array
    cuuint64_t pitch2 = static_cast<cuuint64_t>(member_stride) * es;
    if (members == 1 || pitch2 == 0) pitch2 = ((static_cast<cuuint64_t>(rows) * ld * es + 15) / 16) * 16;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(members)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * es, pitch2};
    cuuint32_t box[3] = {static_cast<cuuint32_t>(128 / es), static_cast<cuuint32_t>(box_rows), 1};
    cuuint32_t elem[3] = {1, 1, 1};
    const CUtensorMapDataType type = dtype == TB200_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                     : dtype == TB200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                          : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    CUresult r = fn(map, type, 3, const_cast<void *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TB200_OK : TB200_ERR_UNSUPPORTED;
}

// The kernel instantiation for (tile width, epilogue, result type), its shared-memory attribute set once per device.
template <int BN, int EPI, int OUT, bool PAIR>
int kernel_for(const DeviceInfo &dev, const void **fn) {
    static std::mutex lock;
    static bool configured[64] = {};
    std::lock_guard<std::mutex> hold(lock);
    if (!configured[dev.device]) {
        TB200_CUDA(cudaFuncSetAttribute(gemm_tcgen05<BN, EPI, OUT, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(dev.smem_optin - 1024)));
        configured[dev.device] = true;
    }
    *fn = reinterpret_cast<const void *>(&gemm_tcgen05<BN, EPI, OUT, PAIR>);
    return TB200_OK;
}

template <int BN, int OUT, bool PAIR = false>
int kernel_by_epilogue(int epilogue, const DeviceInfo &dev, const void **fn) {
    switch (epilogue) {
        case TB200_EPI_NONE: return kernel_for<BN, TB200_EPI_NONE, OUT, PAIR>(dev, fn);
        case TB200_EPI_BIAS: return kernel_for<BN, TB200_EPI_BIAS, OUT, PAIR>(dev, fn);
        case TB200_EPI_AXPY: return kernel_for<BN, TB200_EPI_AXPY, OUT, PAIR>(dev, fn);
        default: break;
    }
    // activations and their pullbacks are instantiated for BFloat16 results only
    if constexpr (OUT == OUT_BF16) {
        switch (epilogue) {
            case TB200_EPI_BIAS_GELU: return kernel_for<BN, TB200_EPI_BIAS_GELU, OUT, PAIR>(dev, fn);
            case TB200_EPI_BIAS_TANH: return kernel_for<BN, TB200_EPI_BIAS_TANH, OUT, PAIR>(dev, fn);
            case TB200_EPI_MUL_GELU_GRAD: return kernel_for<BN, TB200_EPI_MUL_GELU_GRAD, OUT, PAIR>(dev, fn);
            case TB200_EPI_MUL_TANH_GRAD: return kernel_for<BN, TB200_EPI_MUL_TANH_GRAD, OUT, PAIR>(dev, fn);
            default: break;
        }
    }
    return TB200_ERR_UNSUPPORTED;
}

// How many CTA pairs of `kernel` the device holds at once.  A part with an odd number of multiprocessors left in
// some cluster of its die holds fewer pairs than half its multiprocessor count, and a grid with more pairs than
// that would run the surplus after the rest has finished: with a fixed share of the tiles each, at twice the
// time.  Asked of the driver once per device and kernel; half the multiprocessors if it does not answer.
int resident_pairs(const void *kernel, size_t smem, const DeviceInfo &dev) {
    struct Known { int device; const void *kernel; int pairs; };
    static std::mutex lock;
    static std::vector<Known> known;
    std::lock_guard<std::mutex> hold(lock);
    for (const Known &k : known)
        if (k.device == dev.device && k.kernel == kernel) return k.pairs;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(dev.sms / 2 * 2));
    config.blockDim = dim3(kGemmThreads);
    config.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    config.attrs = &attr;
    config.numAttrs = 1;
    int pairs = 0;
    if (cudaOccupancyMaxActiveClusters(&pairs, kernel, &config) != cudaSuccess || pairs <= 0) {
        cudaGetLastError();
        pairs = dev.sms / 2;
    }
    if (pairs > dev.sms / 2) pairs = dev.sms / 2;
    known.push_back(Known{dev.device, kernel, pairs});
    return pairs;
}

int kernel_by_shape(int bn, bool pair, int out_dtype, int epilogue, const DeviceInfo &dev, const void **fn) {
    if (pair) {
        if (out_dtype == TB200_F32) return kernel_by_epilogue<256, OUT_F32, true>(epilogue, dev, fn);
        if (out_dtype == TB200_F16) return kernel_by_epilogue<256, OUT_F16, true>(epilogue, dev, fn);
        return kernel_by_epilogue<256, OUT_BF16, true>(epilogue, dev, fn);
    }
    if (bn == 256) {
        if (out_dtype == TB200_F32) return kernel_by_epilogue<256, OUT_F32>(epilogue, dev, fn);
        if (out_dtype == TB200_F16) return kernel_by_epilogue<256, OUT_F16>(epilogue, dev, fn);
        return kernel_by_epilogue<256, OUT_BF16>(epilogue, dev, fn);
    }
    if (out_dtype == TB200_F32) return kernel_by_epilogue<128, OUT_F32>(epilogue, dev, fn);
    if (out_dtype == TB200_F16) return kernel_by_epilogue<128, OUT_F16>(epilogue, dev, fn);
    return kernel_by_epilogue<128, OUT_BF16>(epilogue, dev, fn);
}

bool is_activation(int e) {
    return e == TB200_EPI_BIAS_GELU || e == TB200_EPI_BIAS_TANH || e == TB200_EPI_MUL_GELU_GRAD ||
           e == TB200_EPI_MUL_TANH_GRAD;
}

// How many ranges the sum over k is cut into, and how many 64-wide blocks each takes.
void choose_split(const tb200_gemm_desc &d, int bn, int sms, int *splits, int *kb_per_split) {
    const int64_t batch = d.batch > 1 ? d.batch : 1;
    const int64_t tiles = ceil_div(d.m, BM) * ceil_div(d.n, bn) * batch;
    const int64_t num_kb = ceil_div(d.k, BK);
    int64_t s = 1;
    if (d.split_k > 1) s = d.split_k;
    else if (d.split_k == 0 && tiles * 4 <= sms && num_kb >= 8) s = sms / tiles;
    if (s > num_kb / 2) s = num_kb / 2;   // a range of fewer than two blocks is not worth a work item
    if (s < 1) s = 1;
    const int64_t per = ceil_div(num_kb, s);
    *kb_per_split = static_cast<int>(per < 1 ? 1 : per);
    *splits = static_cast<int>(num_kb > 0 ? ceil_div(num_kb, *kb_per_split) : 1);
}

int tile_width(const tb200_gemm_desc &d, int sms) {
    // 128 x 256 tiles halve the operand bytes per flop of 128 x 128 ones and measured faster on every
    // shape wide enough to hold one, even when they leave a few SMs idle -- except where the wide tiles fill
    // less than half the device (a replica's slice of a batch against a narrow layer): the narrow ones then
    // put twice the SMs to work in the same single wave
    if (d.tile_n == 256 || d.tile_n == 128) return d.tile_n;
    if (d.tile_n == 512) return 256;   // 256 x 256 tiles, one per pair of CTAs
    if (d.n <= 128) return 128;
    const int64_t batch = d.batch > 1 ? d.batch : 1;
    const int64_t wide = ceil_div(d.m, BM) * ceil_div(d.n, 256) * batch;
    return 2 * wide <= sms ? 128 : 256;
}

// Pairs of CTAs on 256 x 256 tiles: asked for (tile_n 512), or the library's choice where there is at least one such
// tile per pair of SMs -- a third less operand traffic per SM, which is what the single-CTA kernel is short of.
bool tile_pairs(const tb200_gemm_desc &d, int bn, int sms) {
    const int64_t batch = d.batch > 1 ? d.batch : 1;
    const int64_t pair_items = ceil_div(d.m, 2 * BM) * ceil_div(d.n, 256) * batch;
    return d.n > 128 && d.m > BM && (d.tile_n == 512 || (d.tile_n == 0 && bn == 256 && d.split_k <= 1 && 2 * pair_items >= sms));
}

size_t split_workspace_bytes(const tb200_gemm_desc &d, int splits) {
    const int64_t batch = d.batch > 1 ? d.batch : 1;
    const int64_t ld = (d.n + 3) / 4 * 4;
    return static_cast<size_t>(splits) * batch * d.m * ld * sizeof(float);
}

}  // namespace
}  // namespace tb200

using namespace tb200;

// Everything a product's launch needs, worked out once.
struct tb200_gemm_plan {
    tb200_gemm_desc desc;
    const void *a, *b, *bias, *aux;
    void *c, *aux_out;
    int device;
    bool nothing;        // an empty product
    bool tensor;         // the tcgen05 kernel (else the generic one)
    GemmArgs args;
    const void *kernel;
    unsigned grid;
    size_t smem;
    bool merge;          // split-K: a second launch
    MergeArgs merge_args;
    unsigned merge_grid;
    SimtArgs simt;
    dim3 simt_grid;
    bool pair;           // launched as clusters of two CTAs sharing 256 x 256 tiles
    int *counters;       // device memory of a created plan (two ints, zero between launches), else null
};

namespace {

int validate(const tb200_gemm_desc *d, const void *a, const void *b, void *c, const void *bias, const void *aux,
             void *aux_out) {
    if (!d) return TB200_ERR_NULL;
    if (d->m < 0 || d->n < 0 || d->k < 0 || d->m > INT32_MAX || d->n > INT32_MAX || d->k > INT32_MAX)
        return TB200_ERR_SHAPE;
    const auto known = [](int t) { return t == TB200_F32 || t == TB200_BF16 || t == TB200_F16; };
    if (!known(d->in_dtype) || !known(d->out_dtype)) return TB200_ERR_DTYPE;
    // a 16-bit result has the operands' type, or the operands are Float32
    if (d->out_dtype != TB200_F32 && d->in_dtype != TB200_F32 && d->out_dtype != d->in_dtype) return TB200_ERR_DTYPE;
    if (d->epilogue < TB200_EPI_NONE || d->epilogue > TB200_EPI_AXPY) return TB200_ERR_UNSUPPORTED;
    if (d->batch < 0 || d->batch > (1 << 24) || d->split_k < 0) return TB200_ERR_SHAPE;
    if (d->m == 0 || d->n == 0) return TB200_OK;
    const int64_t a_inner = d->a_layout == TB200_MN_MAJOR ? d->m : d->k;
    const int64_t b_inner = d->b_layout == TB200_MN_MAJOR ? d->n : d->k;
    if (d->lda < a_inner || d->ldb < b_inner || d->ldc < d->n) return TB200_ERR_SHAPE;
    if (d->batch > 1) {
        if (d->stride_a < 0 || d->stride_b < 0 || d->stride_bias < 0 || d->stride_aux < 0) return TB200_ERR_SHAPE;
        // members must not write over one another
        if (d->stride_c < (d->m - 1) * d->ldc + d->n) return TB200_ERR_SHAPE;
        if (aux_out && d->stride_aux_out < (d->m - 1) * d->ld_aux_out + d->n) return TB200_ERR_SHAPE;
    }
    if (!c || (d->k > 0 && (!a || !b))) return TB200_ERR_NULL;
    if ((epilogue_reads_bias(d->epilogue) && !bias) || (epilogue_reads_aux(d->epilogue) && !aux)) return TB200_ERR_NULL;
    if (epilogue_reads_aux(d->epilogue) && d->ld_aux < d->n) return TB200_ERR_SHAPE;
    if (aux_out && d->ld_aux_out < d->n) return TB200_ERR_SHAPE;
    const size_t in_size = dtype_size(d->in_dtype), out_size = dtype_size(d->out_dtype);
    if (!aligned_to(a, in_size) || !aligned_to(b, in_size) || !aligned_to(c, out_size) ||
        !aligned_to(bias, in_size) || !aligned_to(aux, 2) || !aligned_to(aux_out, in_size))
        return TB200_ERR_ALIGN;
    return TB200_OK;
}

// Fills `plan` for the current device from its desc and operand addresses.
int prepare(tb200_gemm_plan *plan) {
    const tb200_gemm_desc *d = &plan->desc;
    const void *a = plan->a, *b = plan->b, *bias = plan->bias, *aux = plan->aux;
    void *c = plan->c, *aux_out = plan->aux_out;
    int st = validate(d, a, b, c, bias, aux, aux_out);
    if (st) return st;
    plan->nothing = d->m == 0 || d->n == 0 || d->batch < 0;
    if (plan->nothing) return TB200_OK;
    DeviceInfo dev;
    if ((st = current_device(&dev))) return st;
    plan->device = dev.device;
    const int batch = static_cast<int>(d->batch > 1 ? d->batch : 1);
    const bool batched = batch > 1;
    const bool needs_aux = epilogue_reads_aux(d->epilogue);
    const size_t in_size = dtype_size(d->in_dtype), out_size = dtype_size(d->out_dtype);
    const bool half_in = d->in_dtype == TB200_BF16 || d->in_dtype == TB200_F16;
    // Float16 results of the activation epilogues and Float32 results of any activation: generic kernel
    const bool instantiated = !(is_activation(d->epilogue) && (d->out_dtype != TB200_BF16 || d->in_dtype != TB200_BF16));
    const bool strides_ok = !batched || ((d->stride_a * in_size) % 16 == 0 && (d->stride_b * in_size) % 16 == 0);
    const bool tma_ok = half_in && d->k > 0 && aligned_to(a, 16) && aligned_to(b, 16) && d->lda % 8 == 0 &&
                        d->ldb % 8 == 0 && !d->force_simt && instantiated && strides_ok;
    plan->tensor = tma_ok;
    plan->merge = false;
    if (tma_ok) {
        GemmArgs &p = plan->args;
        p = GemmArgs{};
        const int bn = tile_width(*d, dev.sms);
        const bool pair = tile_pairs(*d, bn, dev.sms);
        plan->pair = pair;
        int splits = 1, kb_per = static_cast<int>(ceil_div(d->k, BK));
        if (!pair) choose_split(*d, bn, dev.sms, &splits, &kb_per);
        if (splits > 1 && (!d->workspace || !aligned_to(d->workspace, 16) ||
                           d->workspace_bytes < split_workspace_bytes(*d, splits))) {
            splits = 1;
            kb_per = static_cast<int>(ceil_div(d->k, BK));
        }
        p.m = static_cast<int>(d->m); p.n = static_cast<int>(d->n); p.k = static_cast<int>(d->k);
        p.in_f16 = d->in_dtype == TB200_F16;
        p.a_mn = d->a_layout == TB200_MN_MAJOR; p.b_mn = d->b_layout == TB200_MN_MAJOR;
        p.a_batched = batched && d->stride_a != 0; p.b_batched = batched && d->stride_b != 0;
        p.batch = batch; p.splits = splits; p.kb_per_split = kb_per;
        p.debug = d->debug;
        p.wait_ns = d->debug ? 20000000ull : 2000000000ull;
        p.tiles_m = static_cast<int>(ceil_div(d->m, pair ? 2 * BM : BM));
        p.tiles_n = static_cast<int>(ceil_div(d->n, bn));
        const int64_t am = p.a_batched ? batch : 1, bm = p.b_batched ? batch : 1;
        if (p.a_mn) st = make_tmap(&p.tmap_a, a, d->m, d->k, d->lda, 64, d->in_dtype, am, d->stride_a);
        else st = make_tmap(&p.tmap_a, a, d->k, d->m, d->lda, BM, d->in_dtype, am, d->stride_a);
        if (st) return st;
        if (p.b_mn) st = make_tmap(&p.tmap_b, b, d->n, d->k, d->ldb, 64, d->in_dtype, bm, d->stride_b);
        else st = make_tmap(&p.tmap_b, b, d->k, d->n, d->ldb, pair ? bn / 2 : bn, d->in_dtype, bm, d->stride_b);
        if (st) return st;
        int kernel_epilogue = d->epilogue, kernel_out = d->out_dtype;
        if (splits > 1) {
            // the ranges' partial tiles go to the workspace as they are; the merge applies alpha and the epilogue
            const int64_t ldp = (d->n + 3) / 4 * 4;
            p.c = d->workspace; p.ldc = ldp; p.stride_c = d->m * ldp;
            p.alpha = 1.0f; p.epilogue = TB200_EPI_NONE;
            kernel_epilogue = TB200_EPI_NONE; kernel_out = TB200_F32;
            p.staged_epilogue = !d->direct_epilogue && aligned_to(d->workspace, 16);
            MergeArgs &q = plan->merge_args;
            q = MergeArgs{};
            q.partial = static_cast<const float *>(d->workspace); q.c = c; q.bias = bias; q.aux = aux; q.aux_out = aux_out;
            q.ld_partial = ldp; q.ldc = d->ldc; q.ld_aux = d->ld_aux; q.ld_aux_out = d->ld_aux_out;
            q.stride_c = d->stride_c; q.stride_bias = d->stride_bias; q.stride_aux = d->stride_aux;
            q.stride_aux_out = d->stride_aux_out;
            q.alpha = d->alpha; q.m = p.m; q.n = p.n; q.batch = batch; q.splits = splits; q.epilogue = d->epilogue;
            q.in_dtype = d->in_dtype; q.out_dtype = d->out_dtype;
            const long long blocks = ceil_div(static_cast<int64_t>(batch) * d->m * d->n, 256);
            plan->merge_grid = static_cast<unsigned>(blocks < dev.sms * 8 ? blocks : dev.sms * 8);
            plan->merge = true;
        } else {
            p.c = c; p.bias = bias; p.aux = aux; p.aux_out = aux_out;
            p.ldc = d->ldc; p.ld_aux = d->ld_aux; p.ld_aux_out = d->ld_aux_out;
            p.stride_c = batched ? d->stride_c : 0; p.stride_bias = batched ? d->stride_bias : 0;
            p.stride_aux = batched ? d->stride_aux : 0; p.stride_aux_out = batched ? d->stride_aux_out : 0;
            p.alpha = d->alpha; p.epilogue = d->epilogue;
            // the epilogue goes through the staging buffers (whole 128-byte lines out, the operand it reads in by TMA)
            // when every array it touches allows 16-byte accesses; otherwise each thread stores its own row
            const size_t aux_size = (d->epilogue == TB200_EPI_AXPY) ? out_size : 2;
            const int aux_dtype = d->epilogue == TB200_EPI_AXPY ? d->out_dtype : d->in_dtype;
            const auto pitch_ok = [&](int64_t stride, size_t es) { return !batched || (stride * es) % 16 == 0; };
            bool staged = !d->direct_epilogue && aligned_to(c, 16) && (d->ldc * out_size) % 16 == 0 &&
                           pitch_ok(d->stride_c, out_size);
            if (needs_aux)
                staged = staged && aux_size == out_size && aligned_to(aux, 16) && (d->ld_aux * aux_size) % 16 == 0 &&
                          pitch_ok(d->stride_aux, aux_size);
            if (aux_out)
                staged = staged && d->out_dtype != TB200_F32 && aligned_to(aux_out, 16) && (d->ld_aux_out * 2) % 16 == 0 &&
                          pitch_ok(d->stride_aux_out, 2);
            if (staged) {
                if (needs_aux && (st = make_tmap(&p.tmap_aux, aux, d->n, d->m, d->ld_aux, 32, aux_dtype,
                                                 d->stride_aux ? batch : 1, d->stride_aux)))
                    return st;
                if (needs_aux && batched && d->stride_aux == 0) staged = false;   // a shared aux: plain loads
            }
            p.staged_epilogue = staged;
        }
        if ((st = kernel_by_shape(bn, pair, kernel_out, kernel_epilogue, dev, &plan->kernel))) return st;
        const size_t stage_bytes = static_cast<size_t>(BM + (pair ? bn / 2 : bn)) * BK * 2;
        const size_t epilogue_bytes = kEpilogueWarps * kEpilogueStage;
        int stages = static_cast<int>((dev.smem_optin - 2048 - epilogue_bytes) / stage_bytes);
        if (stages > 8) stages = 8;
        if (stages < 2) return TB200_ERR_UNSUPPORTED;
        p.stages = stages;
        plan->smem = stages * stage_bytes + epilogue_bytes + 1024;
        const long long items = static_cast<long long>(p.tiles_m) * p.tiles_n * batch * splits;
        if (items > INT32_MAX) return TB200_ERR_SHAPE;
        plan->grid = static_cast<unsigned>(items < dev.sms ? items : dev.sms);
        // more items than blocks: a created plan lets its blocks draw them from a counter
        p.schedule = (plan->counters && items > plan->grid) ? plan->counters : nullptr;
        if (pair) {   // two CTAs per item
            const long long held = resident_pairs(plan->kernel, plan->smem, dev);
            const long long pairs = items < held ? items : held;
            plan->grid = static_cast<unsigned>(2 * pairs);
            p.schedule = (plan->counters && items > pairs) ? plan->counters : nullptr;
        }
        return TB200_OK;
    }

    SimtArgs &p = plan->simt;
    p = SimtArgs{};
    p.a = a; p.b = b; p.c = c; p.bias = bias; p.aux = aux; p.aux_out = aux_out;
    p.lda = d->lda; p.ldb = d->ldb; p.ldc = d->ldc; p.ld_aux = d->ld_aux; p.ld_aux_out = d->ld_aux_out;
    if (batched) {
        p.stride_a = d->stride_a; p.stride_b = d->stride_b; p.stride_c = d->stride_c; p.stride_bias = d->stride_bias;
        p.stride_aux = d->stride_aux; p.stride_aux_out = d->stride_aux_out;
    }
    p.alpha = d->alpha; p.m = static_cast<int>(d->m); p.n = static_cast<int>(d->n); p.k = static_cast<int>(d->k);
    p.batch = batch;
    p.epilogue = d->epilogue; p.in_dtype = d->in_dtype; p.out_dtype = d->out_dtype;
    p.a_mn = d->a_layout == TB200_MN_MAJOR; p.b_mn = d->b_layout == TB200_MN_MAJOR;
    plan->simt_grid = dim3(static_cast<unsigned>(ceil_div(d->n, 64)), static_cast<unsigned>(ceil_div(d->m, 64)),
                           static_cast<unsigned>(batch < 65535 ? batch : 65535));
    if (plan->simt_grid.y > 65535) return TB200_ERR_SHAPE;
    return TB200_OK;
}

int run(const tb200_gemm_plan *plan, cudaStream_t stream) {
    if (plan->nothing) return TB200_OK;
    if (!plan->tensor) {
        gemm_simt<<<plan->simt_grid, 256, 0, stream>>>(plan->simt);
        TB200_CUDA(cudaGetLastError());
        return TB200_OK;
    }
    void *params[1] = {const_cast<GemmArgs *>(&plan->args)};
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(plan->grid);
    config.blockDim = dim3(kGemmThreads);
    config.dynamicSmemBytes = plan->smem;
    config.stream = stream;
    cudaLaunchAttribute attrs[2] = {};
    // the kernel's prologue may run under the tail of the kernel before it (it waits before touching global memory)
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    attrs[1].id = cudaLaunchAttributeClusterDimension;
    attrs[1].val.clusterDim.x = 2; attrs[1].val.clusterDim.y = 1; attrs[1].val.clusterDim.z = 1;
    config.attrs = attrs;
    config.numAttrs = plan->pair ? 2 : 1;
    TB200_CUDA(cudaLaunchKernelExC(&config, plan->kernel, params));
    if (plan->merge) {
        gemm_splitk_merge<<<plan->merge_grid, 256, 0, stream>>>(plan->merge_args);
        TB200_CUDA(cudaGetLastError());
    }
    return TB200_OK;
}

void fill(tb200_gemm_plan *plan, const tb200_gemm_desc *d, const void *a, const void *b, void *c, const void *bias,
          const void *aux, void *aux_out) {
    plan->desc = *d;
    plan->counters = nullptr;
    plan->pair = false;
    plan->a = a; plan->b = b; plan->c = c; plan->bias = bias; plan->aux = aux; plan->aux_out = aux_out;
}

}  // namespace

extern "C" size_t tb200_gemm_workspace_bytes(const tb200_gemm_desc *d) {
    if (!d || d->m <= 0 || d->n <= 0 || d->k <= 0 || d->split_k == 1) return 0;
    DeviceInfo dev;
    int sms = 148;
    if (current_device(&dev) == TB200_OK) sms = dev.sms;
    int splits = 1, per = 1;
    choose_split(*d, tile_width(*d, sms), sms, &splits, &per);
    return splits > 1 ? split_workspace_bytes(*d, splits) : 0;
}

// The tile form the tensor-core path takes for a descriptor: 128 or 256 (columns of a single CTA's 128-row tile) or
// 512 (256 x 256 tiles by pairs of CTAs); 0 for an empty product.  Host arithmetic only (148 SMs assumed where no
// device answers), for cost statements and tests: the layouts, alignments and types that send a product to the
// CUDA-core kernel instead are not looked at.
extern "C" int tb200_gemm_tile_form(const tb200_gemm_desc *d) {
    if (!d || d->m <= 0 || d->n <= 0 || d->k <= 0) return 0;
    DeviceInfo dev;
    int sms = 148;
    if (current_device(&dev) == TB200_OK) sms = dev.sms;
    const int bn = tile_width(*d, sms);
    return tile_pairs(*d, bn, sms) ? 512 : bn;
}

extern "C" int tb200_gemm(const tb200_gemm_desc *d, const void *a, const void *b, void *c, const void *bias,
                          const void *aux, void *aux_out, void *stream_) {
    if (!d) return TB200_ERR_NULL;
    tb200_gemm_plan plan;
    fill(&plan, d, a, b, c, bias, aux, aux_out);
    const int st = prepare(&plan);
    return st ? st : run(&plan, static_cast<cudaStream_t>(stream_));
}

extern "C" int tb200_gemm_plan_create(const tb200_gemm_desc *d, const void *a, const void *b, void *c, const void *bias,
                                      const void *aux, void *aux_out, tb200_gemm_plan **out) {
    if (!d || !out) return TB200_ERR_NULL;
    *out = nullptr;
    tb200_gemm_plan *plan = new (std::nothrow) tb200_gemm_plan;
    if (!plan) return TB200_ERR_WORKSPACE;
    fill(plan, d, a, b, c, bias, aux, aux_out);
    // building may allocate (launching may not): the two counters of the dynamic schedule
    if (cudaMalloc(&plan->counters, 2 * sizeof(int)) != cudaSuccess || cudaMemset(plan->counters, 0, 2 * sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        if (plan->counters) cudaFree(plan->counters);
        plan->counters = nullptr;     // without them the plan deals its items round-robin, as tb200_gemm does
    }
    const int st = prepare(plan);
    if (st) {
        if (plan->counters) cudaFree(plan->counters);
        delete plan;
        return st;
    }
    *out = plan;
    return TB200_OK;
}

extern "C" int tb200_gemm_plan_launch(const tb200_gemm_plan *plan, void *stream_) {
    if (!plan) return TB200_ERR_NULL;
    return run(plan, static_cast<cudaStream_t>(stream_));
}

extern "C" int tb200_gemm_plan_repoint(tb200_gemm_plan *plan, int operand, const void *address) {
    if (!plan) return TB200_ERR_NULL;
    tb200_gemm_plan next = *plan;
    switch (operand) {
        case TB200_GEMM_A: next.a = address; break;
        case TB200_GEMM_B: next.b = address; break;
        case TB200_GEMM_C: next.c = const_cast<void *>(address); break;
        case TB200_GEMM_BIAS: next.bias = address; break;
        case TB200_GEMM_AUX: next.aux = address; break;
        case TB200_GEMM_AUX_OUT: next.aux_out = const_cast<void *>(address); break;
        case TB200_GEMM_WORKSPACE: next.desc.workspace = const_cast<void *>(address); break;
        default: return TB200_ERR_SHAPE;
    }
    const int st = prepare(&next);
    if (st) return st;          // the plan stays as it was
    // a new address must leave the plan on the kernels it was built for (the reference requires the
    // alignment compiled for, src/Compiler/Implement/Implement.jl:162-175)
    if (next.tensor != plan->tensor || (next.tensor && (next.kernel != plan->kernel ||
                                                         next.args.staged_epilogue != plan->args.staged_epilogue)))
        return TB200_ERR_ALIGN;
    *plan = next;
    return TB200_OK;
}

extern "C" void tb200_gemm_plan_destroy(tb200_gemm_plan *plan) {
    if (!plan) return;
    if (plan->counters) cudaFree(plan->counters);   // waits for launches still in flight
    delete plan;
}

// Synchronises the device and returns (then clears) the error code a tensor-core kernel recorded when one
// of its bounded waits ran out: 0 none, 1 loader, 2 accumulator hand-back, 3 operands, 4 epilogue, 5 the
// epilogue's own operand.
extern "C" int tb200_device_error(void) {
    int code = 0, zero = 0;
    TB200_CUDA(cudaDeviceSynchronize());
    TB200_CUDA(cudaMemcpyFromSymbol(&code, g_gemm_error, sizeof(int)));
    if (code) TB200_CUDA(cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int)));
    return code;
}

namespace {
// Device time of `reps` launches of the product after one warm-up launch; negative status on failure.
int time_variant(const tb200_gemm_desc &trial, const void *a, const void *b, void *c, const void *bias, const void *aux,
                 void *aux_out, cudaStream_t stream, cudaEvent_t t0, cudaEvent_t t1, int reps, float *ms) {
    int status = tb200_gemm(&trial, a, b, c, bias, aux, aux_out, stream);   // warm-up and validation
    if (status) return status;
    if (cudaEventRecord(t0, stream) != cudaSuccess) return TB200_ERR_CUDA;
    for (int rep = 0; rep < reps && !status; rep++) status = tb200_gemm(&trial, a, b, c, bias, aux, aux_out, stream);
    if (status) return status;
    if (cudaEventRecord(t1, stream) != cudaSuccess || cudaEventSynchronize(t1) != cudaSuccess ||
        cudaEventElapsedTime(ms, t0, t1) != cudaSuccess)
        return TB200_ERR_CUDA;
    return TB200_OK;
}
}  // namespace

// Times the compiled-in tile variants of one product on its own operands and returns the faster one's
// tile_n (128, 256, or 512 for 256 x 256 tiles by pairs of CTAs) -- the measured stage of the reference's search over a claim's `variants`
// (src/Compiler/Implement/Implement.jl:120, ext/cuTileExt/contract.jl:171-235), restricted to what this
// library holds.  Runs the product several times (C and aux_out are overwritten with the product's own
// result), synchronises the stream: a build-time call, not one for a capture.  Where there is nothing to
// choose (narrow outputs, the CUDA-core path, the accumulating epilogue whose repeats would add up) it returns
// the width tb200_gemm would take without measuring.
extern "C" int tb200_gemm_tune(const tb200_gemm_desc *d, const void *a, const void *b, void *c, const void *bias, const void *aux,
                               void *aux_out, void *stream_) {
    if (!d) return TB200_ERR_NULL;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int fallback = d->n > 128 ? 256 : 128;
    const bool measurable = (d->in_dtype == TB200_BF16 || d->in_dtype == TB200_F16) && d->n > 128 && d->m > 0 &&
                            d->k > 0 && !d->force_simt && d->epilogue != TB200_EPI_AXPY;
    tb200_gemm_desc trial = *d;
    if (!measurable) {
        trial.tile_n = 0;
        const int st = tb200_gemm(&trial, a, b, c, bias, aux, aux_out, stream_);   // still validates the request
        return st ? st : fallback;
    }
    cudaEvent_t t0, t1;
    TB200_CUDA(cudaEventCreate(&t0));
    TB200_CUDA(cudaEventCreate(&t1));
    float best_ms = 0.0f;
    int best = fallback, status = TB200_OK;
    for (int width : {128, 256, 512}) {
        if (width == 512 && d->m <= BM) continue;
        trial.tile_n = width;
        float ms = 0.0f;
        if ((status = time_variant(trial, a, b, c, bias, aux, aux_out, stream, t0, t1, 3, &ms))) break;
        if (width == 128 || ms < best_ms) { best_ms = ms; best = width; }
    }
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    return status ? status : best;
}

// The search over every compiled-in variant: tile width x split or not x how the result is stored.
extern "C" int tb200_gemm_tune_desc(tb200_gemm_desc *d, const void *a, const void *b, void *c, const void *bias,
                                    const void *aux, void *aux_out, void *stream_) {
    if (!d) return TB200_ERR_NULL;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    tb200_gemm_desc trial = *d;
    trial.tile_n = 0; trial.split_k = 0; trial.direct_epilogue = 0;
    int status = tb200_gemm(&trial, a, b, c, bias, aux, aux_out, stream_);
    if (status) return status;
    const bool measurable = (d->in_dtype == TB200_BF16 || d->in_dtype == TB200_F16) && d->m > 0 && d->k > 0 &&
                            !d->force_simt && d->epilogue != TB200_EPI_AXPY;
    if (!measurable) { d->tile_n = 0; d->split_k = 0; d->direct_epilogue = 0; return TB200_OK; }
    cudaEvent_t t0, t1;
    TB200_CUDA(cudaEventCreate(&t0));
    TB200_CUDA(cudaEventCreate(&t1));
    float best_ms = -1.0f;
    tb200_gemm_desc best = trial;
    for (int width : {128, 256, 512}) {
        if (width >= 256 && d->n <= 128) continue;
        if (width == 512 && d->m <= BM) continue;
        for (int split : {1, 0}) {
            if (width == 512 && split == 0) continue;   // pairs do not split the sum
            trial.tile_n = width; trial.split_k = split;
            if (split == 0 && tb200_gemm_workspace_bytes(&trial) == 0) continue;           // would not split
            if (split == 0 && (!d->workspace || d->workspace_bytes < tb200_gemm_workspace_bytes(&trial))) continue;
            for (int direct : {0, 1}) {
                trial.direct_epilogue = direct;
                float ms = 0.0f;
                if ((status = time_variant(trial, a, b, c, bias, aux, aux_out, stream, t0, t1, 3, &ms))) break;
                if (best_ms < 0.0f || ms < best_ms) { best_ms = ms; best = trial; }
            }
            if (status) break;
        }
        if (status) break;
    }
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    if (status) return status;
    d->tile_n = best.tile_n; d->split_k = best.split_k; d->direct_epilogue = best.direct_epilogue;
    return TB200_OK;
}
