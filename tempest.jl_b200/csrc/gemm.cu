// GEMM with fused epilogues for sm_100a.
//
// Fast path (BFloat16 in, Float32 accumulate): a persistent, warp-specialised
// kernel, one CTA per SM.  One thread issues TMA tile loads into a ring of
// 128-byte-swizzled shared-memory stages; one thread issues tcgen05.mma
// (128 x BN x 16 per instruction) accumulating in tensor memory; four warps
// drain finished accumulators with tcgen05.ld, apply the epilogue in
// registers and store.  Tensor memory holds two accumulator tiles, so the
// epilogue of tile i overlaps the main loop of tile i + 1.  Either operand may
// be K-major or MN-major in memory (all of NN / NT / TN / TT), which is what
// lets the backward products dX = dY * W' and dW = X' * dY read the forward's
// arrays in place.  No load uses cluster multicast.
//
// Generic path: a shared-memory tiled SIMT kernel for Float32 operands, odd
// leading dimensions and anything else the TMA path cannot address.
//
// Every wait on an mbarrier is bounded: after about two seconds the kernel
// records an error code, stops issuing work and drains, so a pipeline bug ends
// as a status, not as a hung device.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "sm100.cuh"

namespace tb200 {
namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;          // 64 BFloat16 = one 128-byte swizzle line
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 192;   // warp 0 loads, warp 1 issues MMAs, warps 2-5 run the epilogue
constexpr int kAccumStages = 2;

__device__ int g_gemm_error = 0;

struct GemmArgs {
    CUtensorMap tmap_a;
    CUtensorMap tmap_b;
    CUtensorMap tmap_c;        // output tiles of 32 rows x 128 bytes (TMA epilogue only)
    CUtensorMap tmap_aux;
    CUtensorMap tmap_aux_out;
    int tma_epilogue;
    void *c;
    const void *bias;
    const void *aux;
    void *aux_out;
    long long ldc, ld_aux, ld_aux_out;
    float alpha;
    int m, n, k;
    int epilogue;
    int out_f32;
    int a_mn, b_mn;       // operand is MN-major in memory
    int tiles_m, tiles_n;
    int stages;
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

// `count` (<= 32) consecutive values of one output row, as Float32 or rounded to BFloat16; 128-bit
// stores when the whole chunk is there and the address allows.
__device__ __forceinline__ void store_row32(void *base, int f32, long long offset, const float (&v)[32], int count) {
    if (f32) {
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
        __nv_bfloat16 *o = static_cast<__nv_bfloat16 *>(base) + offset;
        if (count == 32 && aligned_dev(o, 16)) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint4 q;
                q.x = pack_bf16x2(v[8 * j], v[8 * j + 1]);
                q.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
                q.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
                q.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
                reinterpret_cast<uint4 *>(o)[j] = q;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (j < count) o[j] = __float2bfloat16_rn(v[j]);
        }
    }
}

// ------------------------------------------------------- tcgen05 kernel ----

__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait: false once `*failed` is set by anyone or two seconds have passed.
__device__ __forceinline__ bool wait_or_fail(uint64_t *bar, uint32_t parity, volatile int *failed, int code) {
    if (mbar_wait(bar, parity, 4096)) return true;
    const uint64_t t0 = global_ns();
    while (true) {
        if (mbar_wait(bar, parity, 1024)) return true;
        if (*failed) return false;
        if (global_ns() - t0 > 2000000000ull) {
            *failed = code;
            atomicCAS(&g_gemm_error, 0, code);
            return false;
        }
    }
}

constexpr int kStageLine = 128;                   // bytes per staged row: one 128-byte swizzle line
constexpr int kEpilogueStage = 32 * kStageLine;   // 32 rows of one warp

// One warp's share of a finished accumulator tile, through shared memory: 32 rows x 128 bytes at a
// time are written (128-byte swizzled, so a thread writing its own row does not collide with its
// neighbours) into a staging buffer and handed to a TMA store, which writes whole lines; the operand an
// epilogue reads (aux) arrives the same way by a TMA load.  Returns false if a bounded wait gave up.
template <int BN, int EPI, bool OUT_F32>
__device__ __forceinline__ bool epilogue_tile_tma(const GemmArgs &p, uint32_t tmem_acc, int row0, int n0, int lane,
                                                  uint8_t *stage_c, uint8_t *stage_x, uint64_t *aux_bar,
                                                  uint32_t &aux_phase, volatile int *failed) {
    constexpr int EPL = OUT_F32 ? 32 : 64;   // elements per 128-byte line
    constexpr bool reads_bias = epilogue_reads_bias(EPI), reads_aux = epilogue_reads_aux(EPI);
    const bool has_aux_out = EPI == TB200_EPI_BIAS_GELU && p.aux_out != nullptr;
    const int sw = lane & 7;
#pragma unroll 1
    for (int g = 0; g < BN / EPL; g++) {
        const int col0 = n0 + g * EPL;
        if (col0 >= p.n) break;
        // one staging buffer per warp: the previous group's stores must have read it
        if (lane == 0) bulk_wait_group_read<0>();
        __syncwarp();
        if (reads_aux) {
            if (lane == 0) {
                mbar_arrive_expect_tx(aux_bar, kEpilogueStage);
                tma_load_2d(stage_x, &p.tmap_aux, aux_bar, col0, row0);
            }
            if (!wait_or_fail(aux_bar, aux_phase, failed, 5)) return false;
            aux_phase ^= 1;
        }
#pragma unroll 1
        for (int h = 0; h < EPL / 32; h++) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_acc + g * EPL + h * 32, r);
            tmem_ld_wait();
            const int c0 = col0 + h * 32;
            float v[32], auxv[32];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]) * p.alpha;
            if (reads_aux) {
                if constexpr (OUT_F32) {
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const float4 q = *reinterpret_cast<const float4 *>(stage_x + lane * kStageLine + ((j ^ sw) << 4));
                        auxv[4 * j] = q.x; auxv[4 * j + 1] = q.y; auxv[4 * j + 2] = q.z; auxv[4 * j + 3] = q.w;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const uint4 q =
                            *reinterpret_cast<const uint4 *>(stage_x + lane * kStageLine + (((4 * h + j) ^ sw) << 4));
                        Access<__nv_bfloat16, true>::unpack(q, &auxv[8 * j]);
                    }
                }
            }
            float bv[32];
            if (reads_bias) {
                const __nv_bfloat16 *bp = static_cast<const __nv_bfloat16 *>(p.bias) + c0;
                if (c0 + 32 <= p.n && aligned_dev(bp, 16)) {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        Access<__nv_bfloat16, true>::unpack(__ldg(reinterpret_cast<const uint4 *>(bp) + j), &bv[8 * j]);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) bv[j] = (c0 + j < p.n) ? __bfloat162float(bp[j]) : 0.0f;
                }
            }
            float pre[32];
#pragma unroll
            for (int j = 0; j < 32; j++) {
                pre[j] = v[j];
                v[j] = epilogue_fixed<EPI>(v[j], reads_bias ? bv[j] : 0.0f, reads_aux ? auxv[j] : 0.0f, pre[j]);
            }
            if constexpr (OUT_F32) {
#pragma unroll
                for (int j = 0; j < 8; j++)
                    *reinterpret_cast<float4 *>(stage_c + lane * kStageLine + ((j ^ sw) << 4)) =
                        make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint4 q;
                    q.x = pack_bf16x2(v[8 * j], v[8 * j + 1]);
                    q.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
                    q.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
                    q.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
                    *reinterpret_cast<uint4 *>(stage_c + lane * kStageLine + (((4 * h + j) ^ sw) << 4)) = q;
                    if (has_aux_out) {
                        q.x = pack_bf16x2(pre[8 * j], pre[8 * j + 1]);
                        q.y = pack_bf16x2(pre[8 * j + 2], pre[8 * j + 3]);
                        q.z = pack_bf16x2(pre[8 * j + 4], pre[8 * j + 5]);
                        q.w = pack_bf16x2(pre[8 * j + 6], pre[8 * j + 7]);
                        *reinterpret_cast<uint4 *>(stage_x + lane * kStageLine + (((4 * h + j) ^ sw) << 4)) = q;
                    }
                }
            }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(&p.tmap_c, stage_c, col0, row0);
            if (has_aux_out) tma_store_2d(&p.tmap_aux_out, stage_x, col0, row0);
            bulk_commit_group();
        }
    }
    return true;
}

template <int BN, int EPI, bool OUT_F32>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_tcgen05(const __grid_constant__ GemmArgs p) {
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzle atoms are 1024 bytes: align the ring
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr uint32_t A_BYTES = BM * BK * 2;
    constexpr uint32_t B_BYTES = BN * BK * 2;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int MAX_STAGES = 8;

    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t tmem_full_bar[kAccumStages];
    __shared__ __align__(8) uint64_t tmem_empty_bar[kAccumStages];
    __shared__ __align__(8) uint64_t aux_bar[4];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int failed_smem;
    volatile int *failed = &failed_smem;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int stages = p.stages;
    const int num_kb = (p.k + BK - 1) / BK;
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        failed_smem = 0;
        for (int s = 0; s < stages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < kAccumStages; s++) {
            mbar_init(&tmem_full_bar[s], 1);
            mbar_init(&tmem_empty_bar[s], 4);
        }
        for (int s = 0; s < 4; s++) mbar_init(&aux_bar[s], 1);
        fence_barrier_init();
        prefetch_tensormap(&p.tmap_a);
        prefetch_tensormap(&p.tmap_b);
        if (p.tma_epilogue) prefetch_tensormap(&p.tmap_c);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_smem, kAccumStages * BN);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_smem;

    if (warp == 0) {
        // ---- TMA producer
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*failed; tile += gridDim.x) {
                const int m0 = (tile / p.tiles_n) * BM;
                const int n0 = (tile % p.tiles_n) * BN;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!wait_or_fail(&empty_bar[stage], phase ^ 1, failed, 1)) break;
                    uint8_t *sa = smem + stage * STAGE_BYTES;
                    uint8_t *sb = sa + A_BYTES;
                    mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
                    const int k0 = kb * BK;
                    if (p.a_mn) {   // [K][M]: slabs of 64 along M, each 64 K-lines of 128 bytes
                        for (int j = 0; j < BM / 64; j++)
                            tma_load_2d(sa + j * (BK * 128), &p.tmap_a, &full_bar[stage], m0 + j * 64, k0);
                    } else {        // [M][K]: 128 rows of 128 bytes
                        tma_load_2d(sa, &p.tmap_a, &full_bar[stage], k0, m0);
                    }
                    if (p.b_mn) {
                        for (int j = 0; j < BN / 64; j++)
                            tma_load_2d(sb + j * (BK * 128), &p.tmap_b, &full_bar[stage], n0 + j * 64, k0);
                    } else {
                        tma_load_2d(sb, &p.tmap_b, &full_bar[stage], k0, n0);
                    }
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (elect_one()) {
            const uint32_t idesc = umma_idesc_bf16(BM, BN, p.a_mn != 0, p.b_mn != 0);
            // K-major: 8-row groups 1024 bytes apart, 32 bytes per 16 K; MN-major: slabs BK*128 bytes
            // apart, 8-line groups 1024 bytes apart, 2048 bytes per 16 K
            const uint32_t a_lead = p.a_mn ? BK * 128 : 16, b_lead = p.b_mn ? BK * 128 : 16;
            const uint32_t a_step = (p.a_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4;
            const uint32_t b_step = (p.b_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4;
            int stage = 0, it = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*failed; tile += gridDim.x, it++) {
                const int acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!wait_or_fail(&tmem_empty_bar[acc], acc_phase ^ 1, failed, 2)) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!wait_or_fail(&full_bar[stage], phase, failed, 3)) break;
                    tcgen05_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    const uint64_t a_desc = umma_smem_desc(sa, a_lead, 1024);
                    const uint64_t b_desc = umma_smem_desc(sa + A_BYTES, b_lead, 1024);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)
                        tcgen05_mma_f16(d_tmem, a_desc + k * a_step, b_desc + k * b_step, idesc, (kb | k) != 0);
                    tcgen05_commit(&empty_bar[stage]);   // the stage is free once these MMAs have read it
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
                tcgen05_commit(&tmem_full_bar[acc]);     // the accumulator is complete
            }
        }
    } else {
        // ---- epilogue: warp q owns tensor-memory lanes [32 q, 32 q + 32)
        const int q = warp & 3;
        int it = 0;
        // staging for the TMA epilogue sits behind the operand ring: per warp one buffer for the
        // output and one for the operand the epilogue reads or the second array it writes
        uint8_t *stage_c = smem + stages * STAGE_BYTES + (warp - 2) * 2 * kEpilogueStage;
        uint8_t *stage_x = stage_c + kEpilogueStage;
        uint32_t aux_phase = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, it++) {
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            if (!wait_or_fail(&tmem_full_bar[acc], acc_phase, failed, 4)) break;
            tcgen05_fence_after();
            if (p.tma_epilogue) {
                const int row0 = (tile / p.tiles_n) * BM + q * 32;
                const uint32_t tmem_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
                bool ok = true;
                if (row0 < p.m)
                    ok = epilogue_tile_tma<BN, EPI, OUT_F32>(p, tmem_acc, row0, (tile % p.tiles_n) * BN, lane, stage_c,
                                                             stage_x, &aux_bar[warp - 2], aux_phase, failed);
                if (!ok) break;
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
                continue;
            }
            const int m = (tile / p.tiles_n) * BM + q * 32 + lane;
            const int n0 = (tile % p.tiles_n) * BN;
            const bool row_ok = m < p.m;
            constexpr bool reads_bias = epilogue_reads_bias(EPI), reads_aux = epilogue_reads_aux(EPI);
#pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
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
                    if (OUT_F32 && EPI == TB200_EPI_AXPY) {
                        const float *ap = static_cast<const float *>(p.aux) + static_cast<long long>(m) * p.ld_aux + col0;
#pragma unroll
                        for (int j = 0; j < 32; j++) auxv[j] = (whole || col0 + j < p.n) ? ap[j] : 0.0f;
                    } else {
                        const __nv_bfloat16 *ap =
                            static_cast<const __nv_bfloat16 *>(p.aux) + static_cast<long long>(m) * p.ld_aux + col0;
                        if (whole && aligned_dev(ap, 16)) {
#pragma unroll
                            for (int j = 0; j < 4; j++)
                                Access<__nv_bfloat16, true>::unpack(__ldg(reinterpret_cast<const uint4 *>(ap) + j), &auxv[j * 8]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                auxv[j] = (col0 + j < p.n) ? __bfloat162float(ap[j]) : 0.0f;
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    float b = 0.0f;
                    if (reads_bias && (whole || col0 + j < p.n))
                        b = __bfloat162float(static_cast<const __nv_bfloat16 *>(p.bias)[col0 + j]);
                    pre[j] = v[j];
                    v[j] = epilogue_fixed<EPI>(v[j], b, reads_aux ? auxv[j] : 0.0f, pre[j]);
                }
                store_row32(p.c, OUT_F32, static_cast<long long>(m) * p.ldc + col0, v, whole ? 32 : p.n - col0);
                if (p.aux_out)
                    store_row32(p.aux_out, 0, static_cast<long long>(m) * p.ld_aux_out + col0, pre,
                                whole ? 32 : p.n - col0);
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
        }
        // the staging buffers must outlive the stores that read them
        if (p.tma_epilogue && lane == 0) bulk_wait_group<0>();
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kAccumStages * BN);
    }
}

// --------------------------------------------------------- SIMT kernel ----
// C[M][N] = epilogue(alpha * A * B): 64 x 64 tile per block of 256 threads, 4 x 4 outputs per thread,
// operands through shared memory in Float32.  Any layout, any leading dimension, either element type.

struct SimtArgs {
    const void *a, *b;
    void *c;
    const void *bias, *aux;
    void *aux_out;
    long long lda, ldb, ldc, ld_aux, ld_aux_out;
    float alpha;
    int m, n, k;
    int epilogue;
    int in_f32, out_f32;
    int a_mn, b_mn;
};

__device__ __forceinline__ float load_elem(const void *p, long long i, int f32) {
    return f32 ? static_cast<const float *>(p)[i] : __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
}
__device__ __forceinline__ void store_elem(void *p, long long i, float v, int f32) {
    if (f32) static_cast<float *>(p)[i] = v;
    else static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
}

__global__ void __launch_bounds__(256) gemm_simt(const SimtArgs p) {
    __shared__ float sa[16][65];
    __shared__ float sb[16][65];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < p.k; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            // consecutive threads walk the operand's contiguous axis
            int mm, kk;
            if (p.a_mn) { mm = i & 63; kk = i >> 6; } else { kk = i & 15; mm = i >> 4; }
            const int gm = m0 + mm, gk = k0 + kk;
            float v = 0.0f;
            if (gm < p.m && gk < p.k)
                v = load_elem(p.a, p.a_mn ? static_cast<long long>(gk) * p.lda + gm : static_cast<long long>(gm) * p.lda + gk,
                              p.in_f32);
            sa[kk][mm] = v;
            int nn;
            if (p.b_mn) { nn = i & 63; kk = i >> 6; } else { kk = i & 15; nn = i >> 4; }
            const int gn = n0 + nn;
            const int gk2 = k0 + kk;
            v = 0.0f;
            if (gn < p.n && gk2 < p.k)
                v = load_elem(p.b, p.b_mn ? static_cast<long long>(gk2) * p.ldb + gn : static_cast<long long>(gn) * p.ldb + gk2,
                              p.in_f32);
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
    const bool reads_bias = epilogue_reads_bias(p.epilogue), reads_aux = epilogue_reads_aux(p.epilogue);
    const int aux_f32 = p.in_f32 || (p.out_f32 && p.epilogue == TB200_EPI_AXPY);
    for (int i = 0; i < 4; i++)
        for (int j = 0; j < 4; j++) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m >= p.m || n >= p.n) continue;
            const float b = reads_bias ? load_elem(p.bias, n, p.in_f32) : 0.0f;
            const float x = reads_aux ? load_elem(p.aux, static_cast<long long>(m) * p.ld_aux + n, aux_f32) : 0.0f;
            float pre = acc[i][j] * p.alpha;
            const float v = epilogue_value<true>(p.epilogue, pre, b, x, pre);
            store_elem(p.c, static_cast<long long>(m) * p.ldc + n, v, p.out_f32);
            if (p.aux_out) store_elem(p.aux_out, static_cast<long long>(m) * p.ld_aux_out + n, pre, p.in_f32);
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

// A 2-D array `rows` x `cols` (cols contiguous, row pitch ld elements) as 128-byte-swizzled boxes of
// box_rows rows x 128 bytes (64 BFloat16 or 32 Float32).
int make_tmap(CUtensorMap *map, const void *base, int64_t cols, int64_t rows, int64_t ld, int box_rows,
              bool f32 = false) {
    EncodeTiledFn fn;
    int st = encode_fn(&fn);
    if (st) return st;
    const cuuint64_t es = f32 ? 4 : 2;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * es};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / es), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TB200_OK : TB200_ERR_UNSUPPORTED;
}

template <int BN, int EPI, bool OUT_F32>
int launch_tcgen05(GemmArgs &p, const DeviceInfo &dev, cudaStream_t stream) {
    constexpr size_t stage_bytes = (BM + BN) * BK * 2;
    constexpr size_t epilogue_bytes = 4 * 2 * kEpilogueStage;
    int stages = static_cast<int>((dev.smem_optin - 2048 - epilogue_bytes) / stage_bytes);
    if (stages > 8) stages = 8;
    if (stages < 2) return TB200_ERR_UNSUPPORTED;
    p.stages = stages;
    p.tiles_m = static_cast<int>(ceil_div(p.m, BM));
    p.tiles_n = static_cast<int>(ceil_div(p.n, BN));
    const size_t smem = stages * stage_bytes + epilogue_bytes + 1024;
    static std::mutex lock;
    static bool configured[64] = {};
    {
        std::lock_guard<std::mutex> hold(lock);
        if (!configured[dev.device]) {
            TB200_CUDA(cudaFuncSetAttribute(gemm_tcgen05<BN, EPI, OUT_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(dev.smem_optin - 1024)));
            configured[dev.device] = true;
        }
    }
    const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
    const unsigned grid = static_cast<unsigned>(tiles < dev.sms ? tiles : dev.sms);
    gemm_tcgen05<BN, EPI, OUT_F32><<<grid, kGemmThreads, smem, stream>>>(p);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

template <int BN, bool OUT_F32>
int launch_by_epilogue(GemmArgs &p, const DeviceInfo &dev, cudaStream_t stream) {
    switch (p.epilogue) {
        case TB200_EPI_NONE: return launch_tcgen05<BN, TB200_EPI_NONE, OUT_F32>(p, dev, stream);
        case TB200_EPI_BIAS: return launch_tcgen05<BN, TB200_EPI_BIAS, OUT_F32>(p, dev, stream);
        case TB200_EPI_AXPY: return launch_tcgen05<BN, TB200_EPI_AXPY, OUT_F32>(p, dev, stream);
        default: break;
    }
    // activations and their pullbacks are instantiated for BFloat16 results only
    if constexpr (!OUT_F32) {
        switch (p.epilogue) {
            case TB200_EPI_BIAS_GELU: return launch_tcgen05<BN, TB200_EPI_BIAS_GELU, false>(p, dev, stream);
            case TB200_EPI_BIAS_TANH: return launch_tcgen05<BN, TB200_EPI_BIAS_TANH, false>(p, dev, stream);
            case TB200_EPI_MUL_GELU_GRAD: return launch_tcgen05<BN, TB200_EPI_MUL_GELU_GRAD, false>(p, dev, stream);
            case TB200_EPI_MUL_TANH_GRAD: return launch_tcgen05<BN, TB200_EPI_MUL_TANH_GRAD, false>(p, dev, stream);
            default: break;
        }
    }
    return TB200_ERR_UNSUPPORTED;
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" int tb200_gemm(const tb200_gemm_desc *d, const void *a, const void *b, void *c, const void *bias,
                          const void *aux, void *aux_out, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!d) return TB200_ERR_NULL;
    if (d->m < 0 || d->n < 0 || d->k < 0 || d->m > INT32_MAX || d->n > INT32_MAX || d->k > INT32_MAX)
        return TB200_ERR_SHAPE;
    if ((d->in_dtype != TB200_F32 && d->in_dtype != TB200_BF16) ||
        (d->out_dtype != TB200_F32 && d->out_dtype != TB200_BF16))
        return TB200_ERR_DTYPE;
    if (d->epilogue < TB200_EPI_NONE || d->epilogue > TB200_EPI_AXPY) return TB200_ERR_UNSUPPORTED;
    if (d->m == 0 || d->n == 0) return TB200_OK;
    const int64_t a_inner = d->a_layout == TB200_MN_MAJOR ? d->m : d->k;
    const int64_t b_inner = d->b_layout == TB200_MN_MAJOR ? d->n : d->k;
    if (d->lda < a_inner || d->ldb < b_inner || d->ldc < d->n) return TB200_ERR_SHAPE;
    if (!c || (d->k > 0 && (!a || !b))) return TB200_ERR_NULL;
    const bool needs_bias = d->epilogue == TB200_EPI_BIAS || d->epilogue == TB200_EPI_BIAS_GELU ||
                            d->epilogue == TB200_EPI_BIAS_TANH;
    const bool needs_aux = d->epilogue == TB200_EPI_MUL_GELU_GRAD || d->epilogue == TB200_EPI_MUL_TANH_GRAD ||
                           d->epilogue == TB200_EPI_AXPY;
    if ((needs_bias && !bias) || (needs_aux && !aux)) return TB200_ERR_NULL;
    if (needs_aux && d->ld_aux < d->n) return TB200_ERR_SHAPE;
    if (aux_out && d->ld_aux_out < d->n) return TB200_ERR_SHAPE;
    const size_t in_size = dtype_size(d->in_dtype), out_size = dtype_size(d->out_dtype);
    if (!aligned_to(a, in_size) || !aligned_to(b, in_size) || !aligned_to(c, out_size) ||
        !aligned_to(bias, in_size) || !aligned_to(aux, 2) || !aligned_to(aux_out, in_size))
        return TB200_ERR_ALIGN;
    DeviceInfo dev;
    int st = current_device(&dev);
    if (st) return st;

    const bool activation = d->epilogue == TB200_EPI_BIAS_GELU || d->epilogue == TB200_EPI_BIAS_TANH ||
                            d->epilogue == TB200_EPI_MUL_GELU_GRAD || d->epilogue == TB200_EPI_MUL_TANH_GRAD;
    const bool tma_ok = d->in_dtype == TB200_BF16 && d->k > 0 && aligned_to(a, 16) && aligned_to(b, 16) &&
                        d->lda % 8 == 0 && d->ldb % 8 == 0 && !d->force_simt &&
                        !(activation && d->out_dtype == TB200_F32);
    if (tma_ok) {
        GemmArgs p{};
        p.c = c; p.bias = bias; p.aux = aux; p.aux_out = aux_out;
        p.ldc = d->ldc; p.ld_aux = d->ld_aux; p.ld_aux_out = d->ld_aux_out;
        p.alpha = d->alpha; p.m = static_cast<int>(d->m); p.n = static_cast<int>(d->n); p.k = static_cast<int>(d->k);
        p.epilogue = d->epilogue; p.out_f32 = d->out_dtype == TB200_F32;
        p.a_mn = d->a_layout == TB200_MN_MAJOR; p.b_mn = d->b_layout == TB200_MN_MAJOR;
        // 128 x 256 tiles halve the operand bytes per flop of 128 x 128 ones and measured faster on every
        // shape wide enough to hold one, even when they leave a few SMs idle
        const bool wide = d->tile_n == 256 || (d->tile_n == 0 && d->n > 128);
        const int bn = wide ? 256 : 128;
        if (p.a_mn) st = make_tmap(&p.tmap_a, a, d->m, d->k, d->lda, 64);
        else st = make_tmap(&p.tmap_a, a, d->k, d->m, d->lda, BM);
        if (st) return st;
        if (p.b_mn) st = make_tmap(&p.tmap_b, b, d->n, d->k, d->ldb, 64);
        else st = make_tmap(&p.tmap_b, b, d->k, d->n, d->ldb, bn);
        if (st) return st;
        // the epilogue goes through shared memory and TMA when every array it touches can be
        // described to the TMA unit; otherwise each thread stores its own row
        const bool out_f32 = d->out_dtype == TB200_F32;
        const size_t aux_size = (d->epilogue == TB200_EPI_AXPY) ? out_size : 2;
        bool tma_epi = !d->direct_epilogue && aligned_to(c, 16) && (d->ldc * out_size) % 16 == 0;
        if (needs_aux) tma_epi = tma_epi && aux_size == out_size && aligned_to(aux, 16) && (d->ld_aux * aux_size) % 16 == 0;
        if (aux_out) tma_epi = tma_epi && !out_f32 && aligned_to(aux_out, 16) && (d->ld_aux_out * 2) % 16 == 0;
        if (tma_epi) {
            if ((st = make_tmap(&p.tmap_c, c, d->n, d->m, d->ldc, 32, out_f32))) return st;
            if (needs_aux && (st = make_tmap(&p.tmap_aux, aux, d->n, d->m, d->ld_aux, 32, out_f32))) return st;
            if (aux_out && (st = make_tmap(&p.tmap_aux_out, aux_out, d->n, d->m, d->ld_aux_out, 32, false))) return st;
        }
        p.tma_epilogue = tma_epi;
        if (out_f32) return wide ? launch_by_epilogue<256, true>(p, dev, stream) : launch_by_epilogue<128, true>(p, dev, stream);
        return wide ? launch_by_epilogue<256, false>(p, dev, stream) : launch_by_epilogue<128, false>(p, dev, stream);
    }

    SimtArgs p{};
    p.a = a; p.b = b; p.c = c; p.bias = bias; p.aux = aux; p.aux_out = aux_out;
    p.lda = d->lda; p.ldb = d->ldb; p.ldc = d->ldc; p.ld_aux = d->ld_aux; p.ld_aux_out = d->ld_aux_out;
    p.alpha = d->alpha; p.m = static_cast<int>(d->m); p.n = static_cast<int>(d->n); p.k = static_cast<int>(d->k);
    p.epilogue = d->epilogue; p.in_f32 = d->in_dtype == TB200_F32; p.out_f32 = d->out_dtype == TB200_F32;
    p.a_mn = d->a_layout == TB200_MN_MAJOR; p.b_mn = d->b_layout == TB200_MN_MAJOR;
    dim3 grid(static_cast<unsigned>(ceil_div(d->n, 64)), static_cast<unsigned>(ceil_div(d->m, 64)));
    if (grid.y > 65535) return TB200_ERR_SHAPE;
    gemm_simt<<<grid, 256, 0, stream>>>(p);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

// Synchronises the device and returns (then clears) the error code a tensor-core kernel recorded when one
// of its bounded waits ran out: 0 none, 1 loader, 2 accumulator hand-back, 3 operands, 4 epilogue.
extern "C" int tb200_device_error(void) {
    int code = 0, zero = 0;
    TB200_CUDA(cudaDeviceSynchronize());
    TB200_CUDA(cudaMemcpyFromSymbol(&code, g_gemm_error, sizeof(int)));
    if (code) TB200_CUDA(cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int)));
    return code;
}

// Times the compiled-in tile variants of one product on its own operands and returns the faster one's
// tile_n (128 or 256) -- the measured stage of the reference's search over a claim's `variants`
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
    const bool measurable = d->in_dtype == TB200_BF16 && d->n > 128 && d->m > 0 && d->k > 0 && !d->force_simt &&
                            d->epilogue != TB200_EPI_AXPY;
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
    for (int width : {128, 256}) {
        trial.tile_n = width;
        if ((status = tb200_gemm(&trial, a, b, c, bias, aux, aux_out, stream_))) break;   // warm-up and validation
        if (cudaEventRecord(t0, stream) != cudaSuccess) { status = TB200_ERR_CUDA; break; }
        for (int rep = 0; rep < 3 && !status; rep++) status = tb200_gemm(&trial, a, b, c, bias, aux, aux_out, stream_);
        if (status) break;
        float ms = 0.0f;
        if (cudaEventRecord(t1, stream) != cudaSuccess || cudaEventSynchronize(t1) != cudaSuccess ||
            cudaEventElapsedTime(&ms, t0, t1) != cudaSuccess) { status = TB200_ERR_CUDA; break; }
        if (width == 128 || ms < best_ms) { best_ms = ms; best = width; }
    }
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    return status ? status : best;
}
