// Flash-attention backward for sm_100a, the deterministic two-kernel form: no atomics, every
// gradient element is written once, results repeat bit for bit (the reference's `deterministic = true`
// spelling, where dQ is a second fold of its own: ext/cuTileExt/build.jl:295-318, docs/src/cuda.md:64-75).
//
//   stats      delta[m] = sum_d dO[d,m] o[d,m] (o as stored in BFloat16) and lse * log2(e), both
//              re-laid out [batch][head][query] so that consecutive queries are contiguous
//   dK, dV     one item = 128 keys of one (batch, key/value head); steps of 64 queries (of every query
//              head of the group):  S' = K Q', dP' = V dO'  ->  P' = exp2(S' c - lse), dS' = P' (dP' - delta)
//              ->  dV += P' dO,  dK += dS' Q
//   dQ         one item = 128 queries of one (batch, head); steps of 64 keys:
//              S = Q K', dP = dO V'  ->  dS = P (dP - delta)  ->  dQ += dS K
//
// Both run the same warp-specialised pipeline as the forward kernel: one thread issues TMA loads (the
// item's 128-row operands once, the steps' 64-row operands through a 3-stage ring), one thread issues
// tcgen05.mma (the two score products of step t+1 before the gradient products of step t), four warps
// own one tensor-memory lane = one of the item's 128 rows each, read both 64-column score tiles into
// registers, and write P / dS as BFloat16 into 128-byte-swizzled shared tiles that feed the gradient
// products as K-major A operands; the steps' operands serve as MN-major B operands straight from their
// [position][feature] layout.  Accumulators stay in tensor memory for the whole item.
// Tensor memory: 2 x (S, dP) of 64 columns + two 128-column accumulators = 512 columns.
// No load uses cluster multicast.  Every barrier wait is bounded.
#include <cuda.h>

#include <mutex>

#include "attention_simt.cuh"
#include "common.cuh"
#include "sm100.cuh"

namespace tb200 {
namespace {

using namespace sm100;

constexpr int kOuter = 128;                 // rows of an item
constexpr int kInner = 64;                  // positions per step
constexpr int kD = 128;                     // features
constexpr int kOuterSlab = kOuter * 128;    // [128 rows][64 features]: 16 KB
constexpr int kOuterBytes = 2 * kOuterSlab;
constexpr int kInnerSlab = kInner * 128;    // [64 rows][64 features]: 8 KB
constexpr int kInnerBytes = 2 * kInnerSlab;
constexpr int kDsBytes = kOuter * 128;      // [128 rows][64 positions] BFloat16: 16 KB
constexpr int kStages = 3;
constexpr int kBwdThreads = 320;   // loader, MMA issuer, two groups of four row warps taking alternate steps

__device__ int g_attn_bwd_error = 0;

struct AttnBwdArgs {
    CUtensorMap outer_a, outer_b;   // dK/dV: K, V   | dQ: Q, dO     (boxes of 128 rows)
    CUtensorMap inner_a, inner_b;   // dK/dV: Q, dO  | dQ: K, V      (boxes of 64 rows)
    CUtensorMap out1, out2;         // dK/dV: dV, dK | dQ: -, dQ     (boxes of 32 rows)
    const float *lse2;              // [batch][head][query]  lse * log2(e)
    const float *delta;             // [batch][head][query]
    int batch, heads, kv_heads, queries, keys;
    int outer_tiles, items;
    int causal;
    float scale, scale_log2;
};

__device__ __forceinline__ uint64_t bwd_now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool bwd_wait(uint64_t *bar, uint32_t parity, volatile int *failed, int code) {
    if (mbar_wait(bar, parity, 4096)) return true;
    const uint64_t t0 = bwd_now_ns();
    while (true) {
        if (mbar_wait(bar, parity, 1024)) return true;
        if (*failed) return false;
        if (bwd_now_ns() - t0 > 2000000000ull) {
            *failed = code;
            atomicCAS(&g_attn_bwd_error, 0, code);
            return false;
        }
    }
}

// The steps of an item: which head and which 64-position chunk step t reads.
template <bool DKDV>
struct Steps {
    int b, head_outer, tile;   // the item
    int c0, nc, group, count;
    __device__ __forceinline__ Steps(const AttnBwdArgs &p, int item) {
        group = p.heads / p.kv_heads;
        if (DKDV) {
            // heaviest first under the causal mask: the first keys see every query
            const int per = p.batch * p.kv_heads;
            tile = item / per;
            b = (item % per) / p.kv_heads;
            head_outer = item % p.kv_heads;
            const int all = (p.queries + kInner - 1) / kInner;
            c0 = p.causal ? (tile * kOuter) / kInner : 0;
            if (c0 > all) c0 = all;
            nc = all - c0;
            count = nc * group;
        } else {
            const int per = p.batch * p.heads;
            tile = p.outer_tiles - 1 - item / per;
            b = (item % per) / p.heads;
            head_outer = item % p.heads;
            const int all = (p.keys + kInner - 1) / kInner;
            c0 = 0;
            nc = all;
            if (p.causal) {
                const int upto = (tile * kOuter + kOuter - 1) / kInner + 1;
                if (upto < nc) nc = upto;
            }
            count = nc;
        }
    }
    // head the inner operands of step t belong to, and their first position
    __device__ __forceinline__ void at(int t, int &head_inner, int &pos0) const {
        if (DKDV) {
            head_inner = head_outer * group + t / nc;
            pos0 = (c0 + t % nc) * kInner;
        } else {
            head_inner = head_outer / group;
            pos0 = t * kInner;
        }
    }
};

template <bool DKDV>
__global__ void __launch_bounds__(kBwdThreads, 1) attention_bwd_kernel(const __grid_constant__ AttnBwdArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *s_outer_a = smem;
    uint8_t *s_outer_b = s_outer_a + kOuterBytes;
    uint8_t *s_inner = s_outer_b + kOuterBytes;              // kStages x (A 16 KB | B 16 KB)
    uint8_t *s_ds = s_inner + kStages * 2 * kInnerBytes;     // 2 x (P 16 KB | dS 16 KB); also stages the stores

    __shared__ __align__(8) uint64_t outer_full, outer_empty, acc_done, acc_free;
    __shared__ __align__(8) uint64_t inner_full[kStages], inner_empty[kStages];
    __shared__ __align__(8) uint64_t t_full[2], ds_full[2];
    __shared__ __align__(8) uint64_t stats_ready[2];   // a group's four warps have written the step's statistics
    __shared__ uint32_t tmem_base_smem;
    __shared__ int failed_smem;
    // dK/dV: the step's 64 queries' lse*log2(e) [0, 64) and delta [64, 128), per group, double-buffered
    __shared__ __align__(16) float col_stats[2][2][2 * kInner];
    volatile int *failed = &failed_smem;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        failed_smem = 0;
        mbar_init(&outer_full, 1); mbar_init(&outer_empty, 1); mbar_init(&acc_done, 1); mbar_init(&acc_free, 8);
        for (int s = 0; s < kStages; s++) { mbar_init(&inner_full[s], 1); mbar_init(&inner_empty[s], 1); }
        for (int s = 0; s < 2; s++) {
            mbar_init(&t_full[s], 1);
            mbar_init(&ds_full[s], 4);
            mbar_init(&stats_ready[s], 4);
        }
        fence_barrier_init();
        prefetch_tensormap(&p.outer_a); prefetch_tensormap(&p.outer_b);
        prefetch_tensormap(&p.inner_a); prefetch_tensormap(&p.inner_b);
        prefetch_tensormap(&p.out2);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_smem, 512);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_smem;
    const uint32_t tmem_acc1 = tmem_base + 256, tmem_acc2 = tmem_base + 384;

    if (warp == 0) {
        if (elect_one()) {
            uint32_t outer_phase = 0, step_count = 0;
            for (int item = blockIdx.x; item < p.items && !*failed; item += gridDim.x) {
                const Steps<DKDV> steps(p, item);
                if (!bwd_wait(&outer_empty, outer_phase ^ 1, failed, 1)) break;
                outer_phase ^= 1;
                mbar_arrive_expect_tx(&outer_full, 2 * kOuterBytes);
                const int r0 = steps.tile * kOuter;
                tma_load_4d(s_outer_a, &p.outer_a, &outer_full, 0, steps.head_outer, r0, steps.b);
                tma_load_4d(s_outer_a + kOuterSlab, &p.outer_a, &outer_full, 64, steps.head_outer, r0, steps.b);
                tma_load_4d(s_outer_b, &p.outer_b, &outer_full, 0, steps.head_outer, r0, steps.b);
                tma_load_4d(s_outer_b + kOuterSlab, &p.outer_b, &outer_full, 64, steps.head_outer, r0, steps.b);
                for (int t = 0; t < steps.count; t++, step_count++) {
                    const int st = step_count % kStages;
                    const uint32_t ph = (step_count / kStages) & 1;
                    if (!bwd_wait(&inner_empty[st], ph ^ 1, failed, 2)) break;
                    int hi, pos0;
                    steps.at(t, hi, pos0);
                    uint8_t *sa = s_inner + st * 2 * kInnerBytes, *sb = sa + kInnerBytes;
                    mbar_arrive_expect_tx(&inner_full[st], 2 * kInnerBytes);
                    tma_load_4d(sa, &p.inner_a, &inner_full[st], 0, hi, pos0, steps.b);
                    tma_load_4d(sa + kInnerSlab, &p.inner_a, &inner_full[st], 64, hi, pos0, steps.b);
                    tma_load_4d(sb, &p.inner_b, &inner_full[st], 0, hi, pos0, steps.b);
                    tma_load_4d(sb + kInnerSlab, &p.inner_b, &inner_full[st], 64, hi, pos0, steps.b);
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc_t = umma_idesc_bf16(kOuter, kInner, false, false);   // 128 x 64, both K-major
            const uint32_t idesc_g = umma_idesc_bf16(kOuter, kD, false, true);        // 128 x 128, B MN-major
            uint32_t outer_phase = 0, step_count = 0, grad_count = 0, item_count = 0;
            for (int item = blockIdx.x; item < p.items && !*failed; item += gridDim.x) {
                const Steps<DKDV> steps(p, item);
                if (!bwd_wait(&outer_full, outer_phase, failed, 3)) break;
                outer_phase ^= 1;
                tcgen05_fence_after();
                if (steps.count == 0) {   // nothing reads the item's operands
                    mbar_arrive(&outer_empty);
                    continue;
                }
                bool ok = true;
                for (int t = 0; t <= steps.count && ok; t++) {
                    if (t < steps.count) {
                        const uint32_t c = step_count + t;
                        const int st = c % kStages;
                        const uint32_t ph = (c / kStages) & 1;
                        const int tb = c & 1;
                        const uint32_t tph = (c >> 1) & 1;
                        // buffer tb was last read by the gradient products of two steps ago, issued before this
                        // point: MMAs of one CTA run in issue order, so no barrier is needed to reuse it
                        if (!bwd_wait(&inner_full[st], ph, failed, 4)) { ok = false; break; }
                        tcgen05_fence_after();
                        const uint32_t oa = smem_u32(s_outer_a), ob = smem_u32(s_outer_b);
                        const uint32_t ia = smem_u32(s_inner + st * 2 * kInnerBytes), ib = ia + kInnerBytes;
                        const uint32_t t1 = tmem_base + tb * 128, t2 = t1 + 64;
#pragma unroll
                        for (int k = 0; k < kD / 16; k++) {
                            const uint32_t ooff = (k >> 2) * kOuterSlab + (k & 3) * 32;
                            const uint32_t ioff = (k >> 2) * kInnerSlab + (k & 3) * 32;
                            tcgen05_mma_f16(t1, umma_smem_desc(oa + ooff, 16, 1024), umma_smem_desc(ia + ioff, 16, 1024),
                                            idesc_t, k != 0);
                        }
#pragma unroll
                        for (int k = 0; k < kD / 16; k++) {
                            const uint32_t ooff = (k >> 2) * kOuterSlab + (k & 3) * 32;
                            const uint32_t ioff = (k >> 2) * kInnerSlab + (k & 3) * 32;
                            tcgen05_mma_f16(t2, umma_smem_desc(ob + ooff, 16, 1024), umma_smem_desc(ib + ioff, 16, 1024),
                                            idesc_t, k != 0);
                        }
                        tcgen05_commit(&t_full[tb]);
                        if (t == steps.count - 1) tcgen05_commit(&outer_empty);
                    }
                    if (t > 0) {
                        const uint32_t c = grad_count;
                        const int st = c % kStages;
                        const int db = c & 1;
                        const uint32_t dph = (c >> 1) & 1;
                        // the first gradient product of an item overwrites the accumulators
                        if (t == 1 && !bwd_wait(&acc_free, (item_count & 1) ^ 1, failed, 6)) { ok = false; break; }
                        if (!bwd_wait(&ds_full[db], dph, failed, 7)) { ok = false; break; }
                        tcgen05_fence_after();
                        const uint32_t ia = smem_u32(s_inner + st * 2 * kInnerBytes), ib = ia + kInnerBytes;
                        // A: P / dS from tensor memory, 16 positions = 8 packed columns per MMA, written by the row
                        // threads over the scores / dP they were computed from; B: 16 position lines of 128 bytes
                        const uint32_t pa = tmem_base + db * 128, da = pa + 64;
#pragma unroll
                        for (int k = 0; k < kInner / 16; k++) {
                            if (DKDV)
                                tcgen05_mma_f16_ts(tmem_acc1, pa + k * 8, umma_smem_desc(ib + k * 2048, kInnerSlab, 1024), idesc_g,
                                                   (t - 1) | k);
                            tcgen05_mma_f16_ts(tmem_acc2, da + k * 8, umma_smem_desc(ia + k * 2048, kInnerSlab, 1024), idesc_g,
                                               (t - 1) | k);
                        }
                        tcgen05_commit(&inner_empty[st]);
                        if (t == steps.count) tcgen05_commit(&acc_done);
                        grad_count++;
                    }
                }
                step_count += steps.count;
                item_count++;   // items that ran gradient products
                if (!ok) break;
            }
        }
    } else {
        // ---- one thread per row of the item; the two groups of four warps take alternate steps (the
        // score and P / dS buffers of a step are those of its parity), so one group's chain of
        // tensor-memory load -> exponentials -> shared-memory stores overlaps the other's
        const int q4 = warp & 3;
        const int group = (warp - 2) >> 2;
        const int row = q4 * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
        uint32_t step_count = 0, item_count = 0, own_steps = 0;
        for (int item = blockIdx.x; item < p.items; item += gridDim.x) {
            const Steps<DKDV> steps(p, item);
            const int outer_pos = steps.tile * kOuter + row;   // this thread's key (dK/dV) or query (dQ)
            float row_lse2 = 0.0f, row_delta = 0.0f;
            if (!DKDV && outer_pos < p.queries) {
                const long long i = (static_cast<long long>(steps.b) * p.heads + steps.head_outer) * p.queries + outer_pos;
                row_lse2 = p.lse2[i];
                row_delta = p.delta[i];
            }
            bool ok = true;
            const uint32_t step_base = step_count;
            step_count += steps.count;
            for (int t = 0; t < steps.count; t++) {
                const uint32_t sc = step_base + t;
                const int tb = sc & 1;
                if (tb != group) continue;
                const uint32_t tph = (sc >> 1) & 1;
                int hi, pos0;
                steps.at(t, hi, pos0);
                float *stats = col_stats[group][tph];
                if (DKDV) {
                    // fetched before the wait below so that the global-memory latency hides behind it
                    const int i = row & (kInner - 1);
                    const int qpos = pos0 + i;
                    const long long base = (static_cast<long long>(steps.b) * p.heads + hi) * p.queries;
                    const float *src = row < kInner ? p.lse2 : p.delta;
                    stats[row] = qpos < p.queries ? __ldg(src + base + qpos) : 0.0f;
                }
                if (!bwd_wait(&t_full[tb], tph, failed, 8)) { ok = false; break; }
                tcgen05_fence_after();
                if (DKDV) {
                    // the group's four warps meet (a bounded wait, unlike a named barrier: a warp that gave up on a
                    // failed wait elsewhere must not leave the others hanging here)
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&stats_ready[group]);
                    if (!bwd_wait(&stats_ready[group], own_steps & 1, failed, 12)) { ok = false; break; }
                    own_steps++;
                }
                uint32_t s[kInner], dp[kInner];
                const uint32_t t1 = tmem_base + lane_base + tb * 128;
                tmem_ld_32x32(t1, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
                tmem_ld_32x32(t1 + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
                tmem_ld_32x32(t1 + 64, *reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
                tmem_ld_32x32(t1 + 96, *reinterpret_cast<uint32_t(*)[32]>(&dp[32]));
                tmem_ld_wait();
                const bool edge = DKDV ? (pos0 + kInner > p.queries || outer_pos >= p.keys ||
                                          (p.causal && pos0 < steps.tile * kOuter + kOuter))
                                       : (pos0 + kInner > p.keys || outer_pos >= p.queries ||
                                          (p.causal && pos0 + kInner - 1 > steps.tile * kOuter));
                if (edge) {
                    // masked positions get a score of -Inf: their weight and their dS are then exactly zero
#pragma unroll
                    for (int i = 0; i < kInner; i++) {
                        const int inner_pos = pos0 + i;
                        const int key = DKDV ? outer_pos : inner_pos;
                        const int query = DKDV ? inner_pos : outer_pos;
                        if (key >= p.keys || query >= p.queries || (p.causal && key > query)) s[i] = 0xff800000u;
                    }
                }
#pragma unroll
                for (int g = 0; g < kInner / 8; g++) {
                    float pv[8], dv[8];
                    float l8[8], d8[8];
                    if (DKDV) {
                        const float4 a0 = *reinterpret_cast<const float4 *>(stats + 8 * g);
                        const float4 a1 = *reinterpret_cast<const float4 *>(stats + 8 * g + 4);
                        const float4 b0 = *reinterpret_cast<const float4 *>(stats + kInner + 8 * g);
                        const float4 b1 = *reinterpret_cast<const float4 *>(stats + kInner + 8 * g + 4);
                        l8[0] = a0.x; l8[1] = a0.y; l8[2] = a0.z; l8[3] = a0.w;
                        l8[4] = a1.x; l8[5] = a1.y; l8[6] = a1.z; l8[7] = a1.w;
                        d8[0] = b0.x; d8[1] = b0.y; d8[2] = b0.z; d8[3] = b0.w;
                        d8[4] = b1.x; d8[5] = b1.y; d8[6] = b1.z; d8[7] = b1.w;
                    }
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int i = 8 * g + u;
                        const float lse2 = DKDV ? l8[u] : row_lse2;
                        const float dl = DKDV ? d8[u] : row_delta;
                        const float pw = fast_exp2(fmaf(__uint_as_float(s[i]), p.scale_log2, -lse2));
                        pv[u] = pw;
                        dv[u] = pw * (__uint_as_float(dp[i]) - dl);
                    }
                    // packed two per column over the values they came from: s becomes P, dp becomes dS
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        if (DKDV) s[4 * g + u] = pack_bf16x2(pv[2 * u], pv[2 * u + 1]);
                        dp[4 * g + u] = pack_bf16x2(dv[2 * u], dv[2 * u + 1]);
                    }
                }
                if (DKDV) tmem_st_32x32(t1, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
                tmem_st_32x32(t1 + 64, *reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
                tmem_st_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ds_full[tb]);
            }
            if (!ok) break;
            // ---- the item's gradients: accumulators -> BFloat16 -> shared staging -> TMA stores
            if (steps.count > 0) {
                if (!bwd_wait(&acc_done, item_count & 1, failed, 10)) break;
            }
            tcgen05_fence_after();
            // group 0 writes the first accumulator (dV), group 1 the second (dK, or dQ)
#pragma unroll 1
            for (int which = group; which <= group && (DKDV || which == 1); which++) {
                const float mul = which == 0 ? 1.0f : p.scale;
                uint8_t *stage = s_ds + which * 2 * kDsBytes;   // 32 KB: two 64-feature slabs of 128 rows
                uint32_t r[kD];
                if (steps.count > 0) {
#pragma unroll
                    for (int c = 0; c < kD / 32; c++)
                        tmem_ld_32x32((which == 0 ? tmem_acc1 : tmem_acc2) + lane_base + c * 32,
                                      *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < kD; i++) r[i] = 0u;   // no step touched this item: its gradient is zero
                }
#pragma unroll
                for (int g = 0; g < kD / 8; g++) {
                    uint4 v4;
                    v4.x = pack_bf16x2(__uint_as_float(r[8 * g]) * mul, __uint_as_float(r[8 * g + 1]) * mul);
                    v4.y = pack_bf16x2(__uint_as_float(r[8 * g + 2]) * mul, __uint_as_float(r[8 * g + 3]) * mul);
                    v4.z = pack_bf16x2(__uint_as_float(r[8 * g + 4]) * mul, __uint_as_float(r[8 * g + 5]) * mul);
                    v4.w = pack_bf16x2(__uint_as_float(r[8 * g + 6]) * mul, __uint_as_float(r[8 * g + 7]) * mul);
                    *reinterpret_cast<uint4 *>(stage + (g >> 3) * kOuterSlab + row * 128 + (((g & 7) ^ (row & 7)) << 4)) = v4;
                }
            }
            tcgen05_fence_before();
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                const int r0 = steps.tile * kOuter + q4 * 32;
                if (DKDV && group == 0) {
                    tma_store_4d(&p.out1, s_ds + q4 * 32 * 128, 0, steps.head_outer, r0, steps.b);
                    tma_store_4d(&p.out1, s_ds + kOuterSlab + q4 * 32 * 128, 64, steps.head_outer, r0, steps.b);
                }
                if (group == 1) {
                    tma_store_4d(&p.out2, s_ds + 2 * kDsBytes + q4 * 32 * 128, 0, steps.head_outer, r0, steps.b);
                    tma_store_4d(&p.out2, s_ds + 2 * kDsBytes + kOuterSlab + q4 * 32 * 128, 64, steps.head_outer, r0, steps.b);
                }
                bulk_commit_group();
                bulk_wait_group_read<0>();
                if (steps.count > 0) mbar_arrive(&acc_free);
            }
            __syncwarp();
            if (steps.count > 0) item_count++;
        }
        if (lane == 0) bulk_wait_group<0>();
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// delta[b][h][m] = sum_d dO o ; lse2[b][h][m] = lse[b][m][h] * log2(e).  16 threads per (b, m, h) row.
__global__ void __launch_bounds__(256) attention_stats_kernel(const __nv_bfloat16 *o, const __nv_bfloat16 *dout,
                                                              const float *lse, float *lse2, float *delta, int batch,
                                                              int heads, int queries, int d) {
    const long long rows = static_cast<long long>(batch) * queries * heads;
    const long long r = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 4;
    const int t = threadIdx.x & 15;
    float s = 0.0f;
    if (r < rows) {
        for (int i = t * 8; i < d; i += 128) {
            float a[8], g[8];
            Access<__nv_bfloat16, true>::load(o + r * d + i, a);
            Access<__nv_bfloat16, true>::load(dout + r * d + i, g);
#pragma unroll
            for (int e = 0; e < 8; e++) s = fmaf(a[e], g[e], s);
        }
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (r < rows && t == 0) {
        const int h = static_cast<int>(r % heads);
        const long long bm = r / heads;
        const int m = static_cast<int>(bm % queries);
        const long long b = bm / queries;
        const long long out = (b * heads + h) * queries + m;
        delta[out] = s;
        lse2[out] = lse[r] * kLog2e;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int bwd_encode_fn(EncodeTiledFn *out) {
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

int bwd_tmap(CUtensorMap *map, const void *base, int d, int heads, int positions, int batch, int rows) {
    EncodeTiledFn fn;
    int st = bwd_encode_fn(&fn);
    if (st) return st;
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(heads),
                          static_cast<cuuint64_t>(positions), static_cast<cuuint64_t>(batch)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(d) * 2, static_cast<cuuint64_t>(d) * heads * 2,
                             static_cast<cuuint64_t>(d) * heads * positions * 2};
    cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(rows), 1};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TB200_OK : TB200_ERR_UNSUPPORTED;
}

template <bool DKDV>
int launch_bwd(AttnBwdArgs &p, const DeviceInfo &dev, cudaStream_t stream) {
    // the tiles (224 KB, 1024-byte aligned) sit behind the kernel's static shared memory: take all the dynamic
    // shared memory the SM has left
    const size_t tiles = 2 * kOuterBytes + kStages * 2 * kInnerBytes + 2 * 2 * kDsBytes;
    static std::mutex lock;
    static size_t dynamic_bytes[64] = {};
    {
        std::lock_guard<std::mutex> hold(lock);
        if (!dynamic_bytes[dev.device]) {
            cudaFuncAttributes attr;
            TB200_CUDA(cudaFuncGetAttributes(&attr, attention_bwd_kernel<DKDV>));
            const size_t first = (attr.sharedSizeBytes + 1023) / 1024 * 1024;
            if (first + tiles > dev.smem_optin) return TB200_ERR_UNSUPPORTED;
            const size_t room = dev.smem_optin - attr.sharedSizeBytes;
            TB200_CUDA(cudaFuncSetAttribute(attention_bwd_kernel<DKDV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(room)));
            dynamic_bytes[dev.device] = room;
        }
    }
    const size_t smem = dynamic_bytes[dev.device];
    const unsigned grid = static_cast<unsigned>(p.items < dev.sms ? p.items : dev.sms);
    attention_bwd_kernel<DKDV><<<grid, kBwdThreads, smem, stream>>>(p);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" size_t tb200_attention_bwd_workspace_bytes(const tb200_attn_desc *d) {
    if (!d || d->batch <= 0 || d->heads <= 0 || d->queries <= 0) return 0;
    return static_cast<size_t>(2) * d->batch * d->heads * d->queries * sizeof(float);
}

extern "C" int tb200_attention_bwd(const tb200_attn_desc *d, const void *q, const void *k, const void *v,
                                   const void *o, const float *lse, const void *dout, void *dq, void *dk, void *dv,
                                   void *workspace, size_t workspace_bytes, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!d) return TB200_ERR_NULL;
    if (d->batch < 0 || d->heads <= 0 || d->kv_heads <= 0 || d->queries < 0 || d->keys < 0 || d->head_dim <= 0)
        return TB200_ERR_SHAPE;
    if (d->heads % d->kv_heads != 0 || !(d->scale > 0.0f)) return TB200_ERR_SHAPE;
    if (d->causal && d->queries != d->keys) return TB200_ERR_SHAPE;
    if (d->dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (d->head_dim != kD && !attention_simt_takes(d)) return TB200_ERR_UNSUPPORTED;
    if (d->batch == 0 || (d->queries == 0 && d->keys == 0)) return TB200_OK;
    if (d->queries == 0 || d->keys == 0) return TB200_ERR_UNSUPPORTED;
    if (!q || !k || !v || !o || !lse || !dout || !dq || !dk || !dv) return TB200_ERR_NULL;
    for (const void *ptr : {q, k, v, o, dout, static_cast<const void *>(dq), static_cast<const void *>(dk),
                            static_cast<const void *>(dv)})
        if (!aligned_to(ptr, 16)) return TB200_ERR_ALIGN;
    if (!aligned_to(lse, 4)) return TB200_ERR_ALIGN;
    const size_t need = tb200_attention_bwd_workspace_bytes(d);
    if (!workspace || workspace_bytes < need || !aligned_to(workspace, 16)) return TB200_ERR_WORKSPACE;
    if (d->head_dim != kD) return attention_simt_bwd(d, q, k, v, o, lse, dout, dq, dk, dv, stream);
    DeviceInfo dev;
    int st = current_device(&dev);
    if (st) return st;

    const long long stat_len = static_cast<long long>(d->batch) * d->heads * d->queries;
    float *lse2 = static_cast<float *>(workspace);
    float *delta = lse2 + stat_len;
    {
        const long long threads = stat_len * 16;
        const unsigned blocks = static_cast<unsigned>(ceil_div(threads, 256));
        attention_stats_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(o),
                                                           static_cast<const __nv_bfloat16 *>(dout), lse, lse2, delta,
                                                           d->batch, d->heads, d->queries, d->head_dim);
        TB200_CUDA(cudaGetLastError());
    }
    AttnBwdArgs p{};
    p.lse2 = lse2; p.delta = delta;
    p.batch = d->batch; p.heads = d->heads; p.kv_heads = d->kv_heads; p.queries = d->queries; p.keys = d->keys;
    p.causal = d->causal; p.scale = d->scale; p.scale_log2 = d->scale * kLog2e;
    // dK, dV: items over key tiles
    if ((st = bwd_tmap(&p.outer_a, k, kD, d->kv_heads, d->keys, d->batch, kOuter))) return st;
    if ((st = bwd_tmap(&p.outer_b, v, kD, d->kv_heads, d->keys, d->batch, kOuter))) return st;
    if ((st = bwd_tmap(&p.inner_a, q, kD, d->heads, d->queries, d->batch, kInner))) return st;
    if ((st = bwd_tmap(&p.inner_b, dout, kD, d->heads, d->queries, d->batch, kInner))) return st;
    if ((st = bwd_tmap(&p.out1, dv, kD, d->kv_heads, d->keys, d->batch, 32))) return st;
    if ((st = bwd_tmap(&p.out2, dk, kD, d->kv_heads, d->keys, d->batch, 32))) return st;
    p.outer_tiles = static_cast<int>(ceil_div(d->keys, kOuter));
    p.items = p.outer_tiles * d->batch * d->kv_heads;
    if ((st = launch_bwd<true>(p, dev, stream))) return st;
    // dQ: items over query tiles
    if ((st = bwd_tmap(&p.outer_a, q, kD, d->heads, d->queries, d->batch, kOuter))) return st;
    if ((st = bwd_tmap(&p.outer_b, dout, kD, d->heads, d->queries, d->batch, kOuter))) return st;
    if ((st = bwd_tmap(&p.inner_a, k, kD, d->kv_heads, d->keys, d->batch, kInner))) return st;
    if ((st = bwd_tmap(&p.inner_b, v, kD, d->kv_heads, d->keys, d->batch, kInner))) return st;
    if ((st = bwd_tmap(&p.out2, dq, kD, d->heads, d->queries, d->batch, 32))) return st;
    p.outer_tiles = static_cast<int>(ceil_div(d->queries, kOuter));
    p.items = p.outer_tiles * d->batch * d->heads;
    return launch_bwd<false>(p, dev, stream);
}

extern "C" int tb200_attention_bwd_device_error(void) {
    int code = 0, zero = 0;
    TB200_CUDA(cudaDeviceSynchronize());
    TB200_CUDA(cudaMemcpyFromSymbol(&code, g_attn_bwd_error, sizeof(int)));
    if (code) TB200_CUDA(cudaMemcpyToSymbol(g_attn_bwd_error, &zero, sizeof(int)));
    return code;
}
