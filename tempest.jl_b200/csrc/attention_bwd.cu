// Flash-attention backward for sm_100a, in the reference's two spellings.
//
// Default (`deterministic = false`, src/Compiler/runtime/target.jl:31): ONE kernel over key tiles that keeps dK and
// dV in tensor memory, forms each step's dQ contribution as a product of its own and adds it into a Float32
// workspace by TMA reductions, additions done in L2 (ext/cuTileExt/transpose.jl:165-187, `added_folds` / `add_step!`), and a small
// kernel that rounds the workspace to BFloat16 (`late_kernel`, :201-213).  Five products per step, the algorithmic
// count; the order in which key tiles add into a dQ row is whatever the hardware makes it, so dQ repeats to
// Float32 rounding, not bit for bit.
//
// `deterministic = true`: two kernels, no atomics, every gradient element written once, results repeat bit for
// bit (dQ is a second fold of its own: ext/cuTileExt/build.jl:295-318, docs/src/cuda.md:64-75); seven products.
//
//   stats      delta[m] = sum_d dO[d,m] o[d,m] (o as stored in BFloat16) and lse * log2(e), both negated and both
//              re-laid out [batch][head][query] (rows padded to whole steps) so that consecutive queries are
//              contiguous
//   dK, dV     one item = 128 keys of one (batch, key/value head); steps of 128 queries (of every query
//              head of the group):  S' = K Q', dP' = V dO'  ->  P' = exp2(S' c - lse), dS' = P' (dP' - delta)
//              ->  dK += dS' Q,  dV += P' dO
//   dQ         one item = 128 queries of one (batch, head); steps of 128 keys:
//              S = Q K', dP = dO V'  ->  dS = P (dP - delta)  ->  dQ += dS K
//
// Both run one warp-specialised pipeline.  One thread issues TMA loads: the item's 128-row operands once,
// the steps' operands through two rings (one per operand, so that each tile is released by the last product
// that reads it; see Rings for their depths), and for dK/dV the step's per-query statistics by a bulk copy
// on the dO tile's barrier.  One thread issues tcgen05.mma, every product 128 x 128 x 128, in the order
//      S(t+1),  dK(t), dV(t),  dP(t+1),  S(t+2), ...
// (dQ, which keeps one accumulator and so has room for two dP buffers, issues dP(t+1) with S(t+1)).
// Eight warps own the item's 128 rows (one tensor-memory lane each), four per half of the step's 128
// columns.  A row thread reads its 64 scores, releases the score buffer (so the next scores are computed
// while it works), forms P while the gradient products of the step before run, then reads its 64 dP
// values, forms dS and writes P and dS as packed BFloat16 over the dP columns it has just read; the
// gradient products take them from tensor memory as their A operand and the step's tiles, straight from
// their [position][feature] layout, as MN-major B operands.  Only the read-modify-write of dP sits
// between two products, and the next scores fill that gap.  MMAs of one CTA run in issue order, so dP(t+1)
// cannot overwrite P / dS of step t early.  Accumulators stay in tensor memory for the whole item.
// Work is walked (batch, head)-major with a heavy and a light tile paired per CTA (see Steps).
// Tensor memory: S | dP | two 128-column accumulators = 512 columns.
//
// The one-kernel form is the dK/dV pipeline with one more product per step: dS' (keys x queries), which the row
// threads already hold, is also written to shared memory as [key][query] lines, and dQ' (features x queries) =
// K' (features x keys, the item's K tile read as an MN-major A operand) * dS' lands in the dP columns once the
// step's dK and dV products have read P and dS from them (MMAs of a CTA run in issue order).  The row threads
// read it back at the start of the next step -- lanes are now features -- and only then is the next dP issued into
// those columns.  A warp lays its 32 features of 16 queries side by side in its own 4 KB of the dS' buffer and one
// lane hands them to the TMA unit as a reduction into the Float32 workspace (cp.reduce.async.bulk.tensor ... add);
// the additions run in L2 under the step's products.  Per step the tensor pipe runs  S(t+1) | dK(t) dV(t) dQ(t) | dP(t+1).
// With masks the device holds (a length per sequence, the starts of packed documents per query) a hidden key gets a
// score of -Inf like one the causal mask hides; key tiles beyond the length have no steps.
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
constexpr int kInner = 128;                 // positions per step
constexpr int kD = 128;                     // features
constexpr int kSlab = 128 * 128;            // [128 rows][64 features]: 16 KB
constexpr int kTileBytes = 2 * kSlab;       // one operand tile: 32 KB
// Ring depths.  dK/dV: two stages each.  dQ: the K tile is read by the scores and, three products later, by
// dQ += dS K, so its ring is three deep, and the V tile, free as soon as dP has read it, has one stage.
template <bool DKDV> struct Rings { static constexpr int A = DKDV ? 2 : 3, B = DKDV ? 2 : 1; };
constexpr int kBwdThreads = 320;   // loader, MMA issuer, two groups of four row warps (one per column half)
constexpr int kRowWarps = 8;

__device__ int g_attn_bwd_error = 0;

struct AttnBwdArgs {
    CUtensorMap outer_a, outer_b;   // dK/dV: K, V   | dQ: Q, dO     (boxes of 128 rows)
    CUtensorMap inner_a, inner_b;   // dK/dV: Q, dO  | dQ: K, V      (boxes of 128 rows)
    CUtensorMap out1, out2;         // dK/dV: dV, dK | dQ: -, dQ     (boxes of 32 rows)
    const float *lse2;              // [batch][head][q_pad]  -lse * log2(e)
    const float *delta;             // [batch][head][q_pad]  -delta
    float *dq_acc;                  // one-kernel form: [batch][query][head][feature] Float32, zero before the launch
    CUtensorMap dq_map;             // the same as (feature, head, query, batch), boxes of 32 features x 16 queries
    // masks the device holds (null: none).  A key beyond its sequence's length, or before the start of its query's
    // document, gets a score of -Inf like a key the causal mask hides.
    const int *kv_len;              // [batch]
    const int *doc_start;           // [batch][queries]: the dQ kernel's row threads read their own query's
    const int *starts;              // the same as [batch][head][q_pad] rows, which the dK/dV kernels' row threads read
    const int *start_max;           // the largest start of every 64 queries of such a row: [batch][head][q_pad / 64]
    const int *start_min;           // and the smallest (0x7f7f7f7f where a block has no query)
    int batch, heads, kv_heads, queries, keys;
    int q_pad;                      // queries rounded up to whole steps: rows of the arrays above, zero-filled
    int outer_tiles, supers;
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

// The walk over the work.  A CTA takes whole "supers": the i-th heaviest and the i-th lightest 128-row tile of
// one (batch, head), one after the other (walk step j: super blockIdx.x + (j / 2) gridDim.x, half j % 2).  Under
// the causal mask every super costs the same, so the static round-robin over CTAs is balanced; and supers are
// numbered (batch, head)-major, so the CTAs that run at the same time read the step operands of a few heads
// only and find them in L2 instead of streaming them from HBM once per tile.
//
// Steps: the item of one walk step, and which head and which 128-position chunk its step t reads.
__device__ __forceinline__ int sequence_keys(const AttnBwdArgs &p, int b) {
    if (!p.kv_len) return p.keys;
    const int n = p.kv_len[b];
    return n < 0 ? 0 : (n < p.keys ? n : p.keys);
}

template <bool DKDV>
struct Steps {
    int b, head_outer, tile;   // the item
    int c0, nc, group, count, head_first;
    int keys;                  // the sequence's keys (its length when the device holds lengths)
    bool done, skip;           // past the CTA's last super | second half of a super whose halves are one tile
    __device__ __forceinline__ Steps(const AttnBwdArgs &p, int j) {
        const int half_tiles = (p.outer_tiles + 1) / 2;
        const int sup = blockIdx.x + (j >> 1) * gridDim.x;
        done = sup >= p.supers;
        skip = false;
        count = 0;
        if (done) return;
        const int bh = sup / half_tiles, i = sup % half_tiles;
        const int light = i, heavy_or_light = (j & 1);
        skip = heavy_or_light && (light == p.outer_tiles - 1 - light);
        group = p.heads / p.kv_heads;
        if (DKDV) {
            // the first keys see every query: they are the heavy ones under the causal mask
            tile = heavy_or_light ? p.outer_tiles - 1 - i : i;
            b = bh / p.kv_heads;
            head_outer = bh % p.kv_heads;
            keys = sequence_keys(p, b);
            const int all = (p.queries + kInner - 1) / kInner;
            c0 = p.causal ? (tile * kOuter) / kInner : 0;
            if (c0 > all) c0 = all;
            nc = all - c0;
            if (tile * kOuter >= keys) nc = 0;   // every key of the tile lies beyond the length: zero gradients
            if (p.start_min && nc > 0) {
                // packed documents: the chunks of queries past the last one that can see a key of this tile are left
                // out (a chunk sees none when even its smallest start lies beyond the tile's last key)
                const int *mins = p.start_min + static_cast<long long>(b) * p.heads * (p.q_pad / 64);
                const int last_key = tile * kOuter + kOuter - 1;
                int last = c0 + nc - 1;
                while (last >= c0) {
                    const int lo = min(__ldg(mins + 2 * last), __ldg(mins + 2 * last + 1));
                    if (lo <= last_key) break;
                    last--;
                }
                nc = last - c0 + 1;
            }
            count = nc * group;
            head_first = head_outer * group;
        } else {
            tile = heavy_or_light ? i : p.outer_tiles - 1 - i;
            b = bh / p.heads;
            head_outer = bh % p.heads;
            keys = sequence_keys(p, b);
            const int all = (keys + kInner - 1) / kInner;
            c0 = 0;
            nc = all;
            if (p.causal) {
                const int upto = (tile * kOuter + kOuter - 1) / kInner + 1;
                if (upto < nc) nc = upto;
            }
            if (p.start_min) {
                // packed documents: keys before the smallest start among the tile's queries are hidden from all of them
                const int *mins = p.start_min + static_cast<long long>(b) * p.heads * (p.q_pad / 64);
                const int lo = min(__ldg(mins + 2 * tile), __ldg(mins + 2 * tile + 1));
                const int skip = lo == 0x7f7f7f7f ? 0 : lo / kInner;
                c0 = skip < nc ? skip : nc;
                nc -= c0;
            }
            count = nc;
            head_first = head_outer / group;
        }
    }
    // Where a step is: the walkers keep a cursor and advance it, because a division per step and thread sits
    // squarely on the row warps' critical path.
    struct Cursor {
        int hrel = 0, chunk = 0;   // query head within the group (dK/dV), chunk within the head
    };
    __device__ __forceinline__ void advance(Cursor &k) const {
        if (++k.chunk == nc) {
            k.chunk = 0;
            k.hrel++;
        }
    }
    // head the inner operands of the step belong to, and their first position
    __device__ __forceinline__ void at(const Cursor &k, int &head_inner, int &pos0) const {
        head_inner = head_first + k.hrel;   // dQ: one pass over the chunks, hrel stays 0
        pos0 = (c0 + k.chunk) * kInner;
    }
};

// MODE 0: dQ of the deterministic form; 1: its dK / dV; 2: the one-kernel form (dK, dV, and dQ by atomic adds).
template <int MODE>
__global__ void __launch_bounds__(kBwdThreads, 1) attention_bwd_kernel(const __grid_constant__ AttnBwdArgs p) {
    constexpr bool DKDV = MODE != 0, ATOMIC = MODE == 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *s_outer_a = smem;
    uint8_t *s_outer_b = s_outer_a + kTileBytes;
    constexpr int SA = Rings<DKDV>::A, SB = Rings<DKDV>::B;
    uint8_t *s_ring_a = s_outer_b + kTileBytes;          // SA x 32 KB
    uint8_t *s_ring_b = s_ring_a + SA * kTileBytes;      // SB x 32 KB
    uint8_t *s_out = s_ring_b + SB * kTileBytes;         // 2 x 16 KB: one slab per group, stages the stores
    // one-kernel form: the step's dS' as [key][query] lines, one 64-query slab per group; each row warp writes and
    // later stages in its own 32 rows of its group's slab only, and the item's last dQ product has read the lines
    // before the item's results are staged, so the two uses share the buffer
    uint8_t *s_ds = s_out;

    __shared__ __align__(8) uint64_t outer_full, outer_empty, acc_done, acc_free;
    __shared__ __align__(8) uint64_t a_full[SA], a_empty[SA], b_full[SB], b_empty[SB];
    __shared__ __align__(8) uint64_t s_full;            // the step's scores are in tensor memory
    __shared__ __align__(8) uint64_t dp_full[2];        // its dP is (by step parity: dQ computes dP a step ahead)
    __shared__ __align__(8) uint64_t s_read;            // every row warp holds its scores in registers
    // every row warp has written P and dS; by step parity, because the dQ kernel's row warps may finish step
    // t + 1 (its scores and dP are issued ahead) before the issuing thread has looked at step t
    __shared__ __align__(8) uint64_t pds_full[2];
    __shared__ __align__(8) uint64_t dq_full;           // one-kernel form: the step's dQ' is in the dP columns
    __shared__ __align__(8) uint64_t x1_free;           // every row warp has read it: the next dP may be issued
    __shared__ uint32_t tmem_base_smem;
    __shared__ int failed_smem;
    // dK/dV: the step's 128 queries' lse*log2(e) [0, 128) and delta [128, 256), one buffer per stage of the dO ring:
    // the loading thread copies them with the dO tile and they complete on the same barrier
    __shared__ __align__(16) float col_stats[Rings<true>::B][2 * kInner];
    volatile int *failed = &failed_smem;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        failed_smem = 0;
        mbar_init(&outer_full, 1); mbar_init(&outer_empty, 1); mbar_init(&acc_done, 1); mbar_init(&acc_free, kRowWarps);
        for (int s = 0; s < SA; s++) { mbar_init(&a_full[s], 1); mbar_init(&a_empty[s], 1); }
        for (int s = 0; s < SB; s++) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
        mbar_init(&s_full, 1); mbar_init(&dp_full[0], 1); mbar_init(&dp_full[1], 1);
        mbar_init(&s_read, kRowWarps); mbar_init(&pds_full[0], kRowWarps); mbar_init(&pds_full[1], kRowWarps);
        mbar_init(&dq_full, 1); mbar_init(&x1_free, kRowWarps);
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
    const uint32_t tmem_s = tmem_base, tmem_dp = tmem_base + 128;
    const uint32_t tmem_acc1 = tmem_base + 256, tmem_acc2 = tmem_base + 384;

    if (warp == 0) {
        if (elect_one()) {
            uint32_t outer_phase = 0, c = 0;
            for (int j = 0; !*failed; j++) {
                const Steps<DKDV> steps(p, j);
                if (steps.done) break;
                if (steps.skip) continue;
                if (!bwd_wait(&outer_empty, outer_phase ^ 1, failed, 1)) break;
                outer_phase ^= 1;
                mbar_arrive_expect_tx(&outer_full, 2 * kTileBytes);
                const int r0 = steps.tile * kOuter;
                tma_load_4d(s_outer_a, &p.outer_a, &outer_full, 0, steps.head_outer, r0, steps.b);
                tma_load_4d(s_outer_a + kSlab, &p.outer_a, &outer_full, 64, steps.head_outer, r0, steps.b);
                tma_load_4d(s_outer_b, &p.outer_b, &outer_full, 0, steps.head_outer, r0, steps.b);
                tma_load_4d(s_outer_b + kSlab, &p.outer_b, &outer_full, 64, steps.head_outer, r0, steps.b);
                bool ok = true;
                typename Steps<DKDV>::Cursor cur;
                for (int t = 0; t < steps.count; t++, c++) {
                    const int sta = c % SA, stb = c % SB;
                    int hi, pos0;
                    steps.at(cur, hi, pos0);
                    steps.advance(cur);
                    if (!bwd_wait(&a_empty[sta], ((c / SA) & 1) ^ 1, failed, 2)) { ok = false; break; }
                    uint8_t *sa = s_ring_a + sta * kTileBytes;
                    mbar_arrive_expect_tx(&a_full[sta], kTileBytes);
                    tma_load_4d(sa, &p.inner_a, &a_full[sta], 0, hi, pos0, steps.b);
                    tma_load_4d(sa + kSlab, &p.inner_a, &a_full[sta], 64, hi, pos0, steps.b);
                    if (!bwd_wait(&b_empty[stb], ((c / SB) & 1) ^ 1, failed, 13)) { ok = false; break; }
                    uint8_t *sb = s_ring_b + stb * kTileBytes;
                    mbar_arrive_expect_tx(&b_full[stb], kTileBytes + (DKDV ? 2 * kInner * 4 : 0));
                    if (DKDV) {
                        const long long at = (static_cast<long long>(steps.b) * p.heads + hi) * p.q_pad + pos0;
                        bulk_load(&col_stats[stb][0], p.lse2 + at, kInner * 4, &b_full[stb]);
                        bulk_load(&col_stats[stb][kInner], p.delta + at, kInner * 4, &b_full[stb]);
                    }
                    tma_load_4d(sb, &p.inner_b, &b_full[stb], 0, hi, pos0, steps.b);
                    tma_load_4d(sb + kSlab, &p.inner_b, &b_full[stb], 64, hi, pos0, steps.b);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc_t = umma_idesc_bf16(kOuter, kInner, false, false);   // scores: both K-major
            const uint32_t idesc_g = umma_idesc_bf16(kOuter, kD, false, true);        // gradients: B MN-major
            const uint32_t idesc_q = umma_idesc_bf16(kD, kInner, true, true);         // dQ' = K' dS': both MN-major
            const uint32_t ds_smem = smem_u32(s_ds);
            const uint32_t oa = smem_u32(s_outer_a), ob = smem_u32(s_outer_b);
            uint32_t outer_phase = 0, c0 = 0, item_count = 0;
            bool ok = true;
            // scores of step c (a count over all of this CTA's steps) into the score columns
            auto issue_scores = [&](uint32_t c) -> bool {
                // the row warps must hold the scores of the step before in registers
                if (c > 0 && !bwd_wait(&s_read, (c - 1) & 1, failed, 5)) return false;
                const int st = c % SA;
                if (!bwd_wait(&a_full[st], (c / SA) & 1, failed, 4)) return false;
                tcgen05_fence_after();
                const uint32_t ia = smem_u32(s_ring_a + st * kTileBytes);
#pragma unroll
                for (int k = 0; k < kD / 16; k++) {
                    const uint32_t off = (k >> 2) * kSlab + (k & 3) * 32;
                    tcgen05_mma_f16(tmem_s, umma_smem_desc(oa + off, 16, 1024), umma_smem_desc(ia + off, 16, 1024),
                                    idesc_t, k != 0);
                }
                tcgen05_commit(&s_full);
                return true;
            };
            // dP of step c.  dK/dV: one buffer; dP runs after the gradient products issued before it, which read
            // P / dS of the step before from the same columns.  dQ has room for two buffers (it keeps one
            // accumulator), so dP of step c is issued with the scores, before the gradient product of step c - 1.
            auto issue_dp = [&](uint32_t c) -> bool {
                const int st = c % SB;
                // one-kernel form: the dQ' of the step before sits in these columns until the row warps have read it
                if (ATOMIC && c > 0 && !bwd_wait(&x1_free, (c - 1) & 1, failed, 15)) return false;
                if (!bwd_wait(&b_full[st], (c / SB) & 1, failed, 14)) return false;
                tcgen05_fence_after();
                const uint32_t ib = smem_u32(s_ring_b + st * kTileBytes);
#pragma unroll
                for (int k = 0; k < kD / 16; k++) {
                    const uint32_t off = (k >> 2) * kSlab + (k & 3) * 32;
                    tcgen05_mma_f16(tmem_dp + (DKDV ? 0 : (c & 1) * 128), umma_smem_desc(ob + off, 16, 1024),
                                    umma_smem_desc(ib + off, 16, 1024), idesc_t, k != 0);
                }
                tcgen05_commit(&dp_full[c & 1]);
                if (!DKDV) tcgen05_commit(&b_empty[st]);   // dQ: nothing else reads the step's V tile
                return true;
            };
            for (int j = 0; !*failed && ok; j++) {
                const Steps<DKDV> steps(p, j);
                if (steps.done) break;
                if (steps.skip) continue;
                if (!bwd_wait(&outer_full, outer_phase, failed, 3)) break;
                outer_phase ^= 1;
                tcgen05_fence_after();
                if (steps.count == 0) {   // nothing reads the item's operands
                    mbar_arrive(&outer_empty);
                    continue;
                }
                if (!issue_scores(c0) || !issue_dp(c0)) break;
                if (!ATOMIC && steps.count == 1) tcgen05_commit(&outer_empty);
                for (int t = 0; t < steps.count; t++) {
                    const uint32_t c = c0 + t;
                    const int sta = c % SA, stb = c % SB;
                    if (t + 1 < steps.count) {
                        if (!issue_scores(c + 1)) { ok = false; break; }
                        if (!DKDV) {
                            if (!issue_dp(c + 1)) { ok = false; break; }
                            if (t + 2 == steps.count) tcgen05_commit(&outer_empty);
                        }
                    }
                    // the first gradient product of an item overwrites the accumulators
                    if (t == 0 && !bwd_wait(&acc_free, (item_count & 1) ^ 1, failed, 6)) { ok = false; break; }
                    if (!bwd_wait(&pds_full[c & 1], (c >> 1) & 1, failed, 7)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t ia = smem_u32(s_ring_a + sta * kTileBytes);
                    const uint32_t ib = smem_u32(s_ring_b + stb * kTileBytes);
                    // A: P / dS from tensor memory, 16 positions = 8 packed columns per MMA, where the row threads of
                    // each column half left them (P in the first 32 of the half's 64 dP columns, dS in the last 32);
                    // B: 16 position lines of 128 bytes per 64-feature slab
#pragma unroll
                    for (int k = 0; k < kInner / 16; k++) {
                        const uint32_t ds_at = tmem_dp + (DKDV ? 0 : (c & 1) * 128) + (k >> 2) * 64 + 32 + (k & 3) * 8;
                        tcgen05_mma_f16_ts(tmem_acc2, ds_at, umma_smem_desc(ia + k * 2048, kSlab, 1024), idesc_g, t | k);
                    }
                    tcgen05_commit(&a_empty[sta]);
                    if (DKDV) {
#pragma unroll
                        for (int k = 0; k < kInner / 16; k++) {
                            const uint32_t p_at = tmem_dp + (k >> 2) * 64 + (k & 3) * 8;
                            tcgen05_mma_f16_ts(tmem_acc1, p_at, umma_smem_desc(ib + k * 2048, kSlab, 1024), idesc_g, t | k);
                        }
                        tcgen05_commit(&b_empty[stb]);
                    }
                    if (ATOMIC) {
                        // dQ' (features x queries) = K' dS': A = the item's K tile, a line of 64 features per key
                        // and slab; B = the dS' lines the row threads wrote, a line of 64 queries per key and slab
#pragma unroll
                        for (int k = 0; k < kOuter / 16; k++)
                            tcgen05_mma_f16(tmem_dp, umma_smem_desc(oa + k * 2048, kSlab, 1024),
                                            umma_smem_desc(ds_smem + k * 2048, kSlab, 1024), idesc_q, k != 0);
                        tcgen05_commit(&dq_full);
                        if (t + 1 == steps.count) tcgen05_commit(&outer_empty);   // the last reader of the item's K
                    }
                    if (DKDV && t + 1 < steps.count) {
                        if (!issue_dp(c + 1)) { ok = false; break; }
                        if (!ATOMIC && t + 2 == steps.count) tcgen05_commit(&outer_empty);
                    }
                    if (t + 1 == steps.count) tcgen05_commit(&acc_done);
                }
                c0 += steps.count;
                item_count++;   // items that ran gradient products
            }
        }
    } else {
        // ---- one thread per (row of the item, half of the step's columns)
        const int q4 = warp & 3;
        const int group = (warp - 2) >> 2;
        const int row = q4 * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
        const uint32_t t_s = tmem_s + lane_base + group * 64;     // this thread's 64 scores
        const uint32_t t_dp0 = tmem_dp + lane_base + group * 64;  // its 64 dP values; P and dS go over them
        uint32_t c = 0, item_count = 0;
        for (int j = 0;; j++) {
            const Steps<DKDV> steps(p, j);
            if (steps.done) break;
            if (steps.skip) continue;
            const int outer_pos = steps.tile * kOuter + row;   // this thread's key (dK/dV) or query (dQ)
            float row_lse2 = 0.0f, row_delta = 0.0f;
            int row_start = 0;   // dQ: the first key this thread's query sees (packed documents)
            if (!DKDV && outer_pos < p.queries) {
                const long long i = (static_cast<long long>(steps.b) * p.heads + steps.head_outer) * p.q_pad + outer_pos;
                row_lse2 = p.lse2[i];
                row_delta = p.delta[i];
                if (p.doc_start) row_start = p.doc_start[static_cast<long long>(steps.b) * p.queries + outer_pos];
            }
            bool ok = true;
            typename Steps<DKDV>::Cursor cur;
            // One-kernel form: the dQ' of the step before, read out of the dP columns (lanes are features here, so
            // `row` is this thread's feature) and added into the Float32 workspace: 32 consecutive features of one
            // query per warp instruction.  The columns are handed back before the adds are issued.
            int prev_hi = 0, prev_pos0 = 0;
            bool dq_pending = false;   // a reduction may still be reading this warp's part of the slab
            // before that part is written for anything else
            auto slab_free = [&]() {
                if (!dq_pending) return;
                if (lane == 0) bulk_wait_group_read<0>();
                __syncwarp();
                dq_pending = false;
            };
            auto add_dq = [&](uint32_t step) -> bool {
                if (!bwd_wait(&dq_full, step & 1, failed, 16)) return false;
                tcgen05_fence_after();
                uint32_t dq[64];
                tmem_ld_32x32(t_dp0, *reinterpret_cast<uint32_t(*)[32]>(&dq[0]));
                tmem_ld_32x32(t_dp0 + 32, *reinterpret_cast<uint32_t(*)[32]>(&dq[32]));
                tmem_ld_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&x1_free);
                // Added into the Float32 workspace by the TMA unit, not by this thread: the warp lays its 32 features of
                // 16 queries side by side, [query][feature], in its own 4 KB of the dS' slab (the bytes only this warp
                // writes, free now that the dQ' product which read them is complete, written again later in this
                // step) and one lane hands them over as a reduction; two halves of 2 KB take turns, so a round waits
                // only for the reduction two rounds back.  The additions happen in L2 while the step goes on.
                uint8_t *mine = s_ds + group * kSlab + q4 * 4096;
                const int q0 = prev_pos0 + group * 64;
#pragma unroll
                for (int round = 0; round < 4; round++) {
                    if (lane == 0) bulk_wait_group_read<1>();
                    __syncwarp();
                    float *stage = reinterpret_cast<float *>(mine + (round & 1) * 2048);
#pragma unroll
                    for (int i = 0; i < 16; i++) stage[i * 32 + lane] = __uint_as_float(dq[16 * round + i]);
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        // queries past the end: nothing to add, but the (empty) group keeps the count of rounds
                        if (q0 + 16 * round < p.queries)
                            tma_reduce_add_4d(&p.dq_map, stage, q4 * 32, prev_hi, q0 + 16 * round, steps.b);
                        bulk_commit_group();
                    }
                }
                dq_pending = true;
                return true;
            };
            for (int t = 0; t < steps.count; t++, c++) {
                const uint32_t ph = c & 1;
                int hi, pos0;
                steps.at(cur, hi, pos0);
                steps.advance(cur);   // cur is now the next step's
                const int col0 = pos0 + group * 64;   // first position of this thread's columns
                // dK/dV: the statistics of the step's queries are per column; they arrived in shared memory with the
                // step's dO tile (the wait is for a barrier that completed long ago: the issuing thread needed it first)
                const float *stats = col_stats[c % SB] + group * 64;
                if (DKDV && !bwd_wait(&b_full[c % SB], (c / SB) & 1, failed, 12)) { ok = false; break; }
                if (!bwd_wait(&s_full, ph, failed, 8)) { ok = false; break; }
                tcgen05_fence_after();
                uint32_t s[64];
                tmem_ld_32x32(t_s, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
                tmem_ld_32x32(t_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
                tmem_ld_wait();
                // the scores are in registers: the next step's may be computed
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_read);
                // packed documents: the per-element test only where a start can hide a key -- dK/dV: the largest start
                // among the step's 64 queries lies beyond the tile's first key; dQ: this query's start lies beyond the
                // step's first key
                bool doc_edge = false;
                if (p.doc_start) {
                    if (DKDV)
                        doc_edge = __ldg(p.start_max + ((static_cast<long long>(steps.b) * p.heads + hi) * p.q_pad + col0) / 64) >
                                   steps.tile * kOuter;
                    else
                        doc_edge = row_start > col0;
                }
                const bool edge = doc_edge ||
                                  (DKDV ? (pos0 + kInner > p.queries || outer_pos >= steps.keys ||
                                           (p.causal && pos0 < steps.tile * kOuter + kOuter))
                                        : (pos0 + kInner > steps.keys || outer_pos >= p.queries ||
                                           (p.causal && pos0 + kInner - 1 > steps.tile * kOuter)));
                if (edge) {
                    // masked positions get a score of -Inf: their weight and their dS are then exactly zero
                    // dK/dV: the starts of the step's queries, the same 64 for every thread of the group (L1 hands them out)
                    const int4 *starts = reinterpret_cast<const int4 *>(
                        p.starts + (static_cast<long long>(steps.b) * p.heads + hi) * p.q_pad + col0);
#pragma unroll
                    for (int i = 0; i < 64; i++) {
                        const int inner_pos = col0 + i;
                        const int key = DKDV ? outer_pos : inner_pos;
                        const int query = DKDV ? inner_pos : outer_pos;
                        int first = 0;
                        if (p.doc_start) {
                            if (DKDV) {
                                const int4 q4s = __ldg(starts + (i >> 2));
                                first = (i & 3) == 0 ? q4s.x : (i & 3) == 1 ? q4s.y : (i & 3) == 2 ? q4s.z : q4s.w;
                            } else {
                                first = row_start;
                            }
                        }
                        if (key >= steps.keys || query >= p.queries || (p.causal && key > query) || key < first)
                            s[i] = 0xff800000u;
                    }
                }
                // P.  dQ keeps it in Float32 for dS.  dK/dV rounds it to BFloat16 here -- P' feeds dV += P' dO in that
                // precision anyway, the conversions issue in the shadow of the exponentials (this stretch waits on the
                // special-function unit), and dS is then formed from the rounded weights: half the registers, which
                // is what keeps this kernel's row threads from spilling.
                // (two scores at a time: the scaling and the shift by the negated log-sum-exp are one packed multiply-add)
                uint32_t pk[32];
                const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
#pragma unroll
                for (int g = 0; g < 16; g++) {
                    float4 l4 = make_float4(row_lse2, row_lse2, row_lse2, row_lse2);
                    if (DKDV) l4 = *reinterpret_cast<const float4 *>(stats + 4 * g);
                    const float2 x01 = __ffma2_rn(make_float2(__uint_as_float(s[4 * g]), __uint_as_float(s[4 * g + 1])), scale2,
                                                  make_float2(l4.x, l4.y));
                    const float2 x23 = __ffma2_rn(make_float2(__uint_as_float(s[4 * g + 2]), __uint_as_float(s[4 * g + 3])), scale2,
                                                  make_float2(l4.z, l4.w));
                    const float p0 = fast_exp2(x01.x), p1 = fast_exp2(x01.y), p2 = fast_exp2(x23.x), p3 = fast_exp2(x23.y);
                    if (DKDV) {
                        pk[2 * g] = pack_bf16x2(p0, p1);
                        pk[2 * g + 1] = pack_bf16x2(p2, p3);
                    } else {
                        s[4 * g] = __float_as_uint(p0); s[4 * g + 1] = __float_as_uint(p1);
                        s[4 * g + 2] = __float_as_uint(p2); s[4 * g + 3] = __float_as_uint(p3);
                    }
                }
                if (ATOMIC) {
                    if (t > 0 && !add_dq(c - 1)) { ok = false; break; }
                    prev_hi = hi;
                    prev_pos0 = pos0;
                }
                if (!bwd_wait(&dp_full[ph], (c >> 1) & 1, failed, 9)) { ok = false; break; }
                const uint32_t t_dp = t_dp0 + (DKDV ? 0 : ph * 128);
                tcgen05_fence_after();
                // dS = P (dP - delta), packed two per column, in two halves of 32 columns: the first half's columns
                // take P as soon as they are read, the second half's take dS
                uint32_t dp[32], dk[32];
                tmem_ld_32x32(t_dp, dp);
                tmem_ld_wait();
                if (DKDV) tmem_st_32x32(t_dp, pk);
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    if (half == 1) {
                        tmem_ld_32x32(t_dp + 32, dp);
                        tmem_ld_wait();
                    }
#pragma unroll
                    for (int g = 0; g < 8; g++) {
                        const int i = 32 * half + 4 * g;
                        float4 d4 = make_float4(row_delta, row_delta, row_delta, row_delta);
                        if (DKDV) d4 = *reinterpret_cast<const float4 *>(stats + kInner + i);
                        float p0, p1, p2, p3;
                        if (DKDV) {
                            unpack_bf16x2(pk[i / 2], p0, p1);
                            unpack_bf16x2(pk[i / 2 + 1], p2, p3);
                        } else {
                            p0 = __uint_as_float(s[i]); p1 = __uint_as_float(s[i + 1]);
                            p2 = __uint_as_float(s[i + 2]); p3 = __uint_as_float(s[i + 3]);
                        }
                        const float2 e01 = __fmul2_rn(make_float2(p0, p1),
                                                      __fadd2_rn(make_float2(__uint_as_float(dp[4 * g]), __uint_as_float(dp[4 * g + 1])),
                                                                 make_float2(d4.x, d4.y)));
                        const float2 e23 = __fmul2_rn(make_float2(p2, p3),
                                                      __fadd2_rn(make_float2(__uint_as_float(dp[4 * g + 2]), __uint_as_float(dp[4 * g + 3])),
                                                                 make_float2(d4.z, d4.w)));
                        dk[16 * half + 2 * g] = pack_bf16x2(e01.x, e01.y);
                        dk[16 * half + 2 * g + 1] = pack_bf16x2(e23.x, e23.y);
                    }
                }
                tmem_st_32x32(t_dp + 32, dk);
                if (ATOMIC) {
                    // the same dS' as this key's line of its group's slab (64 queries = 128 bytes, 16-byte chunks
                    // swizzled by the row as the tensor core expects), for the dQ' product
                    slab_free();
                    uint8_t *line = s_ds + group * kSlab + row * 128;
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        *reinterpret_cast<uint4 *>(line + ((j ^ (row & 7)) << 4)) =
                            make_uint4(dk[4 * j], dk[4 * j + 1], dk[4 * j + 2], dk[4 * j + 3]);
                    fence_proxy_async();
                }
                tmem_st_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&pds_full[ph]);
            }
            if (!ok) break;
            if (ATOMIC && steps.count > 0 && !add_dq(c - 1)) break;   // the item's last step
            if (ATOMIC) slab_free();   // the staging below uses the same memory
            // ---- the item's gradients: accumulators -> BFloat16 -> shared staging -> TMA stores.
            // dK/dV: group 0 writes dV, group 1 dK, one 64-feature slab at a time; dQ: each group one slab.
            if (steps.count > 0) {
                if (!bwd_wait(&acc_done, item_count & 1, failed, 10)) break;
            }
            tcgen05_fence_after();
            const int rounds = DKDV ? 2 : 1;
            const uint32_t acc = (DKDV && group == 0) ? tmem_acc1 : tmem_acc2;
            const float mul = (DKDV && group == 0) ? 1.0f : p.scale;
            uint8_t *stage = s_out + group * kSlab;   // [128 rows][64 features], this warp's 32 rows of it
#pragma unroll 1
            for (int round = 0; round < rounds; round++) {
                const int f0 = DKDV ? round * 64 : group * 64;
                uint32_t r[64];
                if (steps.count > 0) {
                    tmem_ld_32x32(acc + lane_base + f0, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                    tmem_ld_32x32(acc + lane_base + f0 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
                    tmem_ld_wait();
                    if (round == rounds - 1) {   // this warp has read all it needs of the accumulators
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_free);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 64; i++) r[i] = 0u;   // no step touched this item: its gradient is zero
                }
#pragma unroll
                for (int g = 0; g < 8; g++) {
                    uint4 v4;
                    v4.x = pack_bf16x2(__uint_as_float(r[8 * g]) * mul, __uint_as_float(r[8 * g + 1]) * mul);
                    v4.y = pack_bf16x2(__uint_as_float(r[8 * g + 2]) * mul, __uint_as_float(r[8 * g + 3]) * mul);
                    v4.z = pack_bf16x2(__uint_as_float(r[8 * g + 4]) * mul, __uint_as_float(r[8 * g + 5]) * mul);
                    v4.w = pack_bf16x2(__uint_as_float(r[8 * g + 6]) * mul, __uint_as_float(r[8 * g + 7]) * mul);
                    *reinterpret_cast<uint4 *>(stage + row * 128 + ((g ^ (row & 7)) << 4)) = v4;
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    const int r0 = steps.tile * kOuter + q4 * 32;
                    tma_store_4d((DKDV && group == 0) ? &p.out1 : &p.out2, stage + q4 * 32 * 128, f0, steps.head_outer, r0,
                                 steps.b);
                    bulk_commit_group();
                    bulk_wait_group_read<0>();   // the staging rows may be rewritten
                }
                __syncwarp();
            }
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

// delta[b][h][m] = sum_d dO o ; lse2[b][h][m] = lse[b][m][h] * log2(e), rows of q_pad entries.  16 threads per (b, m, h) row.
__global__ void __launch_bounds__(256) attention_stats_kernel(const __nv_bfloat16 *o, const __nv_bfloat16 *dout,
                                                              const float *lse, float *lse2, float *delta, int batch,
                                                              int heads, int queries, int q_pad, int d,
                                                              const int *doc_start, int *starts, int *start_max,
                                                              int *start_min) {
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
        const long long out = (b * heads + h) * q_pad + m;
        // both negated: the row threads add them with packed (two at a time) instructions, which have no negate
        delta[out] = -s;
        // a query that saw no key has a log-sum-exp of -Inf: its weights are zero whatever the scores (a finite huge
        // shift instead of the infinite one, which would meet the masked scores' -Inf as NaN)
        const float l = lse[r];
        lse2[out] = l == -INFINITY ? -1.0e30f : -l * kLog2e;
        if (starts) {
            const int first = doc_start[b * queries + m];
            starts[out] = first;
            atomicMax(start_max + out / 64, first);   // zero before the launch; starts are not negative
            atomicMin(start_min + out / 64, first);   // 0x7f7f7f7f before the launch
        }
    }
}

// The one-kernel form's second launch: dq = BFloat16(scale * accumulated Float32) (the reference's `late_kernel`,
// ext/cuTileExt/transpose.jl:201-213).  Eight elements a thread.
__global__ void __launch_bounds__(256) attention_dq_round_kernel(const float4 *acc, uint4 *dq, long long vectors, float scale) {
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < vectors; i += gridDim.x * 256ll) {
        const float4 a = __ldcs(acc + 2 * i), b = __ldcs(acc + 2 * i + 1);
        __stcs(dq + i, make_uint4(pack_bf16x2(a.x * scale, a.y * scale), pack_bf16x2(a.z * scale, a.w * scale),
                                  pack_bf16x2(b.x * scale, b.y * scale), pack_bf16x2(b.z * scale, b.w * scale)));
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

template <int MODE>
int launch_bwd(AttnBwdArgs &p, const DeviceInfo &dev, cudaStream_t stream) {
    constexpr bool DKDV = MODE != 0;
    // the tiles (224 KB, 1024-byte aligned) sit behind the kernel's static shared memory: take all the dynamic
    // shared memory the SM has left
    const size_t tiles = 2 * kTileBytes + (Rings<DKDV>::A + Rings<DKDV>::B) * kTileBytes + 2 * kSlab;
    static std::mutex lock;
    static size_t dynamic_bytes[64] = {};
    {
        std::lock_guard<std::mutex> hold(lock);
        if (!dynamic_bytes[dev.device]) {
            cudaFuncAttributes attr;
            TB200_CUDA(cudaFuncGetAttributes(&attr, attention_bwd_kernel<MODE>));
            const size_t first = (attr.sharedSizeBytes + 1023) / 1024 * 1024;
            if (first + tiles > dev.smem_optin) return TB200_ERR_UNSUPPORTED;
            const size_t room = dev.smem_optin - attr.sharedSizeBytes;
            TB200_CUDA(cudaFuncSetAttribute(attention_bwd_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(room)));
            dynamic_bytes[dev.device] = room;
        }
    }
    const size_t smem = dynamic_bytes[dev.device];
    const unsigned grid = static_cast<unsigned>(p.supers < dev.sms ? p.supers : dev.sms);
    attention_bwd_kernel<MODE><<<grid, kBwdThreads, smem, stream>>>(p);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

}  // namespace
}  // namespace tb200

using namespace tb200;

namespace {
size_t bwd_stat_bytes(const tb200_attn_desc *d) {
    const size_t q_pad = (static_cast<size_t>(d->queries) + kInner - 1) / kInner * kInner;
    return (static_cast<size_t>(2) * d->batch * d->heads * q_pad * sizeof(float) + 255) / 256 * 256;
}
}  // namespace

// The per-query statistics, and for the one-kernel form on the tensor-core path the Float32 dQ accumulator.
extern "C" size_t tb200_attention_bwd_workspace_bytes(const tb200_attn_desc *d) {
    if (!d || d->batch <= 0 || d->heads <= 0 || d->queries <= 0) return 0;
    size_t bytes = bwd_stat_bytes(d);
    if (!d->deterministic && attention_tensor_geometry(d))
        bytes += static_cast<size_t>(d->batch) * d->queries * d->heads * kD * sizeof(float);
    return bytes;
}

namespace {
// a row of starts per (batch, head), and behind them the largest and the smallest start of every 64 queries
size_t bwd_start_row_bytes(const tb200_attn_desc *d) {
    const size_t q_pad = (static_cast<size_t>(d->queries) + kInner - 1) / kInner * kInner;
    return (static_cast<size_t>(d->batch) * d->heads * q_pad * sizeof(int) + 255) / 256 * 256;
}
size_t bwd_start_block_bytes(const tb200_attn_desc *d) {
    const size_t q_pad = (static_cast<size_t>(d->queries) + kInner - 1) / kInner * kInner;
    return (static_cast<size_t>(d->batch) * d->heads * (q_pad / 64) * sizeof(int) + 255) / 256 * 256;
}
size_t bwd_start_bytes(const tb200_attn_desc *d) {
    const size_t q_pad = (static_cast<size_t>(d->queries) + kInner - 1) / kInner * kInner;
    return bwd_start_row_bytes(d) + 2 * bwd_start_block_bytes(d);
}
int bwd_run(const tb200_attn_desc *d, const tb200_attn_mask *mask, const void *q, const void *k, const void *v, const void *o,
            const float *lse, const void *dout, void *dq, void *dk, void *dv, void *workspace, size_t workspace_bytes,
            void *stream_);
}  // namespace

extern "C" int tb200_attention_bwd(const tb200_attn_desc *d, const void *q, const void *k, const void *v,
                                   const void *o, const float *lse, const void *dout, void *dq, void *dk, void *dv,
                                   void *workspace, size_t workspace_bytes, void *stream_) {
    return bwd_run(d, nullptr, q, k, v, o, lse, dout, dq, dk, dv, workspace, workspace_bytes, stream_);
}

// The pullback with masks the device holds, on the tensor cores: 128 features, dense arrays (a mask with strides, or
// another head dimension: TB200_ERR_UNSUPPORTED -- tb200_attention_bwd_masked takes those).  The workspace is
// tb200_attention_bwd's plus one row of starts per (batch, head) when documents are packed.
extern "C" size_t tb200_attention_bwd_masked_workspace_bytes(const tb200_attn_desc *d) {
    const size_t base = tb200_attention_bwd_workspace_bytes(d);
    return base ? base + bwd_start_bytes(d) : 0;
}

extern "C" int tb200_attention_bwd_masked_ws(const tb200_attn_desc *d, const tb200_attn_mask *mask, const void *q, const void *k,
                                             const void *v, const void *o, const float *lse, const void *dout, void *dq,
                                             void *dk, void *dv, void *workspace, size_t workspace_bytes, void *stream_) {
    if (!d) return TB200_ERR_NULL;
    if (!attention_tensor_geometry(d)) return TB200_ERR_UNSUPPORTED;
    if (mask)
        for (int i = 0; i < 3; i++)
            if (mask->q_stride[i] || mask->kv_stride[i]) return TB200_ERR_UNSUPPORTED;
    if (workspace_bytes < tb200_attention_bwd_masked_workspace_bytes(d)) return TB200_ERR_WORKSPACE;
    return bwd_run(d, mask, q, k, v, o, lse, dout, dq, dk, dv, workspace, workspace_bytes, stream_);
}

namespace {
int bwd_run(const tb200_attn_desc *d, const tb200_attn_mask *mask, const void *q, const void *k, const void *v, const void *o,
            const float *lse, const void *dout, void *dq, void *dk, void *dv, void *workspace, size_t workspace_bytes,
            void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!d) return TB200_ERR_NULL;
    if (d->batch < 0 || d->heads <= 0 || d->kv_heads <= 0 || d->queries < 0 || d->keys < 0 || d->head_dim <= 0)
        return TB200_ERR_SHAPE;
    if (d->heads % d->kv_heads != 0 || !(d->scale > 0.0f)) return TB200_ERR_SHAPE;
    if (d->causal && d->queries != d->keys) return TB200_ERR_SHAPE;
    if (d->dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (!attention_tensor_geometry(d) && !attention_simt_takes(d)) return TB200_ERR_UNSUPPORTED;
    if (d->batch == 0 || (d->queries == 0 && d->keys == 0)) return TB200_OK;
    if (d->queries == 0 || d->keys == 0) return TB200_ERR_UNSUPPORTED;
    if (!q || !k || !v || !o || !lse || !dout || !dq || !dk || !dv) return TB200_ERR_NULL;
    for (const void *ptr : {q, k, v, o, dout, static_cast<const void *>(dq), static_cast<const void *>(dk),
                            static_cast<const void *>(dv)})
        if (!aligned_to(ptr, 16)) return TB200_ERR_ALIGN;
    if (!aligned_to(lse, 4)) return TB200_ERR_ALIGN;
    const size_t need = tb200_attention_bwd_workspace_bytes(d);
    if (!workspace || workspace_bytes < need || !aligned_to(workspace, 16)) return TB200_ERR_WORKSPACE;
    if (!attention_tensor_geometry(d)) return attention_simt_bwd(d, q, k, v, o, lse, dout, dq, dk, dv, stream);
    DeviceInfo dev;
    int st = current_device(&dev);
    if (st) return st;

    const int q_pad = (d->queries + kInner - 1) / kInner * kInner;
    const long long stat_len = static_cast<long long>(d->batch) * d->heads * q_pad;
    float *lse2 = static_cast<float *>(workspace);
    float *delta = lse2 + stat_len;
    // packed documents: the starts again as rows per (batch, head), behind everything else in the workspace
    const int *doc_start = mask ? mask->doc_start : nullptr;
    int *starts = doc_start ? reinterpret_cast<int *>(static_cast<uint8_t *>(workspace) + tb200_attention_bwd_workspace_bytes(d))
                            : nullptr;
    int *start_max = doc_start ? reinterpret_cast<int *>(reinterpret_cast<uint8_t *>(starts) + bwd_start_row_bytes(d)) : nullptr;
    int *start_min = doc_start ? reinterpret_cast<int *>(reinterpret_cast<uint8_t *>(start_max) + bwd_start_block_bytes(d)) : nullptr;
    {
        if (q_pad != d->queries) TB200_CUDA(cudaMemsetAsync(workspace, 0, bwd_stat_bytes(d), stream));   // the pads are read
        const long long threads = static_cast<long long>(d->batch) * d->heads * d->queries * 16;
        const unsigned blocks = static_cast<unsigned>(ceil_div(threads, 256));
        if (doc_start) {   // pads and maxima start at zero, minima at 0x7f7f7f7f
            TB200_CUDA(cudaMemsetAsync(starts, 0, bwd_start_row_bytes(d) + bwd_start_block_bytes(d), stream));
            TB200_CUDA(cudaMemsetAsync(start_min, 0x7f, bwd_start_block_bytes(d), stream));
        }
        attention_stats_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(o),
                                                           static_cast<const __nv_bfloat16 *>(dout), lse, lse2, delta,
                                                           d->batch, d->heads, d->queries, q_pad, d->head_dim, doc_start,
                                                           starts, start_max, start_min);
        TB200_CUDA(cudaGetLastError());
    }
    AttnBwdArgs p{};
    p.lse2 = lse2; p.delta = delta; p.q_pad = q_pad;
    p.kv_len = mask ? mask->kv_len : nullptr;
    p.doc_start = doc_start;
    p.starts = starts;
    p.start_max = start_max;
    p.start_min = start_min;
    p.batch = d->batch; p.heads = d->heads; p.kv_heads = d->kv_heads; p.queries = d->queries; p.keys = d->keys;
    p.causal = d->causal; p.scale = d->scale; p.scale_log2 = d->scale * kLog2e;
    // dK, dV: items over key tiles
    if ((st = bwd_tmap(&p.outer_a, k, kD, d->kv_heads, d->keys, d->batch, kOuter))) return st;
    if ((st = bwd_tmap(&p.outer_b, v, kD, d->kv_heads, d->keys, d->batch, kOuter))) return st;
    if ((st = bwd_tmap(&p.inner_a, q, kD, d->heads, d->queries, d->batch, kOuter))) return st;
    if ((st = bwd_tmap(&p.inner_b, dout, kD, d->heads, d->queries, d->batch, kOuter))) return st;
    if ((st = bwd_tmap(&p.out1, dv, kD, d->kv_heads, d->keys, d->batch, 32))) return st;
    if ((st = bwd_tmap(&p.out2, dk, kD, d->kv_heads, d->keys, d->batch, 32))) return st;
    p.outer_tiles = static_cast<int>(ceil_div(d->keys, kOuter));
    p.supers = (p.outer_tiles + 1) / 2 * d->batch * d->kv_heads;
    if (!d->deterministic) {
        // one kernel: dK and dV as above, each step's dQ contribution added into the Float32 accumulator, which a
        // second small kernel rounds
        const size_t elements = static_cast<size_t>(d->batch) * d->queries * d->heads * kD;
        p.dq_acc = reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + bwd_stat_bytes(d));
        TB200_CUDA(cudaMemsetAsync(p.dq_acc, 0, elements * sizeof(float), stream));
        {
            EncodeTiledFn fn;
            if ((st = bwd_encode_fn(&fn))) return st;
            cuuint64_t dims[4] = {static_cast<cuuint64_t>(kD), static_cast<cuuint64_t>(d->heads),
                                  static_cast<cuuint64_t>(d->queries), static_cast<cuuint64_t>(d->batch)};
            cuuint64_t strides[3] = {static_cast<cuuint64_t>(kD) * 4, static_cast<cuuint64_t>(kD) * d->heads * 4,
                                     static_cast<cuuint64_t>(kD) * d->heads * d->queries * 4};
            cuuint32_t box[4] = {32, 1, 16, 1};
            cuuint32_t elem[4] = {1, 1, 1, 1};
            if (fn(&p.dq_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.dq_acc, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return TB200_ERR_UNSUPPORTED;
        }
        if ((st = launch_bwd<2>(p, dev, stream))) return st;
        const long long vectors = static_cast<long long>(elements / 8);
        const long long blocks = ceil_div(vectors, 256);
        attention_dq_round_kernel<<<static_cast<unsigned>(blocks < dev.sms * 16ll ? blocks : dev.sms * 16ll), 256, 0, stream>>>(
            reinterpret_cast<const float4 *>(p.dq_acc), static_cast<uint4 *>(dq), vectors, d->scale);
        TB200_CUDA(cudaGetLastError());
        return TB200_OK;
    }
    if ((st = launch_bwd<1>(p, dev, stream))) return st;
    // dQ: items over query tiles
    if ((st = bwd_tmap(&p.outer_a, q, kD, d->heads, d->queries, d->batch, kOuter))) return st;
    if ((st = bwd_tmap(&p.outer_b, dout, kD, d->heads, d->queries, d->batch, kOuter))) return st;
    if ((st = bwd_tmap(&p.inner_a, k, kD, d->kv_heads, d->keys, d->batch, kOuter))) return st;
    if ((st = bwd_tmap(&p.inner_b, v, kD, d->kv_heads, d->keys, d->batch, kOuter))) return st;
    if ((st = bwd_tmap(&p.out2, dq, kD, d->heads, d->queries, d->batch, 32))) return st;
    p.outer_tiles = static_cast<int>(ceil_div(d->queries, kOuter));
    p.supers = (p.outer_tiles + 1) / 2 * d->batch * d->heads;
    return launch_bwd<0>(p, dev, stream);
}
}  // namespace

// Times the two forms of the pullback on the caller's own operands and returns the `deterministic` value of the
// faster one (0 = one kernel with atomic adds, 1 = two kernels): the measured stage of the reference's search over
// a claim's variants (src/Compiler/Implement/Implement.jl:120), here over the two hand-written schedules.  A caller
// that needs bit-repeatable gradients does not ask.  Overwrites dq, dk, dv with the pullback's own result,
// synchronises the stream; `workspace` must hold tb200_attention_bwd_workspace_bytes of the desc with
// deterministic = 0 (the larger of the two).  Other head dimensions than 128 have one schedule: returns 1.
extern "C" int tb200_attention_bwd_tune(const tb200_attn_desc *d, const void *q, const void *k, const void *v, const void *o,
                                        const float *lse, const void *dout, void *dq, void *dk, void *dv, void *workspace,
                                        size_t workspace_bytes, void *stream_) {
    if (!d) return TB200_ERR_NULL;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    tb200_attn_desc trial = *d;
    if (!attention_tensor_geometry(d)) {
        trial.deterministic = 1;
        const int st = tb200_attention_bwd(&trial, q, k, v, o, lse, dout, dq, dk, dv, workspace, workspace_bytes, stream_);
        return st ? st : 1;
    }
    cudaEvent_t t0, t1;
    TB200_CUDA(cudaEventCreate(&t0));
    TB200_CUDA(cudaEventCreate(&t1));
    float best_ms = 0.0f;
    int best = 1, status = TB200_OK;
    for (int form : {1, 0}) {
        trial.deterministic = form;
        if ((status = tb200_attention_bwd(&trial, q, k, v, o, lse, dout, dq, dk, dv, workspace, workspace_bytes, stream_))) break;
        if (cudaEventRecord(t0, stream) != cudaSuccess) { status = TB200_ERR_CUDA; break; }
        for (int rep = 0; rep < 3 && !status; rep++)
            status = tb200_attention_bwd(&trial, q, k, v, o, lse, dout, dq, dk, dv, workspace, workspace_bytes, stream_);
        if (status) break;
        float ms = 0.0f;
        if (cudaEventRecord(t1, stream) != cudaSuccess || cudaEventSynchronize(t1) != cudaSuccess ||
            cudaEventElapsedTime(&ms, t0, t1) != cudaSuccess) { status = TB200_ERR_CUDA; break; }
        if (form == 1 || ms < best_ms) { best_ms = ms; best = form; }
    }
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    return status ? status : best;
}

extern "C" int tb200_attention_bwd_device_error(void) {
    int code = 0, zero = 0;
    TB200_CUDA(cudaDeviceSynchronize());
    TB200_CUDA(cudaMemcpyFromSymbol(&code, g_attn_bwd_error, sizeof(int)));
    if (code) TB200_CUDA(cudaMemcpyToSymbol(g_attn_bwd_error, &zero, sizeof(int)));
    return code;
}
