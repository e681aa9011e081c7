// Flash-attention forward for sm_100a: O = softmax(scale * Q K^T + causal mask) V and the
// log-sum-exp of each query's scores, BFloat16 in and out, Float32 scores and statistics.
//
// Arrays are the reference's (features, heads, positions, batch) Julia arrays, i.e. memory
// [batch][position][head][feature]; the log-sum-exp is (1, heads, queries, batch) = [batch][query][head].
// The scores are computed from the BFloat16 queries and keys with Float32 accumulation, the softmax
// weights are rounded to BFloat16 for the second product, the output is rounded once
// (test/fixtures/operations.jl:21-76 and docs/src/cuda.md:40-46 of the reference).
//
// One persistent CTA per SM works through (batch, head, query tile) items; with more than one query tile the
// pair kernel further down takes two tiles at a time and walks them (batch, head)-major, a heavy and a light
// pair back to back, so that concurrent CTAs share few heads' K and V in L2.  Warp roles of the one-tile kernel:
//   warp 0      TMA loads: Q once per item, K and V tiles of 128 keys through 2-stage rings
//   warp 1      tcgen05.mma: S = Q K^T into one of two tensor-memory score buffers, then
//               O += P V (P from shared memory, V as an MN-major operand straight from its
//               [key][feature] layout); S of tile j+1 is issued before P V of tile j, so the tensor
//               core works while the softmax of tile j runs
//   warps 2-5   softmax: one thread per query row reads its 128 scores from tensor memory, keeps the
//               running maximum and sum (online softmax, exponentials as ex2 of pre-scaled scores),
//               writes P as BFloat16 into a 128-byte-swizzled shared tile, rescales the O accumulator
//               in tensor memory only when a row's maximum grew by more than 2^8 (the sum absorbs
//               smaller drifts exactly), and at the end normalises O, stages it in shared memory and
//               stores it by TMA.
// The one-tile kernel also takes masks the device holds (the starts of packed documents per query, a length per
// sequence) and operands at other strides: every role finds the item's key tiles [lo, hi) the same way -- all lanes of
// its warp read the tile's 128 starts, four a lane, and take their minimum and maximum -- key tiles before the
// earliest start or beyond the length are never loaded, the tiles a start or the length falls in are masked row by
// row, and an item that sees no key at all is answered by the softmax warps alone (zero rows, -Inf).
// No load uses cluster multicast.  Every barrier wait is bounded.
#include <cuda.h>

#include <mutex>

#include "attention_simt.cuh"
#include "common.cuh"
#include "sm100.cuh"

namespace tb200 {
namespace {

using namespace sm100;

constexpr int kTile = 128;            // queries per item, keys per step
constexpr int kHeadDim = 128;
constexpr int kSlab = kTile * 128;    // one 64-feature slab of a 128-row tile: 16 KB
constexpr int kTileBytes = 2 * kSlab; // 128 x 128 BFloat16
constexpr int kAttnThreads = 192;
constexpr float kRescaleThreshold = 8.0f;   // in log2 units

__device__ int g_attn_error = 0;

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

struct AttnFwdArgs {
    CUtensorMap q, k, v, o;   // 4-D (feature, head, position, batch), boxes of 64 features x 128 positions
    float *lse;               // [batch][query][head] or null
    int batch, heads, kv_heads, queries, keys;
    int q_tiles, items;
    int causal;
    float scale_log2;         // scale * log2(e)
    // masks the device holds (the one-tile kernel takes them; null: none)
    const int *doc_start;     // [batch][queries]: with `causal`, query j sees keys doc_start[b][j] <= i <= j
    const int *kv_len;        // [batch]: keys at and beyond kv_len[b] are masked
    __nv_bfloat16 *o_rows;    // O again as a plain pointer with its element strides: items that see no key at all
    long long o_batch, o_pos, o_head;   // write their zeros without the tensor core's help
};

// The key tiles one query tile visits, [lo, hi), under the causal mask, a length and the starts of packed documents.
// `dmax`: the largest start among the tile's queries (key tiles that begin before it need the per-row test).
struct KeyRange { int lo, hi, keys, dmax; };

// Every lane of a warp calls it (the starts of the tile's 128 queries are read four a lane).
__device__ __forceinline__ KeyRange key_range(const AttnFwdArgs &p, int b, int qt, int lane) {
    KeyRange r;
    r.keys = p.keys;
    if (p.kv_len) {
        const int n = p.kv_len[b];
        r.keys = n < 0 ? 0 : (n < p.keys ? n : p.keys);
    }
    r.hi = (r.keys + kTile - 1) / kTile;
    if (p.causal && qt + 1 < r.hi) r.hi = qt + 1;
    int dmin = 0;
    r.dmax = 0;
    if (p.doc_start) {
        int lo = 0x7fffffff, hi = 0;
        for (int i = lane; i < kTile; i += 32) {
            const int qi = qt * kTile + i;
            if (qi < p.queries) {
                int s = p.doc_start[static_cast<long long>(b) * p.queries + qi];
                s = s < 0 ? 0 : s;
                lo = s < lo ? s : lo;
                hi = s > hi ? s : hi;
            }
        }
        dmin = __reduce_min_sync(0xffffffffu, lo);
        r.dmax = __reduce_max_sync(0xffffffffu, hi);
        if (dmin == 0x7fffffff) dmin = 0;
    }
    r.lo = dmin / kTile;
    if (r.lo > r.hi) r.lo = r.hi;
    return r;
}

__device__ __forceinline__ uint64_t now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool wait_bounded(uint64_t *bar, uint32_t parity, volatile int *failed, int code) {
    if (mbar_wait(bar, parity, 4096)) return true;
    const uint64_t t0 = now_ns();
    while (true) {
        if (mbar_wait(bar, parity, 1024)) return true;
        if (*failed) return false;
        if (now_ns() - t0 > 2000000000ull) {
            *failed = code;
            atomicCAS(&g_attn_error, 0, code);
            return false;
        }
    }
}

// item -> (batch*head index, query tile), heaviest query tiles first under the causal mask
__device__ __forceinline__ void decode_item(const AttnFwdArgs &p, int item, int &bh, int &qt) {
    const int per = p.batch * p.heads;
    qt = p.q_tiles - 1 - item / per;
    bh = item % per;
}

__device__ __forceinline__ int kv_tiles_of(const AttnFwdArgs &p, int qt) {
    const int all = (p.keys + kTile - 1) / kTile;
    if (!p.causal) return all;
    const int upto = qt + 1;   // keys <= the tile's last query
    return upto < all ? upto : all;
}

__global__ void __launch_bounds__(kAttnThreads, 1) attention_fwd_kernel(const __grid_constant__ AttnFwdArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sq = smem;                       // Q tile
    uint8_t *sk = sq + kTileBytes;            // K ring, 2 stages
    uint8_t *sv = sk + 2 * kTileBytes;        // V ring, 2 stages
    uint8_t *sp = sv + 2 * kTileBytes;        // P, 2 buffers (buffer 0 also stages the O store)

    __shared__ __align__(8) uint64_t q_full, q_empty, o_done, o_free, pv_done;
    __shared__ __align__(8) uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
    __shared__ __align__(8) uint64_t s_full[2], s_empty[2], p_full[2], p_empty[2];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int failed_smem;
    volatile int *failed = &failed_smem;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        failed_smem = 0;
        mbar_init(&q_full, 1); mbar_init(&q_empty, 1); mbar_init(&o_done, 1); mbar_init(&o_free, 4);
        mbar_init(&pv_done, 1);
        for (int s = 0; s < 2; s++) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 4);
            mbar_init(&p_full[s], 4); mbar_init(&p_empty[s], 1);
        }
        fence_barrier_init();
        prefetch_tensormap(&p.q); prefetch_tensormap(&p.k); prefetch_tensormap(&p.v); prefetch_tensormap(&p.o);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_smem, 512);   // S0 | S1 | O | (spare)
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_smem;
    const uint32_t tmem_o = tmem_base + 2 * kTile;
    const int group = p.heads / p.kv_heads;

    if (warp == 0) {
        // the whole warp walks the items (the key range of an item is found by all its lanes); lane 0 loads
        uint32_t q_phase = 0, kv_count = 0;
        for (int item = blockIdx.x; item < p.items && !*failed; item += gridDim.x) {
            int bh, qt;
            decode_item(p, item, bh, qt);
            const int b = bh / p.heads, h = bh % p.heads, hk = h / group;
            const KeyRange kr = key_range(p, b, qt, lane);
            if (kr.lo >= kr.hi) continue;   // no key to see: the softmax warps write the zeros
            int ok = 1;
            if (lane == 0) {
                do {
                    if (!wait_bounded(&q_empty, q_phase ^ 1, failed, 1)) { ok = 0; break; }
                    mbar_arrive_expect_tx(&q_full, kTileBytes);
                    tma_load_4d(sq, &p.q, &q_full, 0, h, qt * kTile, b);
                    tma_load_4d(sq + kSlab, &p.q, &q_full, 64, h, qt * kTile, b);
                    for (int j = kr.lo; j < kr.hi; j++, kv_count++) {
                        const int st = kv_count & 1;
                        const uint32_t ph = (kv_count >> 1) & 1;
                        if (!wait_bounded(&k_empty[st], ph ^ 1, failed, 2)) { ok = 0; break; }
                        mbar_arrive_expect_tx(&k_full[st], kTileBytes);
                        tma_load_4d(sk + st * kTileBytes, &p.k, &k_full[st], 0, hk, j * kTile, b);
                        tma_load_4d(sk + st * kTileBytes + kSlab, &p.k, &k_full[st], 64, hk, j * kTile, b);
                        if (!wait_bounded(&v_empty[st], ph ^ 1, failed, 3)) { ok = 0; break; }
                        mbar_arrive_expect_tx(&v_full[st], kTileBytes);
                        tma_load_4d(sv + st * kTileBytes, &p.v, &v_full[st], 0, hk, j * kTile, b);
                        tma_load_4d(sv + st * kTileBytes + kSlab, &p.v, &v_full[st], 64, hk, j * kTile, b);
                    }
                } while (false);
            }
            q_phase ^= 1;
            if (!__shfl_sync(0xffffffffu, ok, 0)) break;
        }
    } else if (warp == 1) {
        {
            // S = Q K^T: both operands K-major (feature axis contiguous), two 64-feature slabs
            const uint32_t idesc_qk = umma_idesc_bf16(kTile, kTile, false, false);
            // O += P V: P K-major (key axis contiguous), V MN-major (feature axis contiguous)
            const uint32_t idesc_pv = umma_idesc_bf16(kTile, kHeadDim, false, true);
            uint32_t q_phase = 0, kv_count = 0, pv_count = 0, item_count = 0;
            for (int item = blockIdx.x; item < p.items && !*failed; item += gridDim.x) {
                int bh, qt;
                decode_item(p, item, bh, qt);
                const KeyRange kr = key_range(p, bh / p.heads, qt, lane);
                const int nkv = kr.hi - kr.lo;
                if (nkv <= 0) continue;
                bool ok = true;
                if (lane == 0) {
                if (!wait_bounded(&q_full, q_phase, failed, 4)) ok = false;
                tcgen05_fence_after();
                for (int j = 0; j <= nkv && ok; j++) {
                    if (j < nkv) {
                        const uint32_t c = kv_count + j;
                        const int st = c & 1;
                        const uint32_t ph = (c >> 1) & 1;
                        if (!wait_bounded(&k_full[st], ph, failed, 6)) { ok = false; break; }
                        if (!wait_bounded(&s_empty[st], ph ^ 1, failed, 7)) { ok = false; break; }
                        tcgen05_fence_after();
                        const uint32_t qa = smem_u32(sq), ka = smem_u32(sk + st * kTileBytes);
#pragma unroll
                        for (int k = 0; k < kHeadDim / 16; k++) {
                            const uint32_t off = (k >> 2) * kSlab + (k & 3) * 32;
                            tcgen05_mma_f16(tmem_base + st * kTile, umma_smem_desc(qa + off, 16, 1024),
                                            umma_smem_desc(ka + off, 16, 1024), idesc_qk, k != 0);
                        }
                        tcgen05_commit(&k_empty[st]);
                        tcgen05_commit(&s_full[st]);
                        if (j == nkv - 1) tcgen05_commit(&q_empty);
                    }
                    if (j > 0) {
                        const uint32_t c = pv_count;
                        const int st = c & 1;
                        const uint32_t ph = (c >> 1) & 1;
                        // the first product of an item overwrites O: the previous item's epilogue must have read it
                        if (j == 1 && !wait_bounded(&o_free, (item_count & 1) ^ 1, failed, 5)) { ok = false; break; }
                        if (!wait_bounded(&v_full[st], ph, failed, 8)) { ok = false; break; }
                        if (!wait_bounded(&p_full[st], ph, failed, 9)) { ok = false; break; }
                        tcgen05_fence_after();
                        const uint32_t pa = smem_u32(sp + st * kTileBytes), va = smem_u32(sv + st * kTileBytes);
#pragma unroll
                        for (int k = 0; k < kTile / 16; k++) {
                            const uint32_t poff = (k >> 2) * kSlab + (k & 3) * 32;   // 16 keys = 32 bytes along P's rows
                            const uint32_t voff = k * 16 * 128;                       // 16 key lines of 128 bytes
                            tcgen05_mma_f16(tmem_o, umma_smem_desc(pa + poff, 16, 1024),
                                            umma_smem_desc(va + voff, kSlab, 1024), idesc_pv, (j - 1) | k);
                        }
                        tcgen05_commit(&v_empty[st]);
                        tcgen05_commit(&p_empty[st]);
                        tcgen05_commit(&pv_done);
                        if (j == nkv) tcgen05_commit(&o_done);
                        pv_count++;
                    }
                }
                }
                q_phase ^= 1;
                kv_count += nkv;
                item_count++;
                if (!__shfl_sync(0xffffffffu, static_cast<int>(ok), 0)) break;
            }
        }
    } else {
        // ---- softmax, correction and epilogue: thread = query row
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
        uint32_t kv_count = 0, item_count = 0, pv_seen = 0;
        for (int item = blockIdx.x; item < p.items; item += gridDim.x) {
            int bh, qt;
            decode_item(p, item, bh, qt);
            const int b = bh / p.heads, h = bh % p.heads;
            const KeyRange kr = key_range(p, b, qt, lane);
            const int qi = qt * kTile + row;    // this thread's query
            if (kr.lo >= kr.hi) {
                // no key to see for any query of the tile: zero rows, a log-sum-exp of -Inf, no product
                if (qi < p.queries) {
                    uint4 *dst = reinterpret_cast<uint4 *>(p.o_rows + b * p.o_batch + qi * p.o_pos + h * p.o_head);
#pragma unroll
                    for (int c = 0; c < kHeadDim / 8; c++) dst[c] = make_uint4(0u, 0u, 0u, 0u);
                    if (p.lse) p.lse[(static_cast<long long>(b) * p.queries + qi) * p.heads + h] = -INFINITY;
                }
                continue;
            }
            // the first key this query sees (packed documents), 0 without
            const int first_key = (p.doc_start && qi < p.queries) ? p.doc_start[static_cast<long long>(b) * p.queries + qi] : 0;
            float m_used = -INFINITY, l = 0.0f;
            bool ok = true;
            for (int j = kr.lo; j < kr.hi; j++, kv_count++) {
                const int st = kv_count & 1;
                const uint32_t ph = (kv_count >> 1) & 1;
                if (!wait_bounded(&s_full[st], ph, failed, 10)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t ts = tmem_base + lane_base + st * kTile;
                const int key0 = j * kTile;
                const bool edge = (p.causal && key0 + kTile - 1 > qt * kTile) || key0 + kTile > kr.keys || key0 < kr.dmax;
                // the whole row of 128 scores into registers: the four loads are in flight together
                // (one load-then-wait at a time costs about 800 cycles each)
                uint32_t r[kTile];
#pragma unroll
                for (int c = 0; c < kTile / 32; c++)
                    tmem_ld_32x32(ts + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
                tmem_ld_wait();
                // the score buffer is free for the tile after next
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_empty[st]);
                if (edge) {
#pragma unroll
                    for (int i = 0; i < kTile; i++) {
                        const int key = key0 + i;
                        if ((p.causal && key > qi) || key >= kr.keys || key < first_key) r[i] = 0xff800000u;   // -Inf
                    }
                }
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < kTile; i += 4) {
#pragma unroll
                    for (int u = 0; u < 4; u++) mx[u] = fmaxf(mx[u], __uint_as_float(r[i + u]));
                }
                float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                m_tile *= p.scale_log2;   // scale > 0: the maximum commutes with the scaling
                float alpha = 1.0f;
                bool grew = false;
                if (m_tile > m_used + kRescaleThreshold || (m_used == -INFINITY && m_tile > -INFINITY)) {
                    alpha = (m_used == -INFINITY) ? 0.0f : fast_exp2(m_used - m_tile);
                    grew = j > kr.lo && m_used != -INFINITY;
                    m_used = m_tile;
                    l *= alpha;
                }
                // the P buffer must have been read by the product that used it two tiles ago
                if (!wait_bounded(&p_empty[st], ph ^ 1, failed, 11)) { ok = false; break; }
                // weights, their sum, P to shared memory
                const float neg_m = (m_used == -INFINITY) ? 0.0f : -m_used;
                uint8_t *prow = sp + st * kTileBytes + row * 128;
                float ls[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int g = 0; g < kTile / 8; g++) {
                    float w[8];
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        w[u] = fast_exp2(fmaf(__uint_as_float(r[8 * g + u]), p.scale_log2, neg_m));
                        ls[u & 3] += w[u];
                    }
                    uint4 v4;
                    v4.x = pack_bf16x2(w[0], w[1]);
                    v4.y = pack_bf16x2(w[2], w[3]);
                    v4.z = pack_bf16x2(w[4], w[5]);
                    v4.w = pack_bf16x2(w[6], w[7]);
                    // keys [8g, 8g+8) = slab g/8, 16-byte chunk g%8 of the row
                    *reinterpret_cast<uint4 *>(prow + (g >> 3) * kSlab + (((g & 7) ^ (row & 7)) << 4)) = v4;
                }
                l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
                // O holds the products up to tile j-1 once pv_done has completed that many times for this item
                if (j > kr.lo) {
                    if (!wait_bounded(&pv_done, pv_seen & 1, failed, 12)) { ok = false; break; }
                    pv_seen++;
                    tcgen05_fence_after();
                    if (__any_sync(0xffffffffu, grew)) {
#pragma unroll 1
                        for (int c = 0; c < kHeadDim / 32; c++) {
                            uint32_t r[32];
                            tmem_ld_32x32(tmem_o + lane_base + c * 32, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                            tmem_st_32x32(tmem_o + lane_base + c * 32, r);
                        }
                        tmem_st_wait();
                    }
                }
                tcgen05_fence_before();
                fence_proxy_async();   // P was written by ordinary stores; the MMA reads it through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_full[st]);
            }
            if (!ok) break;
            // ---- epilogue: O / l, the log-sum-exp, store
            if (!wait_bounded(&o_done, item_count & 1, failed, 13)) break;
            if (!wait_bounded(&pv_done, pv_seen & 1, failed, 14)) break;   // the last product's arrival
            pv_seen++;
            tcgen05_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;   // a query that sees no key: a zero row
            // every product of the item is complete, so P buffer 0 is idle: each warp stages its own 32
            // rows of O there (the rows it alone writes when the buffer next holds P)
            {
                uint32_t r[kHeadDim];
#pragma unroll
                for (int c = 0; c < kHeadDim / 32; c++)
                    tmem_ld_32x32(tmem_o + lane_base + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
                tmem_ld_wait();
#pragma unroll
                for (int g = 0; g < kHeadDim / 8; g++) {
                    uint4 v4;
                    v4.x = pack_bf16x2(__uint_as_float(r[8 * g]) * inv, __uint_as_float(r[8 * g + 1]) * inv);
                    v4.y = pack_bf16x2(__uint_as_float(r[8 * g + 2]) * inv, __uint_as_float(r[8 * g + 3]) * inv);
                    v4.z = pack_bf16x2(__uint_as_float(r[8 * g + 4]) * inv, __uint_as_float(r[8 * g + 5]) * inv);
                    v4.w = pack_bf16x2(__uint_as_float(r[8 * g + 6]) * inv, __uint_as_float(r[8 * g + 7]) * inv);
                    // P buffer 0 is idle: all products are done
                    *reinterpret_cast<uint4 *>(sp + row * 128 + (g >> 3) * kSlab + (((g & 7) ^ (row & 7)) << 4)) = v4;
                }
            }
            if (p.lse && qi < p.queries)
                p.lse[(static_cast<long long>(b) * p.queries + qi) * p.heads + h] =
                    (m_used == -INFINITY) ? -INFINITY : (m_used + log2f(l)) * 0.6931471805599453f;
            tcgen05_fence_before();
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                // this warp's 32 rows, two 64-feature slabs
                tma_store_4d(&p.o, sp + q * 32 * 128, 0, h, qt * kTile + q * 32, b);
                tma_store_4d(&p.o, sp + kSlab + q * 32 * 128, 64, h, qt * kTile + q * 32, b);
                bulk_commit_group();
                bulk_wait_group_read<0>();   // P buffer 0 is written again by the next item's first tile
                mbar_arrive(&o_free);
            }
            __syncwarp();
            item_count++;
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

// ---------------------------------------------------------------- two query tiles per CTA ----
//
// The kernel above leaves its four softmax warps alone on their schedulers: every wait on tensor memory, on
// the exponential unit or on a barrier is a bubble.  Here a CTA takes 256 queries of one head as two
// independent 128-query tiles, each with its own four softmax warps, score buffer and accumulator in tensor
// memory (S_A | S_B | O_A | O_B = 512 columns).  The two tiles have nothing to exchange, so one tile's
// softmax fills the other's bubbles and the tensor core always has the other tile's product to run.  The
// weights do not go through shared memory: each softmax thread writes its row of P as packed BFloat16 over
// the first 64 columns of its own score buffer and the second product reads its A operand from tensor memory.
// The MMAs of one CTA execute in issue order, so S of the next key tile (issued after P V of this one) cannot
// overwrite P early.  Shared memory: Q_A, Q_B, two K stages, two V stages; a tile's Q buffer stages its O
// store once the tile's products are complete.
constexpr int kPairThreads = 320;

__device__ __forceinline__ int pair_kv_tiles(const AttnFwdArgs &p, int qt) {
    if (qt >= p.q_tiles) return 0;
    return kv_tiles_of(p, qt);
}

__global__ void __launch_bounds__(kPairThreads, 1) attention_fwd_pair_kernel(const __grid_constant__ AttnFwdArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sq = smem;                       // Q_A, Q_B
    uint8_t *sk = sq + 2 * kTileBytes;        // K ring, 2 stages
    uint8_t *sv = sk + 2 * kTileBytes;        // V ring, 2 stages

    __shared__ __align__(8) uint64_t q_full[2], q_empty[2], s_full[2], p_half[2][2], pv_done[2], o_free[2];
    __shared__ __align__(8) uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int failed_smem;
    volatile int *failed = &failed_smem;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        failed_smem = 0;
        for (int s = 0; s < 2; s++) {
            mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 4); mbar_init(&s_full[s], 1); mbar_init(&p_half[s][0], 4); mbar_init(&p_half[s][1], 4);
            mbar_init(&pv_done[s], 1); mbar_init(&o_free[s], 4);
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
        }
        fence_barrier_init();
        prefetch_tensormap(&p.q); prefetch_tensormap(&p.k); prefetch_tensormap(&p.v); prefetch_tensormap(&p.o);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_smem, 512);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_smem;
    const int group = p.heads / p.kv_heads;
    // The walk over the work: a CTA takes whole "supers" = the i-th heaviest and the i-th lightest pair of query
    // tiles of one (batch, head), one after the other.  Under the causal mask every super then costs the same, so
    // the static round-robin over CTAs is balanced, and because supers are numbered (batch, head)-major the CTAs
    // that run at the same time read the K and V of a few heads only: the tiles stay in L2 instead of
    // being streamed from HBM once per query tile.
    const int pair_tiles = (p.q_tiles + 1) / 2;
    const int half_tiles = (pair_tiles + 1) / 2;
    const int supers = half_tiles * p.batch * p.heads;
    // walk step j of this CTA -> (batch*head, pair tile); false when the CTA is done, pt < 0 for the second half of
    // a super whose two halves are the same tile
    auto walk = [&](int j, int &bh, int &pt) -> bool {
        const int sup = blockIdx.x + (j >> 1) * gridDim.x;
        if (sup >= supers) return false;
        bh = sup / half_tiles;
        const int i = sup % half_tiles;
        pt = (j & 1) ? i : pair_tiles - 1 - i;
        if ((j & 1) && i == pair_tiles - 1 - i) pt = -1;
        return true;
    };

    if (warp == 0) {
        if (elect_one()) {
            uint32_t kv_count = 0, q_loads[2] = {0, 0};
            for (int j = 0; !*failed; j++) {
                int bh, pt;
                if (!walk(j, bh, pt)) break;
                if (pt < 0) continue;
                const int b = bh / p.heads, h = bh % p.heads, hk = h / group;
                bool ok = true;
                for (int g = 0; g < 2 && ok; g++) {
                    const int qt = 2 * pt + g;
                    if (qt >= p.q_tiles) continue;
                    // a tile's Q buffer is released by its softmax warps once their O store has read it; the
                    // second tile is absent from some items, so each tile counts its own loads
                    if (!wait_bounded(&q_empty[g], (q_loads[g] & 1) ^ 1, failed, 1)) { ok = false; break; }
                    q_loads[g]++;
                    mbar_arrive_expect_tx(&q_full[g], kTileBytes);
                    tma_load_4d(sq + g * kTileBytes, &p.q, &q_full[g], 0, h, qt * kTile, b);
                    tma_load_4d(sq + g * kTileBytes + kSlab, &p.q, &q_full[g], 64, h, qt * kTile, b);
                }
                if (!ok) break;
                const int n0 = pair_kv_tiles(p, 2 * pt), n1 = pair_kv_tiles(p, 2 * pt + 1);
                const int nkv = n0 > n1 ? n0 : n1;
                for (int j = 0; j < nkv; j++, kv_count++) {
                    const int st = kv_count & 1;
                    const uint32_t ph = (kv_count >> 1) & 1;
                    if (!wait_bounded(&k_empty[st], ph ^ 1, failed, 2)) break;
                    mbar_arrive_expect_tx(&k_full[st], kTileBytes);
                    tma_load_4d(sk + st * kTileBytes, &p.k, &k_full[st], 0, hk, j * kTile, b);
                    tma_load_4d(sk + st * kTileBytes + kSlab, &p.k, &k_full[st], 64, hk, j * kTile, b);
                    if (!wait_bounded(&v_empty[st], ph ^ 1, failed, 3)) break;
                    mbar_arrive_expect_tx(&v_full[st], kTileBytes);
                    tma_load_4d(sv + st * kTileBytes, &p.v, &v_full[st], 0, hk, j * kTile, b);
                    tma_load_4d(sv + st * kTileBytes + kSlab, &p.v, &v_full[st], 64, hk, j * kTile, b);
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc_qk = umma_idesc_bf16(kTile, kTile, false, false);
            const uint32_t idesc_pv = umma_idesc_bf16(kTile, kHeadDim, false, true);
            uint32_t kv_count = 0;
            uint32_t items_of[2] = {0, 0}, p_count[2] = {0, 0};
            auto scores = [&](int g, int st) {   // S_g = Q_g K^T
                const uint32_t qa = smem_u32(sq + g * kTileBytes), ka = smem_u32(sk + st * kTileBytes);
#pragma unroll
                for (int k = 0; k < kHeadDim / 16; k++) {
                    const uint32_t off = (k >> 2) * kSlab + (k & 3) * 32;
                    tcgen05_mma_f16(tmem_base + g * kTile, umma_smem_desc(qa + off, 16, 1024), umma_smem_desc(ka + off, 16, 1024),
                                    idesc_qk, k != 0);
                }
                tcgen05_commit(&s_full[g]);
            };
            for (int j = 0; !*failed; j++) {
                int bh, pt;
                if (!walk(j, bh, pt)) break;
                if (pt < 0) continue;
                const int n[2] = {pair_kv_tiles(p, 2 * pt), pair_kv_tiles(p, 2 * pt + 1)};
                const int nkv = n[0] > n[1] ? n[0] : n[1];
                bool ok = true;
                for (int g = 0; g < 2 && ok; g++)
                    if (n[g] > 0) {
                        if (!wait_bounded(&q_full[g], items_of[g] & 1, failed, 4)) ok = false;
                    }
                if (!ok) break;
                tcgen05_fence_after();
                // the first key tile's scores for both query tiles
                {
                    const int st = kv_count & 1;
                    if (!wait_bounded(&k_full[st], (kv_count >> 1) & 1, failed, 6)) break;
                    tcgen05_fence_after();
                    for (int g = 0; g < 2; g++)
                        if (n[g] > 0) {
                            scores(g, st);
                        }
                    tcgen05_commit(&k_empty[st]);   // K of tile 0 is free once both score products have run
                }
                for (int j = 0; j < nkv && ok; j++) {
                    const uint32_t c = kv_count + j;
                    const int st = c & 1;
                    const uint32_t ph = (c >> 1) & 1;
                    const int st_next = (c + 1) & 1;
                    const uint32_t ph_next = ((c + 1) >> 1) & 1;
                    bool k_next_ready = false;
                    for (int g = 0; g < 2 && ok; g++) {
                        if (j >= n[g]) continue;
                        // O_g += P_g V_j
                        if (j == 0 && !wait_bounded(&o_free[g], (items_of[g] & 1) ^ 1, failed, 5)) { ok = false; break; }
                        if (!wait_bounded(&v_full[st], ph, failed, 8)) { ok = false; break; }
                        // the weights arrive in two halves of 64 keys: the first four steps run while the second
                        // half's exponentials are still being taken
                        const uint32_t va = smem_u32(sv + st * kTileBytes);
                        if (!wait_bounded(&p_half[g][0], p_count[g] & 1, failed, 9)) { ok = false; break; }
                        tcgen05_fence_after();
#pragma unroll
                        for (int k = 0; k < kTile / 32; k++)
                            tcgen05_mma_f16_ts(tmem_base + (2 + g) * kTile, tmem_base + g * kTile + k * 8,
                                               umma_smem_desc(va + k * 16 * 128, kSlab, 1024), idesc_pv, j | k);
                        if (!wait_bounded(&p_half[g][1], p_count[g] & 1, failed, 9)) { ok = false; break; }
                        p_count[g]++;
                        tcgen05_fence_after();
#pragma unroll
                        for (int k = kTile / 32; k < kTile / 16; k++)
                            tcgen05_mma_f16_ts(tmem_base + (2 + g) * kTile, tmem_base + g * kTile + k * 8,
                                               umma_smem_desc(va + k * 16 * 128, kSlab, 1024), idesc_pv, 1);
                        tcgen05_commit(&pv_done[g]);
                        // scores of the next key tile for this query tile
                        if (j + 1 < n[g]) {
                            if (!k_next_ready) {
                                if (!wait_bounded(&k_full[st_next], ph_next, failed, 6)) { ok = false; break; }
                                tcgen05_fence_after();
                                k_next_ready = true;
                            }
                            scores(g, st_next);
                        }
                    }
                    if (!ok) break;
                    tcgen05_commit(&v_empty[st]);                       // V_j: both products issued
                    if (j + 1 < nkv) tcgen05_commit(&k_empty[st_next]);  // K_{j+1}: both score products issued
                }
                kv_count += nkv;
                for (int g = 0; g < 2; g++)
                    if (n[g] > 0) items_of[g]++;
                if (!ok) break;
            }
        }
    } else {
        // ---- softmax warps: tile g, thread = query row
        const int g = (warp - 2) >> 2;
        const int q = warp & 3;   // the warp's quarter of the 128 tensor-memory lanes (warp id mod 4)
        const int row = q * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
        const uint32_t tmem_s = tmem_base + lane_base + g * kTile;
        const uint32_t tmem_o = tmem_base + lane_base + (2 + g) * kTile;
        uint8_t *stage = sq + g * kTileBytes;
        uint32_t s_count = 0, pv_seen = 0;
        for (int j = 0;; j++) {
            int bh, pt;
            if (!walk(j, bh, pt)) break;
            if (pt < 0) continue;
            const int b = bh / p.heads, h = bh % p.heads;
            const int qt = 2 * pt + g;
            const int nkv = pair_kv_tiles(p, qt);
            if (nkv == 0) continue;
            const int qi = qt * kTile + row;
            float m_used = -INFINITY, l = 0.0f;
            bool ok = true;
            for (int j = 0; j < nkv; j++, s_count++) {
                if (!wait_bounded(&s_full[g], s_count & 1, failed, 10)) { ok = false; break; }
                tcgen05_fence_after();
                const int key0 = j * kTile;
                const bool edge = (p.causal && key0 + kTile - 1 > qt * kTile) || key0 + kTile > p.keys;
                uint32_t r[kTile];
#pragma unroll
                for (int c = 0; c < kTile / 32; c++) tmem_ld_32x32(tmem_s + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
                tmem_ld_wait();
                if (edge) {
#pragma unroll
                    for (int i = 0; i < kTile; i++) {
                        const int key = key0 + i;
                        if ((p.causal && key > qi) || key >= p.keys) r[i] = 0xff800000u;
                    }
                }
                // the row's maximum with three-input maxima, four chains: 64 instructions for the 128 scores
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < kTile; i += 8) {
#pragma unroll
                    for (int u = 0; u < 4; u++) mx[u] = max3(mx[u], __uint_as_float(r[i + 2 * u]), __uint_as_float(r[i + 2 * u + 1]));
                }
                float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
                float alpha = 1.0f;
                bool grew = false;
                if (m_tile > m_used + kRescaleThreshold || (m_used == -INFINITY && m_tile > -INFINITY)) {
                    alpha = (m_used == -INFINITY) ? 0.0f : fast_exp2(m_used - m_tile);
                    grew = j > 0 && m_used != -INFINITY;
                    m_used = m_tile;
                    l *= alpha;
                }
                const float neg_m = (m_used == -INFINITY) ? 0.0f : -m_used;
                // weights packed two per column over the row's own scores, in two halves of 64 keys: the first half is
                // handed to the product P V while the second half's exponentials are still being taken, so the
                // product's first four steps run under them instead of after them
                const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), neg_m2 = make_float2(neg_m, neg_m);
                float2 ls2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
                // two scores at a time with packed Float32 arithmetic (the scaling and the row sum are one instruction
                // per pair): this loop is bound by issue slots, not by the special-function unit -- taking part of the
                // exponentials as a polynomial on the FMA pipe instead made it slower in every proportion tried
                auto weights = [&](int i) {   // scores i, i + 1 -> their packed weights in r[i / 2]
                    const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), scale2, neg_m2);
                    const float2 w = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                    ls2[(i >> 1) & 1] = __fadd2_rn(ls2[(i >> 1) & 1], w);
                    r[i >> 1] = pack_bf16x2(w.x, w.y);
                };
#pragma unroll
                for (int i = 0; i < kTile / 2; i += 2) weights(i);
                tmem_st_32x32(tmem_s, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                // O_g holds the products up to tile j-1 once pv_done has completed; a rescale has to be in place
                // before any step of this tile's product adds to it
                if (j > 0) {
                    if (!wait_bounded(&pv_done[g], pv_seen & 1, failed, 12)) { ok = false; break; }
                    pv_seen++;
                    tcgen05_fence_after();
                    if (__any_sync(0xffffffffu, grew)) {
#pragma unroll 1
                        for (int c = 0; c < kHeadDim / 32; c++) {
                            uint32_t o[32];
                            tmem_ld_32x32(tmem_o + c * 32, o);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st_32x32(tmem_o + c * 32, o);
                        }
                    }
                }
                tmem_st_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_half[g][0]);
#pragma unroll
                for (int i = kTile / 2; i < kTile; i += 2) weights(i);
                l += (ls2[0].x + ls2[0].y) + (ls2[1].x + ls2[1].y);
                tmem_st_32x32(tmem_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
                tmem_st_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_half[g][1]);
            }
            if (!ok) break;
            // ---- epilogue: O / l, the log-sum-exp, store through the tile's own Q buffer
            if (!wait_bounded(&pv_done[g], pv_seen & 1, failed, 14)) break;
            pv_seen++;
            tcgen05_fence_after();
            const float inv = 1.0f / l;
            {
                uint32_t r[kHeadDim];
#pragma unroll
                for (int c = 0; c < kHeadDim / 32; c++) tmem_ld_32x32(tmem_o + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
                tmem_ld_wait();
#pragma unroll
                for (int gg = 0; gg < kHeadDim / 8; gg++) {
                    uint4 v4;
                    v4.x = pack_bf16x2(__uint_as_float(r[8 * gg]) * inv, __uint_as_float(r[8 * gg + 1]) * inv);
                    v4.y = pack_bf16x2(__uint_as_float(r[8 * gg + 2]) * inv, __uint_as_float(r[8 * gg + 3]) * inv);
                    v4.z = pack_bf16x2(__uint_as_float(r[8 * gg + 4]) * inv, __uint_as_float(r[8 * gg + 5]) * inv);
                    v4.w = pack_bf16x2(__uint_as_float(r[8 * gg + 6]) * inv, __uint_as_float(r[8 * gg + 7]) * inv);
                    *reinterpret_cast<uint4 *>(stage + row * 128 + (gg >> 3) * kSlab + (((gg & 7) ^ (row & 7)) << 4)) = v4;
                }
            }
            if (p.lse && qi < p.queries)
                p.lse[(static_cast<long long>(b) * p.queries + qi) * p.heads + h] =
                    (m_used == -INFINITY) ? -INFINITY : (m_used + log2f(l)) * 0.6931471805599453f;
            tcgen05_fence_before();
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_store_4d(&p.o, stage + q * 32 * 128, 0, h, qt * kTile + q * 32, b);
                tma_store_4d(&p.o, stage + kSlab + q * 32 * 128, 64, h, qt * kTile + q * 32, b);
                bulk_commit_group();
                bulk_wait_group_read<0>();
                mbar_arrive(&o_free[g]);    // the accumulator has been read
                mbar_arrive(&q_empty[g]);   // and the Q buffer is free for the next item's load
            }
            __syncwarp();
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int attn_encode_fn(EncodeTiledFn *out) {
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

// (feature, head, position, batch) BFloat16 array, dense, as boxes of 64 features x `rows` positions.
// `stride`: elements from one batch member, position, head to the next (null: dense).
int attn_tmap(CUtensorMap *map, const void *base, int d, int heads, int positions, int batch, int rows,
              const long long *stride = nullptr) {
    EncodeTiledFn fn;
    int st = attn_encode_fn(&fn);
    if (st) return st;
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(heads),
                          static_cast<cuuint64_t>(positions), static_cast<cuuint64_t>(batch)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(d) * 2, static_cast<cuuint64_t>(d) * heads * 2,
                             static_cast<cuuint64_t>(d) * heads * positions * 2};
    if (stride) {
        strides[0] = static_cast<cuuint64_t>(stride[2]) * 2;
        strides[1] = static_cast<cuuint64_t>(stride[1]) * 2;
        strides[2] = static_cast<cuuint64_t>(stride[0]) * 2;
    }
    cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(rows), 1};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TB200_OK : TB200_ERR_UNSUPPORTED;
}

}  // namespace
}  // namespace tb200

using namespace tb200;

namespace tb200 {

// The tensor-core forward on checked arguments.  `mask` (may be null): masks the device holds and operands at other
// strides -- those run on the one-tile kernel, which finds each item's key range and masks row by row; the plain
// programs with more than one query tile take the pair kernel.  TB200_ERR_UNSUPPORTED: strides the TMA unit cannot
// describe (the caller then falls to the CUDA-core kernels).
int attention_tensor_fwd(const tb200_attn_desc *d, const tb200_attn_mask *mask, const void *q, const void *k, const void *v,
                         void *o, float *lse, cudaStream_t stream) {
    DeviceInfo dev;
    int st = current_device(&dev);
    if (st) return st;
    long long qs[3] = {static_cast<long long>(d->queries) * d->heads * d->head_dim, static_cast<long long>(d->heads) * d->head_dim,
                       d->head_dim};
    long long ks[3] = {static_cast<long long>(d->keys) * d->kv_heads * d->head_dim,
                       static_cast<long long>(d->kv_heads) * d->head_dim, d->head_dim};
    bool masked = false;
    if (mask) {
        if (mask->q_stride[0] || mask->q_stride[1] || mask->q_stride[2])
            for (int i = 0; i < 3; i++) qs[i] = mask->q_stride[i];
        if (mask->kv_stride[0] || mask->kv_stride[1] || mask->kv_stride[2])
            for (int i = 0; i < 3; i++) ks[i] = mask->kv_stride[i];
        masked = mask->doc_start || mask->kv_len;
        for (int i = 0; i < 3; i++)
            if (qs[i] <= 0 || ks[i] <= 0 || qs[i] % 8 || ks[i] % 8) return TB200_ERR_UNSUPPORTED;
    }
    AttnFwdArgs p{};
    if ((st = attn_tmap(&p.q, q, d->head_dim, d->heads, d->queries, d->batch, kTile, qs))) return st;
    if ((st = attn_tmap(&p.k, k, d->head_dim, d->kv_heads, d->keys, d->batch, kTile, ks))) return st;
    if ((st = attn_tmap(&p.v, v, d->head_dim, d->kv_heads, d->keys, d->batch, kTile, ks))) return st;
    if ((st = attn_tmap(&p.o, o, d->head_dim, d->heads, d->queries, d->batch, 32, qs))) return st;
    p.lse = lse;
    p.batch = d->batch; p.heads = d->heads; p.kv_heads = d->kv_heads; p.queries = d->queries; p.keys = d->keys;
    p.q_tiles = static_cast<int>(ceil_div(d->queries, kTile));
    p.items = p.q_tiles * d->batch * d->heads;
    p.causal = d->causal;
    p.scale_log2 = d->scale * kLog2e;
    p.doc_start = mask ? mask->doc_start : nullptr;
    p.kv_len = mask ? mask->kv_len : nullptr;
    p.o_rows = static_cast<__nv_bfloat16 *>(o);
    p.o_batch = qs[0]; p.o_pos = qs[1]; p.o_head = qs[2];
    const size_t smem = 7 * kTileBytes + 1024;
    static std::mutex lock;
    static bool configured[64] = {};
    {
        std::lock_guard<std::mutex> hold(lock);
        if (!configured[dev.device]) {
            TB200_CUDA(cudaFuncSetAttribute(attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(smem)));
            configured[dev.device] = true;
        }
    }
    // more than one query tile and nothing but the causal mask: two tiles per CTA, each with its own softmax warps
    if (p.q_tiles > 1 && !masked) {
        const size_t pair_smem = 6 * kTileBytes + 1024;
        {
            std::lock_guard<std::mutex> hold(lock);
            static bool pair_configured[64] = {};
            if (!pair_configured[dev.device]) {
                TB200_CUDA(cudaFuncSetAttribute(attention_fwd_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                static_cast<int>(pair_smem)));
                pair_configured[dev.device] = true;
            }
        }
        const int supers = ((p.q_tiles + 1) / 2 + 1) / 2 * d->batch * d->heads;
        const unsigned pair_grid = static_cast<unsigned>(supers < dev.sms ? supers : dev.sms);
        attention_fwd_pair_kernel<<<pair_grid, kPairThreads, pair_smem, stream>>>(p);
        TB200_CUDA(cudaGetLastError());
        return TB200_OK;
    }
    const unsigned grid = static_cast<unsigned>(p.items < dev.sms ? p.items : dev.sms);
    attention_fwd_kernel<<<grid, kAttnThreads, smem, stream>>>(p);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

}  // namespace tb200

extern "C" int tb200_attention_fwd(const tb200_attn_desc *d, const void *q, const void *k, const void *v, void *o,
                                   float *lse, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!d) return TB200_ERR_NULL;
    if (d->batch < 0 || d->heads <= 0 || d->kv_heads <= 0 || d->queries < 0 || d->keys < 0 || d->head_dim <= 0)
        return TB200_ERR_SHAPE;
    if (d->heads % d->kv_heads != 0 || !(d->scale > 0.0f)) return TB200_ERR_SHAPE;
    if (d->causal && d->queries != d->keys) return TB200_ERR_SHAPE;
    if (d->dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (!attention_tensor_geometry(d) && !attention_simt_takes(d)) return TB200_ERR_UNSUPPORTED;
    if (d->batch == 0 || d->queries == 0) return TB200_OK;
    if (d->keys == 0) return TB200_ERR_UNSUPPORTED;
    if (!q || !k || !v || !o) return TB200_ERR_NULL;
    if (!aligned_to(q, 16) || !aligned_to(k, 16) || !aligned_to(v, 16) || !aligned_to(o, 16) || !aligned_to(lse, 4))
        return TB200_ERR_ALIGN;
    if (d->queries > (1 << 24) || d->keys > (1 << 24)) return TB200_ERR_SHAPE;
    if (!attention_tensor_geometry(d)) return attention_simt_fwd(d, q, k, v, o, lse, stream);
    return attention_tensor_fwd(d, nullptr, q, k, v, o, lse, stream);
}

extern "C" int tb200_attention_device_error(void) {
    int code = 0, zero = 0;
    TB200_CUDA(cudaDeviceSynchronize());
    TB200_CUDA(cudaMemcpyFromSymbol(&code, g_attn_error, sizeof(int)));
    if (code) TB200_CUDA(cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int)));
    return code;
}
