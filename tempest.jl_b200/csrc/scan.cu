// Scans (running folds) for sm_100a: cumulative sum / product / maximum / minimum, the affine recurrence
// h = a h_prev + b named with a GenericFold, and a running variance -- the folds of the reference's scan tests
// (test/cuda/scans.jl:12-22; the user folds are test/fixtures/programs.jl:44, 51-54; the documented recurrence is
// src/Compiler/IR/folds.jl:279-288), forward or reversed (a cumulative sum's derivative scans backwards), along
// the contiguous axis of a (n, rows) matrix or across its rows, over a batch of such matrices.  They stand for
// the kernels the reference generates for `:scan` groups (ext/cuTileExt/build.jl:715-760: a block per tile of
// the kept axes sweeps the scanned axis a tile at a step, carrying each lane's state).
//
// Along a row (the scanned axis is contiguous): one block per row sweeps it in tiles of 256 threads x 8
// elements.  A thread reads its own eight elements with 128-bit accesses (one at a time when addresses or lengths
// do not allow it) and scans them in registers, the threads' totals are scanned by warp shuffles and one exchange
// through shared memory with a single barrier per tile, and the carry of the tiles before is combined in front:
// every element is read once and written once.  States combine strictly left to right (the affine recurrence does not commute).
// Across the rows (the scanned axis is the strided one): one thread per column walks the rows in order with its
// state in a register, eight rows' loads in flight at a time; neighbouring threads read neighbouring columns, so
// every access is coalesced.  Parallelism is the number of columns: a scan across many rows of few columns keeps
// few SMs busy (measured: 16384 rows of 4096 Float32 columns, 16 blocks, 0.32 TB/s); with scratch for their totals
// the rows are cut into slabs that are folded side by side and swept a second time from the totals before them
// (2.6 TB/s at that shape).
// Float32 or BFloat16 elements; states and arithmetic in Float32, each result rounded once.
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kScanThreads = 256;
constexpr int kScanPer = 8;   // elements a thread scans in registers

// One state per fold: `lift` an element, `combine` (earlier, later), `observe` the running result.
struct SumState { float v; };
struct AffineState { float a, b; };        // x -> a x + b
struct MomentState { float n, mean, m2; }; // count, mean, centred sum of squares (Chan's merge)

template <int OP> struct Fold;
template <> struct Fold<TB200_SCAN_SUM> {
    using S = SumState;
    static __device__ __forceinline__ S identity() { return {0.0f}; }
    static __device__ __forceinline__ S lift(float x, float) { return {x}; }
    static __device__ __forceinline__ S combine(S l, S r) { return {l.v + r.v}; }
    static __device__ __forceinline__ float observe(S s) { return s.v; }
};
template <> struct Fold<TB200_SCAN_PROD> {
    using S = SumState;
    static __device__ __forceinline__ S identity() { return {1.0f}; }
    static __device__ __forceinline__ S lift(float x, float) { return {x}; }
    static __device__ __forceinline__ S combine(S l, S r) { return {l.v * r.v}; }
    static __device__ __forceinline__ float observe(S s) { return s.v; }
};
template <> struct Fold<TB200_SCAN_MAX> {
    using S = SumState;
    static __device__ __forceinline__ S identity() { return {-INFINITY}; }
    static __device__ __forceinline__ S lift(float x, float) { return {x}; }
    static __device__ __forceinline__ S combine(S l, S r) { return {fmaxf(l.v, r.v)}; }
    static __device__ __forceinline__ float observe(S s) { return s.v; }
};
template <> struct Fold<TB200_SCAN_MIN> {
    using S = SumState;
    static __device__ __forceinline__ S identity() { return {INFINITY}; }
    static __device__ __forceinline__ S lift(float x, float) { return {x}; }
    static __device__ __forceinline__ S combine(S l, S r) { return {fminf(l.v, r.v)}; }
    static __device__ __forceinline__ float observe(S s) { return s.v; }
};
// combine((a1, b1), (a2, b2)) = (a2 a1, a2 b1 + b2), observe = last, from init (1, 0): h_t = a_t h_{t-1} + b_t
template <> struct Fold<TB200_SCAN_AFFINE> {
    using S = AffineState;
    static __device__ __forceinline__ S identity() { return {1.0f, 0.0f}; }
    static __device__ __forceinline__ S lift(float a, float b) { return {a, b}; }
    static __device__ __forceinline__ S combine(S l, S r) { return {r.a * l.a, fmaf(r.a, l.b, r.b)}; }
    static __device__ __forceinline__ float observe(S s) { return s.b; }
};
// Welford's state merged Chan's way; observe = m2 / n, the population variance of the prefix
template <> struct Fold<TB200_SCAN_VARIANCE> {
    using S = MomentState;
    static __device__ __forceinline__ S identity() { return {0.0f, 0.0f, 0.0f}; }
    static __device__ __forceinline__ S lift(float x, float) { return {1.0f, x, 0.0f}; }
    static __device__ __forceinline__ S combine(S l, S r) {
        const float n = l.n + r.n;
        if (n == 0.0f) return {0.0f, 0.0f, 0.0f};
        // counts are small whole numbers: the approximate division (two ulp) is far inside the scans' tolerance, and
        // an IEEE division per element was what a running variance spent its time on
        const float d = r.mean - l.mean, w = __fdividef(r.n, n);
        return {n, fmaf(d, w, l.mean), l.m2 + r.m2 + d * d * l.n * w};
    }
    static __device__ __forceinline__ float observe(S s) { return s.n > 0.0f ? __fdividef(s.m2, s.n) : 0.0f; }
};

template <typename S> struct Words { static constexpr int N = sizeof(S) / 4; };

template <typename S>
__device__ __forceinline__ S shuffle_up(S s, int delta) {
    union { S s; float f[Words<S>::N]; } u;
    u.s = s;
#pragma unroll
    for (int i = 0; i < Words<S>::N; i++) u.f[i] = __shfl_up_sync(0xffffffffu, u.f[i], delta);
    return u.s;
}

template <typename T> __device__ __forceinline__ float load1(const T *p);
template <> __device__ __forceinline__ float load1<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float load1<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void store1(T *p, float v);
template <> __device__ __forceinline__ void store1<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void store1<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

struct ScanArgs {
    const void *x, *x2;
    void *y;
    long long n, rows, batch;
    long long ld_x, ld_x2, ld_y;            // row pitches, elements
    long long stride_x, stride_x2, stride_y;   // between the matrices of the batch
    int reverse;
    int vec;   // along rows: every row is a whole number of 16-byte aligned groups of eight elements
    int slabs;       // across rows: runs the rows are cut into (1: one thread walks a column)
    int quad;        // across rows in slabs: every row is a whole number of aligned groups of four columns
    float *totals;   // the slabs' totals (caller's workspace)
};

// ---- along each row
// eight neighbouring elements of a row as one or two 128-bit accesses (`p` 16-byte aligned)
__device__ __forceinline__ void load8(const float *p, float (&v)[8]) {
    const float4 lo = __ldcs(reinterpret_cast<const float4 *>(p)), hi = __ldcs(reinterpret_cast<const float4 *>(p) + 1);
    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16 *p, float (&v)[8]) {
    const uint4 q = __ldcs(reinterpret_cast<const uint4 *>(p));
    unpack_bf16x2(q.x, v[0], v[1]); unpack_bf16x2(q.y, v[2], v[3]);
    unpack_bf16x2(q.z, v[4], v[5]); unpack_bf16x2(q.w, v[6], v[7]);
}
__device__ __forceinline__ void store8(float *p, const float (&v)[8]) {
    __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
    __stcs(reinterpret_cast<float4 *>(p) + 1, make_float4(v[4], v[5], v[6], v[7]));
}
__device__ __forceinline__ void store8(__nv_bfloat16 *p, const float (&v)[8]) {
    __stcs(reinterpret_cast<uint4 *>(p), make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                                    pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7])));
}

template <int OP, typename T>
__global__ void __launch_bounds__(kScanThreads) scan_rows_kernel(const ScanArgs a) {
    using F = Fold<OP>;
    using S = typename F::S;
    __shared__ S warp_total[2][kScanThreads / 32];   // two buffers, tiles alternate: one barrier per tile
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int turn = 0;
    for (long long item = blockIdx.x; item < a.rows * a.batch; item += gridDim.x) {
        const long long m = item / a.rows, row = item - m * a.rows;
        const T *x = static_cast<const T *>(a.x) + m * a.stride_x + row * a.ld_x;
        const T *x2 = a.x2 ? static_cast<const T *>(a.x2) + m * a.stride_x2 + row * a.ld_x2 : nullptr;
        T *y = static_cast<T *>(a.y) + m * a.stride_y + row * a.ld_y;
        S carry = F::identity();
        for (long long base = 0; base < a.n; base += kScanThreads * kScanPer, turn ^= 1) {
            // this thread's eight consecutive scan positions; position p is element p, or n - 1 - p when reversed
            const long long p0 = base + threadIdx.x * kScanPer;
            // with 128-bit accesses (every row a whole number of aligned groups of eight) a thread's eight
            // positions are all inside the row or all outside; reversed, they are the mirrored group read backwards
            const bool whole = a.vec && p0 < a.n;
            const long long i0 = a.reverse ? a.n - kScanPer - p0 : p0;
            float v[kScanPer], v2[kScanPer];
            if (whole) {
                load8(x + i0, v);
                if (x2) load8(x2 + i0, v2);
            }
            S local[kScanPer];
            S run = F::identity();
#pragma unroll
            for (int e = 0; e < kScanPer; e++) {
                const long long p = p0 + e;
                S s = F::identity();
                if (whole) {
                    const int at = a.reverse ? kScanPer - 1 - e : e;
                    s = F::lift(v[at], x2 ? v2[at] : 0.0f);
                } else if (!a.vec && p < a.n) {
                    const long long i = a.reverse ? a.n - 1 - p : p;
                    s = F::lift(load1(x + i), x2 ? load1(x2 + i) : 0.0f);
                }
                run = F::combine(run, s);
                local[e] = run;
            }
            // inclusive scan of the threads' totals inside the warp, then of the warps' totals
            S incl = run;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const S left = shuffle_up(incl, d);
                if (lane >= d) incl = F::combine(left, incl);
            }
            if (lane == 31) warp_total[turn][warp] = incl;
            __syncthreads();
            // everything ahead of this thread: earlier tiles, warps, lanes; and the carry for the next tile
            S before = carry, running = carry;
#pragma unroll
            for (int w = 0; w < kScanThreads / 32; w++) {
                if (w == warp) before = running;
                running = F::combine(running, warp_total[turn][w]);
            }
            carry = running;
            const S lane_excl = shuffle_up(incl, 1);
            if (lane > 0) before = F::combine(before, lane_excl);
            if (whole) {
#pragma unroll
                for (int e = 0; e < kScanPer; e++)
                    v[a.reverse ? kScanPer - 1 - e : e] = F::observe(F::combine(before, local[e]));
                store8(y + i0, v);
            } else if (!a.vec) {
#pragma unroll
                for (int e = 0; e < kScanPer; e++) {
                    const long long p = p0 + e;
                    if (p < a.n) {
                        const long long i = a.reverse ? a.n - 1 - p : p;
                        store1(y + i, F::observe(F::combine(before, local[e])));
                    }
                }
            }
        }
    }
}

// ---- across the rows: one thread per column
template <int OP, typename T>
__global__ void __launch_bounds__(kScanThreads) scan_columns_kernel(const ScanArgs a) {
    using F = Fold<OP>;
    using S = typename F::S;
    const long long col = blockIdx.x * static_cast<long long>(kScanThreads) + threadIdx.x;
    if (col >= a.n) return;
    for (long long m = blockIdx.y; m < a.batch; m += gridDim.y) {
        const T *x = static_cast<const T *>(a.x) + m * a.stride_x + col;
        const T *x2 = a.x2 ? static_cast<const T *>(a.x2) + m * a.stride_x2 + col : nullptr;
        T *y = static_cast<T *>(a.y) + m * a.stride_y + col;
        S run = F::identity();
        // eight rows' loads are issued before the first is used: the chain through `run` is arithmetic only, so
        // the walk waits for memory once per eight rows instead of once per row
        constexpr int B = 8;
        for (long long p0 = 0; p0 < a.rows; p0 += B) {
            float v[B], w[B];
#pragma unroll
            for (int j = 0; j < B; j++) {
                const long long p = p0 + j < a.rows ? p0 + j : a.rows - 1;
                const long long r = a.reverse ? a.rows - 1 - p : p;
                v[j] = load1(x + r * a.ld_x);
                w[j] = x2 ? load1(x2 + r * a.ld_x2) : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < B; j++) {
                if (p0 + j < a.rows) {
                    const long long r = a.reverse ? a.rows - 1 - (p0 + j) : p0 + j;
                    run = F::combine(run, F::lift(v[j], w[j]));
                    store1(y + r * a.ld_y, F::observe(run));
                }
            }
        }
    }
}

// ---- across the rows, in slabs: the rows are cut into `slabs` runs; first every (slab, column) folds its run to a
// total (kept in the workspace as the state's Float32 words, [slab][word][column]), then every (slab, column) folds
// the totals of the slabs before it, in order, and sweeps its run again from there.  Two reads and one write per
// element; which states are combined in which order is fixed by the shape alone.
template <int OP, typename T, bool WRITE>
__global__ void __launch_bounds__(kScanThreads) scan_slabs_kernel(const ScanArgs a, float *totals, int slabs, long long per) {
    using F = Fold<OP>;
    using S = typename F::S;
    constexpr int W = Words<S>::N;
    const long long col = blockIdx.x * static_cast<long long>(kScanThreads) + threadIdx.x;
    if (col >= a.n) return;
    const int slab = blockIdx.y;
    for (long long m = blockIdx.z; m < a.batch; m += gridDim.z) {
        const T *x = static_cast<const T *>(a.x) + m * a.stride_x + col;
        const T *x2 = a.x2 ? static_cast<const T *>(a.x2) + m * a.stride_x2 + col : nullptr;
        T *y = static_cast<T *>(a.y) + m * a.stride_y + col;
        float *mine = totals + (m * slabs * W) * a.n + col;   // [slab][word] at this column
        union { S s; float f[W]; } u;
        S run = F::identity();
        if (WRITE) {
            for (int b = 0; b < slab; b++) {
#pragma unroll
                for (int w = 0; w < W; w++) u.f[w] = mine[(static_cast<long long>(b) * W + w) * a.n];
                run = F::combine(run, u.s);
            }
        }
        const long long p_begin = slab * per, p_end = p_begin + per < a.rows ? p_begin + per : a.rows;
        constexpr int B = 8;
        for (long long p0 = p_begin; p0 < p_end; p0 += B) {
            float v[B], w2[B];
#pragma unroll
            for (int j = 0; j < B; j++) {
                const long long p = p0 + j < p_end ? p0 + j : p_end - 1;
                const long long r = a.reverse ? a.rows - 1 - p : p;
                v[j] = load1(x + r * a.ld_x);
                w2[j] = x2 ? load1(x2 + r * a.ld_x2) : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < B; j++) {
                if (p0 + j < p_end) {
                    run = F::combine(run, F::lift(v[j], w2[j]));
                    if (WRITE) {
                        const long long r = a.reverse ? a.rows - 1 - (p0 + j) : p0 + j;
                        store1(y + r * a.ld_y, F::observe(run));
                    }
                }
            }
        }
        if (!WRITE) {
            u.s = run;
#pragma unroll
            for (int w = 0; w < W; w++) mine[(static_cast<long long>(slab) * W + w) * a.n] = u.f[w];
        }
    }
}

// four neighbouring columns of one row as one access (128 bits of Float32, 64 of BFloat16; `p` aligned to that),
// kept as loaded until they are used.  `keep`: the line is wanted again soon (the totals' sweep leaves the head of
// every slab in L2 for the second sweep)
template <typename T> struct Quad;
template <> struct Quad<float> {
    using Raw = float4;
    static __device__ __forceinline__ Raw load(const float *p, bool keep) {
        return keep ? __ldg(reinterpret_cast<const float4 *>(p)) : __ldcs(reinterpret_cast<const float4 *>(p));
    }
    static __device__ __forceinline__ void unpack(const Raw &q, float (&v)[4]) { v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
    static __device__ __forceinline__ void store(float *p, const float (&v)[4]) {
        __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
    }
};
template <> struct Quad<__nv_bfloat16> {
    using Raw = uint2;
    static __device__ __forceinline__ Raw load(const __nv_bfloat16 *p, bool keep) {
        return keep ? __ldg(reinterpret_cast<const uint2 *>(p)) : __ldcs(reinterpret_cast<const uint2 *>(p));
    }
    static __device__ __forceinline__ void unpack(const Raw &q, float (&v)[4]) {
        unpack_bf16x2(q.x, v[0], v[1]); unpack_bf16x2(q.y, v[2], v[3]);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float (&v)[4]) {
        __stcs(reinterpret_cast<uint2 *>(p), make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3])));
    }
};

// The same two sweeps with four columns a thread (rows that are whole aligned groups of four): a quarter of the
// instructions per byte, and the next rows' loads (B of them) are in flight while these are folded.  The totals'
// sweep walks its slab from the last row to the first, putting each element *before* what it has (the folds are
// associative, so the total is the same product of the same elements in the same order, grouped from the right);
// it ends on the rows the second sweep begins with, which are then still in L2.
template <int OP, typename T, bool WRITE>
__global__ void __launch_bounds__(kScanThreads, 2) scan_slabs_quad_kernel(const ScanArgs a, float *totals, int slabs,
                                                                           long long per) {
    using F = Fold<OP>;
    using S = typename F::S;
    constexpr int W = Words<S>::N;
    constexpr bool PAIRS = OP == TB200_SCAN_AFFINE;
    using Q = Quad<T>;
    using Raw = typename Q::Raw;
    constexpr int B = sizeof(T) == 2 ? (PAIRS ? 6 : 12) : (PAIRS ? 4 : 8);   // rows in flight: 96-128 bytes a thread per array
    const long long col = (blockIdx.x * static_cast<long long>(kScanThreads) + threadIdx.x) * 4;
    if (col >= a.n) return;
    const int slab = blockIdx.y;
    const long long p_begin = slab * per, p_end = p_begin + per < a.rows ? p_begin + per : a.rows;
    const long long count = p_end - p_begin;
    for (long long m = blockIdx.z; m < a.batch; m += gridDim.z) {
        const T *x = static_cast<const T *>(a.x) + m * a.stride_x + col;
        const T *x2 = PAIRS ? static_cast<const T *>(a.x2) + m * a.stride_x2 + col : nullptr;
        T *y = static_cast<T *>(a.y) + m * a.stride_y + col;
        float *mine = totals + (m * slabs * W) * a.n + col;   // [slab][word] at these columns
        union State { S s; float f[W]; };
        S run[4];
#pragma unroll
        for (int c = 0; c < 4; c++) run[c] = F::identity();
        if (WRITE) {
            for (int b = 0; b < slab; b++) {
                float4 t[W];
#pragma unroll
                for (int w = 0; w < W; w++)
                    t[w] = *reinterpret_cast<const float4 *>(mine + (static_cast<long long>(b) * W + w) * a.n);
                State u[4];
#pragma unroll
                for (int w = 0; w < W; w++) { u[0].f[w] = t[w].x; u[1].f[w] = t[w].y; u[2].f[w] = t[w].z; u[3].f[w] = t[w].w; }
#pragma unroll
                for (int c = 0; c < 4; c++) run[c] = F::combine(run[c], u[c].s);
            }
        }
        // the i-th row this sweep visits: forward from the slab's first when writing, backward from its last when not
        const auto row_of = [&](long long i) {
            if (i >= count) i = count - 1;
            const long long p = WRITE ? p_begin + i : p_end - 1 - i;
            return a.reverse ? a.rows - 1 - p : p;
        };
        Raw cv[B], cw[B], nv[B], nw[B];
        if (count > 0) {   // (a slab past the last row has none: its total is the identity)
#pragma unroll
            for (int j = 0; j < B; j++) {
                const long long r = row_of(j);
                cv[j] = Q::load(x + r * a.ld_x, !WRITE);
                if (PAIRS) cw[j] = Q::load(x2 + r * a.ld_x2, !WRITE);
            }
        }
        for (long long i0 = 0; i0 < count; i0 += B) {
            if (i0 + B < count) {
#pragma unroll
                for (int j = 0; j < B; j++) {
                    const long long r = row_of(i0 + B + j);
                    nv[j] = Q::load(x + r * a.ld_x, !WRITE);
                    if (PAIRS) nw[j] = Q::load(x2 + r * a.ld_x2, !WRITE);
                }
            }
#pragma unroll
            for (int j = 0; j < B; j++) {
                if (i0 + j < count) {
                    float v[4], w[4] = {0.0f, 0.0f, 0.0f, 0.0f}, out[4];
                    Q::unpack(cv[j], v);
                    if (PAIRS) Q::unpack(cw[j], w);
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const S e = F::lift(v[c], w[c]);
                        run[c] = WRITE ? F::combine(run[c], e) : F::combine(e, run[c]);
                        out[c] = F::observe(run[c]);
                    }
                    if (WRITE) Q::store(y + row_of(i0 + j) * a.ld_y, out);
                }
            }
#pragma unroll
            for (int j = 0; j < B; j++) {
                cv[j] = nv[j];
                if (PAIRS) cw[j] = nw[j];
            }
        }
        if (!WRITE) {
            State u[4];
#pragma unroll
            for (int c = 0; c < 4; c++) u[c].s = run[c];
#pragma unroll
            for (int w = 0; w < W; w++)
                *reinterpret_cast<float4 *>(mine + (static_cast<long long>(slab) * W + w) * a.n) =
                    make_float4(u[0].f[w], u[1].f[w], u[2].f[w], u[3].f[w]);
        }
    }
}

// Slabs for a scan across `rows` rows of `n` columns: enough blocks to fill the device eight times over, at least
// 64 rows a slab; 1 = not worth splitting.
inline int scan_slabs(long long n, long long rows, long long batch, int sms) {
    const long long col_blocks = ceil_div(n, kScanThreads) * (batch < 1 ? 1 : batch);
    long long slabs = ceil_div(static_cast<long long>(sms) * 8, col_blocks);
    if (slabs > rows / 64) slabs = rows / 64;
    if (slabs > 1024) slabs = 1024;
    return static_cast<int>(slabs < 1 ? 1 : slabs);
}
inline size_t scan_slab_bytes(int op, long long n, long long batch, int slabs) {
    const int words = op == TB200_SCAN_AFFINE ? 2 : op == TB200_SCAN_VARIANCE ? 3 : 1;
    return slabs <= 1 ? 0 : static_cast<size_t>(slabs) * words * n * (batch < 1 ? 1 : batch) * sizeof(float);
}

template <int OP, typename T>
int launch_scan(const ScanArgs &a, bool across, const DeviceInfo &dev, cudaStream_t stream) {
    if (across && a.slabs > 1) {
        const long long per = ceil_div(a.rows, static_cast<long long>(a.slabs));
        if (a.quad) {
            dim3 grid(static_cast<unsigned>(ceil_div(a.n, 4ll * kScanThreads)), static_cast<unsigned>(a.slabs),
                      static_cast<unsigned>(a.batch < 64 ? a.batch : 64));
            scan_slabs_quad_kernel<OP, T, false><<<grid, kScanThreads, 0, stream>>>(a, a.totals, a.slabs, per);
            TB200_CUDA(cudaGetLastError());
            scan_slabs_quad_kernel<OP, T, true><<<grid, kScanThreads, 0, stream>>>(a, a.totals, a.slabs, per);
            TB200_CUDA(cudaGetLastError());
            return TB200_OK;
        }
        dim3 grid(static_cast<unsigned>(ceil_div(a.n, kScanThreads)), static_cast<unsigned>(a.slabs),
                  static_cast<unsigned>(a.batch < 64 ? a.batch : 64));
        scan_slabs_kernel<OP, T, false><<<grid, kScanThreads, 0, stream>>>(a, a.totals, a.slabs, per);
        TB200_CUDA(cudaGetLastError());
        scan_slabs_kernel<OP, T, true><<<grid, kScanThreads, 0, stream>>>(a, a.totals, a.slabs, per);
        TB200_CUDA(cudaGetLastError());
        return TB200_OK;
    }
    if (across) {
        dim3 grid(static_cast<unsigned>(ceil_div(a.n, kScanThreads)), static_cast<unsigned>(a.batch < 65535 ? a.batch : 65535));
        scan_columns_kernel<OP, T><<<grid, kScanThreads, 0, stream>>>(a);
    } else {
        const long long items = a.rows * a.batch;
        int per_sm = 0;   // persistent blocks: as many as are resident at once, so that no block starts late
        TB200_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, scan_rows_kernel<OP, T>, kScanThreads, 0));
        const long long most = static_cast<long long>(dev.sms) * (per_sm > 0 ? per_sm : 1);
        scan_rows_kernel<OP, T><<<static_cast<unsigned>(items < most ? items : most), kScanThreads, 0, stream>>>(a);
    }
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

template <typename T>
int launch_by_op(int op, const ScanArgs &a, bool across, const DeviceInfo &dev, cudaStream_t stream) {
    switch (op) {
        case TB200_SCAN_SUM: return launch_scan<TB200_SCAN_SUM, T>(a, across, dev, stream);
        case TB200_SCAN_PROD: return launch_scan<TB200_SCAN_PROD, T>(a, across, dev, stream);
        case TB200_SCAN_MAX: return launch_scan<TB200_SCAN_MAX, T>(a, across, dev, stream);
        case TB200_SCAN_MIN: return launch_scan<TB200_SCAN_MIN, T>(a, across, dev, stream);
        case TB200_SCAN_AFFINE: return launch_scan<TB200_SCAN_AFFINE, T>(a, across, dev, stream);
        case TB200_SCAN_VARIANCE: return launch_scan<TB200_SCAN_VARIANCE, T>(a, across, dev, stream);
        default: return TB200_ERR_UNSUPPORTED;
    }
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" size_t tb200_scan_workspace_bytes(const tb200_scan_desc *d) {
    if (!d || !d->across || d->n <= 0 || d->rows <= 0 || d->op < TB200_SCAN_SUM || d->op > TB200_SCAN_VARIANCE) return 0;
    DeviceInfo dev;
    if (current_device(&dev) != TB200_OK) return 0;
    const long long batch = d->batch > 1 ? d->batch : 1;
    return scan_slab_bytes(d->op, d->n, batch, scan_slabs(d->n, d->rows, batch, dev.sms));
}

extern "C" int tb200_scan(const tb200_scan_desc *d, const void *x, const void *x2, void *y, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!d) return TB200_ERR_NULL;
    if (d->dtype != TB200_F32 && d->dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (d->op < TB200_SCAN_SUM || d->op > TB200_SCAN_VARIANCE) return TB200_ERR_UNSUPPORTED;
    const long long batch = d->batch > 1 ? d->batch : 1;
    if (d->n < 0 || d->rows < 0 || d->batch < 0 || d->ld_x < d->n || d->ld_y < d->n) return TB200_ERR_SHAPE;
    const bool pairs = d->op == TB200_SCAN_AFFINE;
    if (pairs && d->ld_x2 < d->n) return TB200_ERR_SHAPE;
    if (d->n == 0 || d->rows == 0) return TB200_OK;
    if (!x || !y || (pairs && !x2)) return TB200_ERR_NULL;
    const size_t es = dtype_size(d->dtype);
    if (!aligned_to(x, es) || !aligned_to(y, es) || !aligned_to(x2, es)) return TB200_ERR_ALIGN;
    if (batch > 1 && (d->stride_x < 0 || d->stride_y < (d->rows - 1) * d->ld_y + d->n)) return TB200_ERR_SHAPE;
    DeviceInfo dev;
    int st = current_device(&dev);
    if (st) return st;
    ScanArgs a{};
    a.x = x; a.x2 = pairs ? x2 : nullptr; a.y = y;
    a.n = d->n; a.rows = d->rows; a.batch = batch;
    a.ld_x = d->ld_x; a.ld_x2 = d->ld_x2; a.ld_y = d->ld_y;
    a.stride_x = d->stride_x; a.stride_x2 = d->stride_x2; a.stride_y = d->stride_y;
    a.reverse = d->reverse != 0;
    {
        const long long per = 16 / static_cast<long long>(es);   // elements per 128-bit access
        const bool pitches = a.ld_x % per == 0 && a.ld_y % per == 0 && (!pairs || a.ld_x2 % per == 0) &&
                             (batch == 1 || (a.stride_x % per == 0 && a.stride_y % per == 0 && (!pairs || a.stride_x2 % per == 0)));
        a.vec = !d->across && a.n % 8 == 0 && pitches && aligned_to(x, 16) && aligned_to(y, 16) && (!pairs || aligned_to(x2, 16));
    }
    a.slabs = 1;
    if (d->across && d->workspace) {
        const int slabs = scan_slabs(d->n, d->rows, batch, dev.sms);
        const size_t need = scan_slab_bytes(d->op, d->n, batch, slabs);
        if (need) {
            if (d->workspace_bytes < need || !aligned_to(d->workspace, 16)) return TB200_ERR_WORKSPACE;
            a.slabs = slabs;
            a.totals = static_cast<float *>(d->workspace);
            const bool pitches4 = a.n % 4 == 0 && a.ld_x % 4 == 0 && a.ld_y % 4 == 0 && (!pairs || a.ld_x2 % 4 == 0) &&
                                  (batch == 1 || (a.stride_x % 4 == 0 && a.stride_y % 4 == 0 && (!pairs || a.stride_x2 % 4 == 0)));
            a.quad = pitches4 && aligned_to(x, 4 * es) && aligned_to(y, 4 * es) && (!pairs || aligned_to(x2, 4 * es));
        }
    }
    if (d->dtype == TB200_F32) return launch_by_op<float>(d->op, a, d->across != 0, dev, stream);
    return launch_by_op<__nv_bfloat16>(d->op, a, d->across != 0, dev, stream);
}
