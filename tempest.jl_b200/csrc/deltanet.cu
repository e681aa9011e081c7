// Chunked gated DeltaNet (delta-rule linear attention), forward and pullback, for sm_100a.
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
// the two 64 x 64 x 128 products as warp-level BFloat16 MMAs (exact products of the BFloat16 operands, Float32
// sums), (I + A)^-1 by 16 x 16 blocks as the reference's `blocks` does (examples/deltanet.jl:39-54: the diagonal
// blocks by substitution in Float32, the blocks below them by small products in 3xTF32), and
// [W | Ut] = (I + A)^-1 [beta e^ca K | beta V] as TF32 MMAs.  (The first version solved the 256 right-hand columns
// by forward substitution, one column per thread: 2016 dependent multiply-adds a thread; measured 1.61 -> 1.39 ms
// for the whole forward with the products on MMAs and the sums split four ways, and less again with the inverse.)
// `deltanet_scan_kernel` carries the state, one block per (head, 32 value features): the state
// slice (128 x 32 Float32) lives in shared memory for all 128 chunks and each chunk costs three small
// products, issued as TF32 warp-level MMAs with operands in shared memory and results in registers (each
// product feeds the next one of the chain at once; about 0.1 TFLOP in all).  The path is bound by the chain
// of chunks, not by the tensor cores or HBM; W, Ut and P are rounded to BFloat16 when they cross from one
// launch to the other.  The pullback (further down) recomputes the forward keeping the state at every chunk
// start, walks the chunks backwards for the state gradient, and finishes per chunk.
#include <mutex>

#include "common.cuh"
#include "sm100.cuh"

namespace tb200 {
namespace {

constexpr int kC = 64;        // chunk length
constexpr int kDK = 128;
constexpr int kDV = 128;
constexpr int kDVP = 32;      // value features per scan block
constexpr int kPadH = 136;    // BFloat16 row pitch of a 128-wide tile
constexpr int kPadP = 72;     // BFloat16 row pitch of a 64-wide tile


// Inclusive running sum of a chunk's 64 log-decay gates by one warp: lane l gets ca[l] and ca[l + 32].  (One
// thread adding them in turn would wait for 64 loads one after another at the head of every link of the
// chain of chunks.)
__device__ __forceinline__ void chunk_cumsum_of(int lane, float &lo, float &hi) {   // lo, hi: the gates themselves on entry
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const float l2 = __shfl_up_sync(0xffffffffu, lo, off), h2 = __shfl_up_sync(0xffffffffu, hi, off);
        if (lane >= off) { lo += l2; hi += h2; }
    }
    hi += __shfl_sync(0xffffffffu, lo, 31);
}
__device__ __forceinline__ void chunk_cumsum(const float *a, int lane, float &lo, float &hi) {
    lo = __ldg(a + lane);
    hi = __ldg(a + lane + 32);
    chunk_cumsum_of(lane, lo, hi);
}

// ---------------------------------------------------------------- within a chunk ----

// Warp-level BFloat16 tensor-core product step: D(16 x 8) += A(16 x 16) B(16 x 8), Float32 accumulate.  With
// g = lane / 4 and t = lane % 4 a thread holds A[g][2t, 2t+1], A[g+8][2t, 2t+1], A[g][2t+8, 2t+9], A[g+8][2t+8, 2t+9];
// B[2t, 2t+1][g], B[2t+8, 2t+9][g]; D[g][2t], D[g][2t+1], D[g+8][2t], D[g+8][2t+1].
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kGateFloats = 196;   // e^ca (64), e^(ca_C - ca) (64), beta (64), e^ca_C, padded to a multiple of 16 bytes
constexpr int kPadA = 68;   // Float32 row pitch of the 64 x 64 tiles A, (I + A)^-1 and the scratch beside them

// 3xTF32: a Float32 operand as the sum of two TF32 values; hi*hi + lo*hi + hi*lo keeps about 21 bits of the product.
__device__ __forceinline__ void split_tf32(float x, uint32_t &hi, uint32_t &lo) {
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
    const float rest = x - __uint_as_float(hi);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(rest));
}
__device__ __forceinline__ void mma_tf32_raw(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// acc(16 x 16) += L(16 x 16) R(16 x 16), both Float32 blocks of pitch-kPadA tiles, by one warp in 3xTF32.
__device__ __forceinline__ void block_product(float (&acc)[2][4], const float *L, const float *R, int lane) {
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int kk = 0; kk < 16; kk += 8) {
        uint32_t ah[4], al[4];
        split_tf32(L[g * kPadA + kk + t4], ah[0], al[0]);
        split_tf32(L[(g + 8) * kPadA + kk + t4], ah[1], al[1]);
        split_tf32(L[g * kPadA + kk + t4 + 4], ah[2], al[2]);
        split_tf32(L[(g + 8) * kPadA + kk + t4 + 4], ah[3], al[3]);
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            uint32_t bh0, bl0, bh1, bl1;
            split_tf32(R[(kk + t4) * kPadA + 8 * nt + g], bh0, bl0);
            split_tf32(R[(kk + t4 + 4) * kPadA + 8 * nt + g], bh1, bl1);
            mma_tf32_raw(acc[nt], al, bh0, bh1);
            mma_tf32_raw(acc[nt], ah, bl0, bl1);
            mma_tf32_raw(acc[nt], ah, bh0, bh1);
        }
    }
}
__device__ __forceinline__ void block_store(float *dst, const float (&acc)[2][4], int lane, float sign) {
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
        *reinterpret_cast<float2 *>(dst + g * kPadA + 8 * nt + 2 * t4) = make_float2(sign * acc[nt][0], sign * acc[nt][1]);
        *reinterpret_cast<float2 *>(dst + (g + 8) * kPadA + 8 * nt + 2 * t4) = make_float2(sign * acc[nt][2], sign * acc[nt][3]);
    }
}

// One block of 256 threads per (head, chunk).  minv_save (the backward's first launch) receives (I + A)^-1, rounded.
__device__ __forceinline__ uint32_t tf32_bits(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

__global__ void __launch_bounds__(256, 3) deltanet_chunk_kernel(const __nv_bfloat16 *q, const __nv_bfloat16 *k,
                                                             const __nv_bfloat16 *v, const float *a, const float *beta,
                                                             __nv_bfloat16 *w_out, __nv_bfloat16 *u_out,
                                                             __nv_bfloat16 *p_out, __nv_bfloat16 *minv_save,
                                                             float *gates_out, int T) {
    extern __shared__ float sm[];
    float *A = sm;                        // [64][68]
    float *Mi = A + kC * kPadA;           // [64][68]  (I + A)^-1
    float *ca = Mi + kC * kPadA;          // [64]
    float *be = ca + kC;                  // [64]
    float *sk = be + kC;                  // [64]  beta e^ca: the scale of K's rows on the right-hand side
    __nv_bfloat16 *Kh = reinterpret_cast<__nv_bfloat16 *>(sk + kC);   // [64][136]
    __nv_bfloat16 *Qh = Kh + kC * kPadH;                              // [64][136]: Q, then (once A and P are formed) V
    __nv_bfloat16 *Vh = Qh;
    const int chunks = T / kC;
    const int head = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const long long row0 = static_cast<long long>(head) * T + static_cast<long long>(chunk) * kC;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;

    for (int i = tid; i < kC * kDK / 8; i += blockDim.x) {
        const int r = i / (kDK / 8), c = (i % (kDK / 8)) * 8;
        *reinterpret_cast<uint4 *>(Kh + r * kPadH + c) = __ldg(reinterpret_cast<const uint4 *>(k + (row0 + r) * kDK + c));
        *reinterpret_cast<uint4 *>(Qh + r * kPadH + c) = __ldg(reinterpret_cast<const uint4 *>(q + (row0 + r) * kDK + c));
    }
    if (tid < 32) {
        float lo, hi;
        chunk_cumsum(a + row0, tid, lo, hi);
        const float b0 = beta[row0 + tid], b1 = beta[row0 + tid + 32];
        ca[tid] = lo; ca[tid + 32] = hi;
        be[tid] = b0; be[tid + 32] = b1;
        sk[tid] = b0 * __expf(lo); sk[tid + 32] = b1 * __expf(hi);
    }
    __syncthreads();
    // what the scan across the chunks needs of the gates: e^ca, e^(ca_C - ca) and e^ca_C, kGateFloats a chunk
    if (tid < kC) {
        float *dst = gates_out + (static_cast<long long>(head) * chunks + chunk) * kGateFloats;
        const float last = ca[kC - 1];
        dst[tid] = __expf(ca[tid]);
        dst[kC + tid] = __expf(last - ca[tid]);
        dst[2 * kC + tid] = be[tid];
        if (tid == 0) dst[3 * kC] = __expf(last);
    }

    // A = beta .* decay(t > s) .* (K K'), P = decay(t >= s) .* (Q K') on the tensor cores: the operands are BFloat16 as
    // they arrive, so the products are exact and only the order of the Float32 additions differs from a sequential
    // sum.  Warp w takes rows 16 (w % 4) .. + 15 and columns 32 (w / 4) .. + 31 (four 8-column tiles) of both; both
    // operands are read along the feature axis from the row-major tiles (pitch 136: the 32 lanes of a fragment read hit
    // 32 banks).  Tiles wholly above the diagonal are skipped.
    {
        const int m0 = 16 * (warp & 3), n0 = 32 * (warp >> 2);
        float kk[4][4] = {}, qk[4][4] = {};
        const int live = n0 > m0 + 15 ? 0 : (m0 + 15 - n0) / 8 + 1;   // 8-column tiles that reach the diagonal
        if (live > 0) {
            for (int d = 0; d < kDK; d += 16) {
                uint32_t ak[4], aq[4];
                const __nv_bfloat16 *kr = Kh + (m0 + g) * kPadH + d + 2 * t4, *qr = Qh + (m0 + g) * kPadH + d + 2 * t4;
                ak[0] = *reinterpret_cast<const uint32_t *>(kr);
                ak[1] = *reinterpret_cast<const uint32_t *>(kr + 8 * kPadH);
                ak[2] = *reinterpret_cast<const uint32_t *>(kr + 8);
                ak[3] = *reinterpret_cast<const uint32_t *>(kr + 8 * kPadH + 8);
                aq[0] = *reinterpret_cast<const uint32_t *>(qr);
                aq[1] = *reinterpret_cast<const uint32_t *>(qr + 8 * kPadH);
                aq[2] = *reinterpret_cast<const uint32_t *>(qr + 8);
                aq[3] = *reinterpret_cast<const uint32_t *>(qr + 8 * kPadH + 8);
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (j < live) {
                        const __nv_bfloat16 *br = Kh + (n0 + 8 * j + g) * kPadH + d + 2 * t4;
                        const uint32_t b0 = *reinterpret_cast<const uint32_t *>(br), b1 = *reinterpret_cast<const uint32_t *>(br + 8);
                        mma_bf16(kk[j], ak, b0, b1);
                        mma_bf16(qk[j], aq, b0, b1);
                    }
            }
        }
        __nv_bfloat16 *pc = p_out + (static_cast<long long>(head) * chunks + chunk) * kC * kC;
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
                const int t = m0 + g + 8 * (e >> 1), s = n0 + 8 * j + 2 * t4;
                const float d0 = t >= s ? __expf(ca[t] - ca[s]) : 0.0f, d1 = t >= s + 1 ? __expf(ca[t] - ca[s + 1]) : 0.0f;
                A[t * kPadA + s] = t > s ? be[t] * d0 * kk[j][e] : 0.0f;
                A[t * kPadA + s + 1] = t > s + 1 ? be[t] * d1 * kk[j][e + 1] : 0.0f;
                *reinterpret_cast<uint32_t *>(pc + t * kC + s) = pack_bf16x2(d0 * qk[j][e], d1 * qk[j][e + 1]);
            }
    }
    __syncthreads();   // A is complete; Q's tile is free from here on: V takes its place (read again two phases on)
    for (int i = tid; i < kC * kDV / 8; i += blockDim.x) {
        const int r = i / (kDV / 8), c = (i % (kDV / 8)) * 8;
        *reinterpret_cast<uint4 *>(Vh + r * kPadH + c) = __ldg(reinterpret_cast<const uint4 *>(v + (row0 + r) * kDV + c));
    }

    // (I + A)^-1 by 16 x 16 blocks, as the reference's `blocks` does (examples/deltanet.jl:39-54).  Diagonal blocks:
    // 64 threads solve (I + A_ii) x = e_j by substitution, one column each, in Float32.
    if (tid < kC) {
        const int blk = tid >> 4, j = tid & 15;
        const float *D = A + (16 * blk) * kPadA + 16 * blk;
        float x[16];
#pragma unroll
        for (int r = 0; r < 16; r++) {
            float acc = r == j ? 1.0f : 0.0f;
#pragma unroll
            for (int c = 0; c < r; c++) acc = fmaf(-D[r * kPadA + c], x[c], acc);
            x[r] = acc;
        }
#pragma unroll
        for (int r = 0; r < 16; r++) Mi[(16 * blk + r) * kPadA + 16 * blk + j] = x[r];
    }
    __syncthreads();
    // Blocks below the diagonal, one distance from it at a time:  M_ij = -M_ii (sum_{j <= k < i} A_ik M_kj), each block
    // by one warp, products in 3xTF32 (close to Float32: the inverse is an operand of everything after it).
    for (int dist = 1; dist < 4; dist++) {
        if (warp < 4 - dist) {
            const int bi = warp + dist, bj = warp;
            float acc[2][4] = {};
            for (int bk = bj; bk < bi; bk++)
                block_product(acc, A + (16 * bi) * kPadA + 16 * bk, Mi + (16 * bk) * kPadA + 16 * bj, lane);
            // the sum is parked in the mirrored block above the diagonal (zero in the result, and nobody reads it:
            // it is cleared again below)
            float *scratch = Mi + (16 * bj) * kPadA + 16 * bi;
            block_store(scratch, acc, lane, 1.0f);
            __syncwarp();
            float out[2][4] = {};
            block_product(out, Mi + (16 * bi) * kPadA + 16 * bi, scratch, lane);
            block_store(Mi + (16 * bi) * kPadA + 16 * bj, out, lane, -1.0f);
        }
        __syncthreads();
    }
    if (minv_save)   // rounded: the reverse scan takes it as a BFloat16 operand
        for (int i = tid; i < kC * kC / 4; i += blockDim.x) {
            const int r = i / (kC / 4), c = (i % (kC / 4)) * 4;
            float4 m4 = *reinterpret_cast<const float4 *>(Mi + r * kPadA + c);
            if ((c >> 4) > (r >> 4)) m4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);   // blocks above the diagonal (scratch)
            *reinterpret_cast<uint2 *>(minv_save + (row0 + r) * kC + c) = make_uint2(pack_bf16x2(m4.x, m4.y), pack_bf16x2(m4.z, m4.w));
        }

    // [W | Ut] = (I + A)^-1 [beta e^ca K | beta V]: warp w takes rows 16 (w % 4) .. + 15 of the 128 columns of W
    // (w < 4) or of Ut, as TF32 MMAs (W and Ut leave as BFloat16, whose rounding is four times coarser than TF32's);
    // the right-hand side is formed from the BFloat16 tiles as the fragments are read, and the inverse's zero blocks
    // above the diagonal are skipped.
    {
        const int m0 = 16 * (warp & 3), side = warp >> 2;
        const __nv_bfloat16 *rhs = side ? Vh : Kh;
        const float *scale = side ? be : sk;
        __nv_bfloat16 *dst = (side ? u_out : w_out) + row0 * 128;
#pragma unroll 1
        for (int half = 0; half < 2; half++) {   // 64 columns at a time: half the accumulators in registers
            float acc[8][4] = {};
            for (int kk = 0; kk < m0 + 16; kk += 8) {
                uint32_t af[4];
                af[0] = tf32_bits(Mi[(m0 + g) * kPadA + kk + t4]);
                af[1] = tf32_bits(Mi[(m0 + g + 8) * kPadA + kk + t4]);
                af[2] = tf32_bits(Mi[(m0 + g) * kPadA + kk + t4 + 4]);
                af[3] = tf32_bits(Mi[(m0 + g + 8) * kPadA + kk + t4 + 4]);
                const float s0 = scale[kk + t4], s1 = scale[kk + t4 + 4];
                const __nv_bfloat16 *r0 = rhs + (kk + t4) * kPadH + 64 * half + g, *r1 = r0 + 4 * kPadH;
#pragma unroll
                for (int nt = 0; nt < 8; nt++) {
                    const uint32_t b0 = tf32_bits(s0 * __bfloat162float(r0[8 * nt]));
                    const uint32_t b1 = tf32_bits(s1 * __bfloat162float(r1[8 * nt]));
                    mma_tf32_raw(acc[nt], af, b0, b1);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                const int col = 64 * half + 8 * nt + 2 * t4;
                *reinterpret_cast<uint32_t *>(dst + (m0 + g) * 128 + col) = pack_bf16x2(acc[nt][0], acc[nt][1]);
                *reinterpret_cast<uint32_t *>(dst + (m0 + g + 8) * 128 + col) = pack_bf16x2(acc[nt][2], acc[nt][3]);
            }
        }
    }
}

// ----------------------------------------------------------------- across chunks ----


// Four 8 x 8 BFloat16 matrices from shared memory into a warp's registers, as the m16n8k16 fragments want them: each
// lane gives the address of one 16-byte row (lanes 0-7 the first matrix, 8-15 the second, ...); with `trans` the
// matrices arrive transposed (an operand stored with the other axis contiguous).
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void *row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(row))));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void *row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(row))));
}

__device__ int g_deltanet_error = 0;   // 1 once a wait for a chunk's tiles has given up

constexpr int kPadB = 40;   // BFloat16 row pitch of the 32-wide operand copies of the state and of U: ldmatrix rows hit 32 banks

// One block of 512 threads per (head, 64 value features) walks the chunks in order: two groups of eight warps, each
// with its own 32 features, share the chunk's W, Q, K and P tiles.  A group's state slice (128 x 32) lives in the
// accumulator registers of the product that updates it (warp w of the group: state rows 16 w .. + 15) for the whole
// sequence; what the other products read is a BFloat16 copy in shared memory, rewritten after every update -- the
// reference rounds the Float32 factor of a mixed product to the half type in the same way
// (ext/cuTileExt/emit.jl:914-921).  All four products of a chunk are BFloat16 m16n8k16 MMAs whose fragments come
// through ldmatrix (transposed where the operand lies the other way: the state and U as B operands, K' as an A
// operand), about 40 instructions a product a warp where the TF32 form with scalar fragment loads and conversions
// needed 300; the chain of chunks was bound by exactly those instructions (measured: 4.8 us a chunk, issue slots
// 42 % active).  Every tile has two buffers: the next chunk's tiles are copied asynchronously while this chunk's
// products run (a whole link of the chain ahead), and the next chunk's gates and Ut values are fetched meanwhile.
constexpr int kScanThreads = 512;
constexpr int kDVB = 64;          // value features per scan block (two groups of kDVP)
constexpr int kBoxBytes = kC * 128;        // a TMA box: 64 rows of 64 BFloat16 (one 128-byte swizzled line each)
constexpr int kTileSetBytes = 7 * kBoxBytes;   // one chunk's W, Q, K (two boxes each) and P (one)
struct ScanMaps { CUtensorMap w, q, k, p; };   // [rows][128] for W, Q, K; [heads * chunks * 64][64] for P

// Address of the 16-byte piece that holds (row, col .. col + 7) of a [64][128] tile kept as two 128-byte-swizzled
// boxes (or of a [64][64] tile: one box): what ldmatrix is given.
__device__ __forceinline__ const unsigned char *swz(const unsigned char *tile, int row, int col) {
    return tile + (col >> 6) * kBoxBytes + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4);
}

__global__ void __launch_bounds__(kScanThreads) deltanet_scan_kernel(const __grid_constant__ ScanMaps maps,
                                                                     const float *gates_in,
                                                                     const __nv_bfloat16 *u_in, __nv_bfloat16 *o,
                                                                     __nv_bfloat16 *s_save, __nv_bfloat16 *u_save, int T) {
    extern __shared__ unsigned char sm_raw[];
    // the tiles want 1024-byte alignment (the swizzle's period); the launch asks for 1 KB more than the layout
    unsigned char *tiles = sm_raw + ((1024u - (sm100::smem_u32(sm_raw) & 1023u)) & 1023u);   // [2][7 boxes]
    float *gate2 = reinterpret_cast<float *>(tiles + 2 * kTileSetBytes);   // [2][kGateFloats] the chunk's gates, per parity
    __nv_bfloat16 *group_base = reinterpret_cast<__nv_bfloat16 *>(gate2 + 2 * kGateFloats);
    __shared__ __align__(8) uint64_t tile_full[2];

    const int head = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31;
    const int group = tid >> 8, gtid = tid & 255, warp = (tid >> 5) & 7;   // warp: index inside the group
    const int part = blockIdx.y * (kDVB / kDVP) + group;                  // which 32 features
    const int g = lane >> 2, t4 = lane & 3;
    const int chunks = T / kC;
    // this group's operand copies and output staging
    __nv_bfloat16 *Sb2 = group_base + group * (2 * kDK * kPadB + 2 * kC * kPadB + kDVP * kPadP);   // [2][128][40] the state
    __nv_bfloat16 *Ub = Sb2 + 2 * kDK * kPadB;          // [64][40] U
    __nv_bfloat16 *Ud = Ub + kC * kPadB;                // [64][40] e^{ca_C - ca} U
    __nv_bfloat16 *Oh = Ud + kC * kPadB;                // [32][72] output staging, [feature][position]
    // ldmatrix lane -> (row, column) offsets inside a 16 x 16 operand block: `plain` for A operands stored
    // [row][k] and (transposed) for B operands stored [k][n]; `flip` for A operands stored [k][row]
    const int plain_r = (lane & 7) + 8 * ((lane >> 3) & 1), plain_c = 8 * (lane >> 4);
    const int flip_r = (lane & 7) + 8 * (lane >> 4), flip_c = 8 * ((lane >> 3) & 1);

    // U and o: warp -> 16 positions (mt) x 16 features (nh), two 8-feature tiles
    const int mt = warp & 3, nh = warp >> 2;
    const long long head_row = static_cast<long long>(head) * T;
    // A chunk's tiles arrive by TMA, seven boxes (four without a result to form) issued by one thread and counted in
    // bytes on the buffer's mbarrier.
    const uint32_t tile_bytes = (o ? 7u : 4u) * kBoxBytes + kGateFloats * 4u;
    auto copy_tiles = [&](int chunk) {
        if (tid != 0) return;
        unsigned char *set = tiles + (chunk & 1) * kTileSetBytes;
        uint64_t *bar = &tile_full[chunk & 1];
        const int row = static_cast<int>(head_row) + chunk * kC;
        sm100::mbar_arrive_expect_tx(bar, tile_bytes);
        sm100::bulk_load(gate2 + (chunk & 1) * kGateFloats, gates_in + (static_cast<long long>(head) * chunks + chunk) * kGateFloats,
                         kGateFloats * 4, bar);
        sm100::tma_load_2d(set, &maps.w, bar, 0, row);
        sm100::tma_load_2d(set + kBoxBytes, &maps.w, bar, 64, row);
        sm100::tma_load_2d(set + 4 * kBoxBytes, &maps.k, bar, 0, row);
        sm100::tma_load_2d(set + 5 * kBoxBytes, &maps.k, bar, 64, row);
        if (o) {
            sm100::tma_load_2d(set + 2 * kBoxBytes, &maps.q, bar, 0, row);
            sm100::tma_load_2d(set + 3 * kBoxBytes, &maps.q, bar, 64, row);
            sm100::tma_load_2d(set + 6 * kBoxBytes, &maps.p, bar, 0, (head * chunks + chunk) * kC);
        }
    };
    // Waits for a buffer's tiles, but not for ever: after about two seconds the thread records the failure and
    // goes on without waiting again, so that the launch ends and the host can read the status.
    bool gave_up = false;
    auto wait_tiles = [&](int chunk) {
        if (gave_up) return;
        uint64_t *bar = &tile_full[chunk & 1];
        const uint32_t parity = (chunk >> 1) & 1;
        if (sm100::mbar_wait(bar, parity, 4096)) return;
        unsigned long long t0, t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        while (!sm100::mbar_wait(bar, parity, 1024)) {
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > 2000000000ull) {
                gave_up = true;
                atomicCAS(&g_deltanet_error, 0, 1);
                return;
            }
        }
    };
    // Ut at this thread's accumulator positions, as the packed pairs they are stored in: unpacked where they are
    // used, a chunk later, so that nothing waits for these loads where they are issued
    auto fetch_ut = [&](int chunk, uint32_t (&raw)[2][2]) {
        const long long row0 = head_row + static_cast<long long>(chunk) * kC;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int hr = 0; hr < 2; hr++)
                raw[nt][hr] = __ldg(reinterpret_cast<const uint32_t *>(
                    u_in + (row0 + 16 * mt + g + 8 * hr) * kDV + part * kDVP + 16 * nh + 8 * nt + 2 * t4));
    };
    // the state rows of this warp as an operand copy: rows 16 warp + g (+8), columns 8 nt + 2 t4 (+1)
    auto put_state = [&](__nv_bfloat16 *Sb, const float (&st)[4][4]) {
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            *reinterpret_cast<uint32_t *>(Sb + (16 * warp + g) * kPadB + 8 * nt + 2 * t4) = pack_bf16x2(st[nt][0], st[nt][1]);
            *reinterpret_cast<uint32_t *>(Sb + (16 * warp + g + 8) * kPadB + 8 * nt + 2 * t4) = pack_bf16x2(st[nt][2], st[nt][3]);
        }
    };
    auto write_out = [&](int chunk) {   // the result is (positions, features): 128 contiguous bytes per feature
        const int f = gtid >> 3, c = (gtid & 7) * 8;
        *reinterpret_cast<uint4 *>(o + (static_cast<long long>(head) * kDV + part * kDVP + f) * T +
                                   static_cast<long long>(chunk) * kC + c) = *reinterpret_cast<const uint4 *>(Oh + f * kPadP + c);
    };

    float state[4][4] = {};
    uint32_t ut_raw[2][2];
    put_state(Sb2, state);
    if (tid == 0) {
        sm100::mbar_init(&tile_full[0], 1);
        sm100::mbar_init(&tile_full[1], 1);
        sm100::fence_barrier_init();
    }
    __syncthreads();
    if (chunks > 0) {
        copy_tiles(0);
        fetch_ut(0, ut_raw);
    }
    for (int chunk = 0; chunk < chunks; chunk++) {
        const long long row0 = head_row + static_cast<long long>(chunk) * kC;
        const float *eca = gate2 + (chunk & 1) * kGateFloats, *ekd = eca + kC;
        const unsigned char *Wt = tiles + (chunk & 1) * kTileSetBytes, *Qt = Wt + 2 * kBoxBytes, *Kt = Wt + 4 * kBoxBytes,
                            *Pt = Wt + 6 * kBoxBytes;
        const __nv_bfloat16 *Sb = Sb2 + (chunk & 1) * kDK * kPadB;
        const bool more = chunk + 1 < chunks;
        __syncthreads();   // this chunk's gates and state copy are in place; everything of the chunk before is done
        if (more) copy_tiles(chunk + 1);   // into the buffers the chunk before has left
        wait_tiles(chunk);
        if (o && chunk > 0) write_out(chunk - 1);
        if (s_save) {      // the state this chunk starts from, for the backward
            __nv_bfloat16 *dst = s_save + (static_cast<long long>(head) * chunks + chunk) * kDK * kDV + part * kDVP;
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                *reinterpret_cast<uint32_t *>(dst + (16 * warp + g) * kDV + 8 * nt + 2 * t4) = pack_bf16x2(state[nt][0], state[nt][1]);
                *reinterpret_cast<uint32_t *>(dst + (16 * warp + g + 8) * kDV + 8 * nt + 2 * t4) = pack_bf16x2(state[nt][2], state[nt][3]);
            }
        }

        // U = Ut - W S (the sum over the state rows in two halves, so that four accumulators are in flight)
        {
            float ws[2][4] = {}, ws2[2][4] = {};
#pragma unroll
            for (int k0 = 0; k0 < kDK / 2; k0 += 16) {
                uint32_t af[4], bf[4], af2[4], bf2[4];
                ldsm_x4(af, swz(Wt, 16 * mt + plain_r, k0 + plain_c));
                ldsm_x4_trans(bf, Sb + (k0 + plain_r) * kPadB + 16 * nh + plain_c);
                ldsm_x4(af2, swz(Wt, 16 * mt + plain_r, kDK / 2 + k0 + plain_c));
                ldsm_x4_trans(bf2, Sb + (kDK / 2 + k0 + plain_r) * kPadB + 16 * nh + plain_c);
                mma_bf16(ws[0], af, bf[0], bf[1]);
                mma_bf16(ws[1], af, bf[2], bf[3]);
                mma_bf16(ws2[0], af2, bf2[0], bf2[1]);
                mma_bf16(ws2[1], af2, bf2[2], bf2[3]);
            }
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) ws[nt][e] += ws2[nt][e];
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int hr = 0; hr < 2; hr++) {
                    float ut0, ut1;
                    unpack_bf16x2(ut_raw[nt][hr], ut0, ut1);
                    const float2 u2 = make_float2(ut0 - ws[nt][2 * hr], ut1 - ws[nt][2 * hr + 1]);
                    const int row = 16 * mt + g + 8 * hr, col = 16 * nh + 8 * nt + 2 * t4;
                    const float ed = ekd[row];
                    *reinterpret_cast<uint32_t *>(Ub + row * kPadB + col) = pack_bf16x2(u2.x, u2.y);
                    *reinterpret_cast<uint32_t *>(Ud + row * kPadB + col) = pack_bf16x2(ed * u2.x, ed * u2.y);
                    if (u_save) *reinterpret_cast<uint32_t *>(u_save + (row0 + row) * kDV + part * kDVP + col) = pack_bf16x2(u2.x, u2.y);
                }
        }
        __syncthreads();   // U is complete
        if (more) fetch_ut(chunk + 1, ut_raw);

        // S <- e^{ca_C} S + K' (e^{ca_C - ca} U): warp -> 16 state rows, all 32 features; then the operand copy for
        // the next chunk (the other buffer: this chunk's output product still reads the current one).
        // o = e^ca (Q S) + P U is off the chain: its MMAs are issued between the update's, whose four accumulators
        // each wait for their own previous step, so that the tensor pipe has independent work in the gaps.
        {
            const float gamma = eca[3 * kC];
#pragma unroll
            for (int nt = 0; nt < 4; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) state[nt][e] *= gamma;
            float oa[2][4] = {}, ob[2][4] = {};   // Q S and P U apart: the first is scaled by e^ca afterwards
            auto qs_step = [&](int k0) {
                uint32_t af[4], bf[4];
                ldsm_x4(af, swz(Qt, 16 * mt + plain_r, k0 + plain_c));
                ldsm_x4_trans(bf, Sb + (k0 + plain_r) * kPadB + 16 * nh + plain_c);
                mma_bf16(oa[0], af, bf[0], bf[1]);
                mma_bf16(oa[1], af, bf[2], bf[3]);
            };
            auto pu_step = [&](int k0) {
                uint32_t af[4], bf[4];
                ldsm_x4(af, swz(Pt, 16 * mt + plain_r, k0 + plain_c));
                ldsm_x4_trans(bf, Ub + (k0 + plain_r) * kPadB + 16 * nh + plain_c);
                mma_bf16(ob[0], af, bf[0], bf[1]);
                mma_bf16(ob[1], af, bf[2], bf[3]);
            };
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int k0 = 16 * j;
                uint32_t af[4], b0[4], b1[4];
                ldsm_x4_trans(af, swz(Kt, k0 + flip_r, 16 * warp + flip_c));
                ldsm_x4_trans(b0, Ud + (k0 + plain_r) * kPadB + plain_c);
                ldsm_x4_trans(b1, Ud + (k0 + plain_r) * kPadB + 16 + plain_c);
                mma_bf16(state[0], af, b0[0], b0[1]);
                mma_bf16(state[1], af, b0[2], b0[3]);
                mma_bf16(state[2], af, b1[0], b1[1]);
                mma_bf16(state[3], af, b1[2], b1[3]);
                if (o) {
                    qs_step(32 * j);
                    pu_step(16 * j);
                    qs_step(32 * j + 16);
                }
            }
            put_state(Sb2 + ((chunk + 1) & 1) * kDK * kPadB, state);
            if (o) {
                const float e0 = eca[16 * mt + g], e1 = eca[16 * mt + g + 8];
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
                    oa[nt][0] = fmaf(oa[nt][0], e0, ob[nt][0]); oa[nt][1] = fmaf(oa[nt][1], e0, ob[nt][1]);
                    oa[nt][2] = fmaf(oa[nt][2], e1, ob[nt][2]); oa[nt][3] = fmaf(oa[nt][3], e1, ob[nt][3]);
                }
#pragma unroll
                for (int nt = 0; nt < 2; nt++)
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        Oh[(16 * nh + 8 * nt + 2 * t4 + (e & 1)) * kPadP + 16 * mt + g + 8 * (e >> 1)] = __float2bfloat16_rn(oa[nt][e]);
            }
        }
    }
    if (o && chunks > 0) {
        __syncthreads();
        write_out(chunks - 1);
    }
}

// ------------------------------------------------------------------ the backward ----
//
// With e = exp(ca), ed = exp(ca_C - ca), g = exp(ca_C), D[t][s] = exp(ca_t - ca_s) for t >= s, S the state a
// chunk starts from, dS' the state gradient arriving from the chunks after it, and Minv = (I + A)^-1:
//   reverse scan   dU = P' dO + (ed K) dS';   dZ = Minv' dU;   dV = beta dZ
//                  dS = g dS' + (e Q)' dO - (e K)' (beta dZ)
//   per chunk      X = tril(dO U') .* D;   G = -stril(dZ U') .* D
//                  dQ = e (dO S') + X K
//                  dK = -(e beta) (dZ S') + ed (U dS'') + X' Q + beta (G K) + G' (beta K)
//                  dbeta = rowsum(dZ .* (V - e (K S))) + rowsum(K .* (G K))
//                  da = reverse cumulative sum within the chunk of the gradient of ca (below)
// It is the chain rule through examples/deltanet.jl:58-85 taken by hand; Tempest derives the same
// pullback from the forward program (examples/deltanet.jl:96-101).

// One block of 512 threads per (head, 64 value features), chunks walked last to first, built like the forward scan:
// two groups of eight warps with 32 features each share a chunk's K, Q, P and (I + A)^-1 tiles, which arrive by TMA
// into swizzled boxes in two buffers, a chunk ahead, together with each group's box of dO (read as it lies,
// [feature][position]) and the chunk's gates.  A group's slice of the state gradient lives in the accumulators of the
// product that updates it; the other products read a BFloat16 copy.  The four products are BFloat16 m16n8k16 MMAs
// through ldmatrix; the scalings along a summed axis go into the small operand as it is written (e into a copy of
// dO, -e beta into the copy of dZ).
struct BwdScanMaps { CUtensorMap k, q, p, minv, dout; };
constexpr int kBwdSetBytes = 6 * kBoxBytes + 2 * (kDVP * 128);   // K, Q (two boxes each), P, Minv; dO for two groups

__device__ __forceinline__ const unsigned char *swz_row128(const unsigned char *tile, int row, int col) {   // one box
    return tile + row * 128 + (((col >> 3) ^ (row & 7)) << 4);
}

__global__ void __launch_bounds__(kScanThreads) deltanet_bwd_scan_kernel(const __grid_constant__ BwdScanMaps maps,
                                                                         const float *gates_in, __nv_bfloat16 *dsin_save,
                                                                         __nv_bfloat16 *dz_save, __nv_bfloat16 *dv_out, int T) {
    extern __shared__ unsigned char sm_raw[];
    unsigned char *tiles = sm_raw + ((1024u - (sm100::smem_u32(sm_raw) & 1023u)) & 1023u);   // [2] sets
    float *gate2 = reinterpret_cast<float *>(tiles + 2 * kBwdSetBytes);   // [2][kGateFloats]
    __nv_bfloat16 *group_base = reinterpret_cast<__nv_bfloat16 *>(gate2 + 2 * kGateFloats);
    __shared__ __align__(8) uint64_t tile_full[2];

    const int head = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31;
    const int group = tid >> 8, gtid = tid & 255, warp = (tid >> 5) & 7;
    const int part = blockIdx.y * (kDVB / kDVP) + group;
    const int g = lane >> 2, t4 = lane & 3;
    const int chunks = T / kC;
    constexpr int kGroupElems = 2 * kDK * kPadB + 2 * kC * kPadB + kDVP * kPadP;
    __nv_bfloat16 *Sb2 = group_base + group * kGroupElems;   // [2][128][40] the state gradient as an operand
    __nv_bfloat16 *Ub = Sb2 + 2 * kDK * kPadB;               // [64][40] dU
    __nv_bfloat16 *Zs = Ub + kC * kPadB;                     // [64][40] -e beta dZ
    __nv_bfloat16 *Oe = Zs + kC * kPadB;                     // [32][72] e dO, [feature][position]
    const int plain_r = (lane & 7) + 8 * ((lane >> 3) & 1), plain_c = 8 * (lane >> 4);
    const int flip_r = (lane & 7) + 8 * (lane >> 4), flip_c = 8 * ((lane >> 3) & 1);
    const int mt = warp & 3, nh = warp >> 2;
    const long long head_row = static_cast<long long>(head) * T;

    const uint32_t tile_bytes = kBwdSetBytes + kGateFloats * 4u;
    auto copy_tiles = [&](int chunk) {   // one thread
        if (tid != 0) return;
        unsigned char *set = tiles + (chunk & 1) * kBwdSetBytes;
        uint64_t *bar = &tile_full[chunk & 1];
        const int row = static_cast<int>(head_row) + chunk * kC;
        sm100::mbar_arrive_expect_tx(bar, tile_bytes);
        sm100::bulk_load(gate2 + (chunk & 1) * kGateFloats, gates_in + (static_cast<long long>(head) * chunks + chunk) * kGateFloats,
                         kGateFloats * 4, bar);
        sm100::tma_load_2d(set, &maps.k, bar, 0, row);
        sm100::tma_load_2d(set + kBoxBytes, &maps.k, bar, 64, row);
        sm100::tma_load_2d(set + 2 * kBoxBytes, &maps.q, bar, 0, row);
        sm100::tma_load_2d(set + 3 * kBoxBytes, &maps.q, bar, 64, row);
        sm100::tma_load_2d(set + 4 * kBoxBytes, &maps.p, bar, 0, row);
        sm100::tma_load_2d(set + 5 * kBoxBytes, &maps.minv, bar, 0, row);
        const int feature0 = head * kDV + blockIdx.y * kDVB;
        sm100::tma_load_2d(set + 6 * kBoxBytes, &maps.dout, bar, chunk * kC, feature0);
        sm100::tma_load_2d(set + 6 * kBoxBytes + kDVP * 128, &maps.dout, bar, chunk * kC, feature0 + kDVP);
    };
    bool gave_up = false;
    auto wait_tiles = [&](int chunk, uint32_t parity) {
        if (gave_up) return;
        uint64_t *bar = &tile_full[chunk & 1];
        if (sm100::mbar_wait(bar, parity, 4096)) return;
        unsigned long long t0, t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        while (!sm100::mbar_wait(bar, parity, 1024)) {
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > 2000000000ull) {
                gave_up = true;
                atomicCAS(&g_deltanet_error, 0, 2);
                return;
            }
        }
    };
    auto put_state = [&](__nv_bfloat16 *Sb, const float (&st)[4][4]) {
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            *reinterpret_cast<uint32_t *>(Sb + (16 * warp + g) * kPadB + 8 * nt + 2 * t4) = pack_bf16x2(st[nt][0], st[nt][1]);
            *reinterpret_cast<uint32_t *>(Sb + (16 * warp + g + 8) * kPadB + 8 * nt + 2 * t4) = pack_bf16x2(st[nt][2], st[nt][3]);
        }
    };

    float state[4][4] = {};
    put_state(Sb2, state);
    if (tid == 0) {
        sm100::mbar_init(&tile_full[0], 1);
        sm100::mbar_init(&tile_full[1], 1);
        sm100::fence_barrier_init();
    }
    __syncthreads();
    if (chunks > 0) copy_tiles(chunks - 1);
    int step = 0;   // chunks done so far: the copy buffers and barrier phases go by it
    for (int chunk = chunks - 1; chunk >= 0; chunk--, step++) {
        const long long row0 = head_row + static_cast<long long>(chunk) * kC;
        const long long cidx = static_cast<long long>(head) * chunks + chunk;
        const float *eca = gate2 + (chunk & 1) * kGateFloats, *ekd = eca + kC, *be = eca + 2 * kC;
        const unsigned char *Kt = tiles + (chunk & 1) * kBwdSetBytes, *Qt = Kt + 2 * kBoxBytes, *Pt = Kt + 4 * kBoxBytes,
                            *Mt = Kt + 5 * kBoxBytes, *Ot = Kt + 6 * kBoxBytes + group * (kDVP * 128);
        const __nv_bfloat16 *Sb = Sb2 + (step & 1) * kDK * kPadB;
        __syncthreads();   // the state copy is in place; everything of the chunk before (after, in time order) is done
        if (chunk > 0) copy_tiles(chunk - 1);
        // a buffer is used by every other chunk: chunks - 1, chunks - 3, ... share one, so its phase goes by step / 2
        wait_tiles(chunk, static_cast<uint32_t>((step >> 1) & 1));
        {   // the incoming state gradient, for the per-chunk kernel
            __nv_bfloat16 *dst = dsin_save + cidx * kDK * kDV + part * kDVP;
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                *reinterpret_cast<uint32_t *>(dst + (16 * warp + g) * kDV + 8 * nt + 2 * t4) = pack_bf16x2(state[nt][0], state[nt][1]);
                *reinterpret_cast<uint32_t *>(dst + (16 * warp + g + 8) * kDV + 8 * nt + 2 * t4) = pack_bf16x2(state[nt][2], state[nt][3]);
            }
        }
        {   // e dO beside dO: eight positions of one feature a thread
            const int f = gtid >> 3, t8 = (gtid & 7) * 8;
            const uint4 d8 = *reinterpret_cast<const uint4 *>(swz_row128(Ot, f, t8));
            const uint32_t w4[4] = {d8.x, d8.y, d8.z, d8.w};
            uint32_t o4[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float lo, hi;
                unpack_bf16x2(w4[e], lo, hi);
                o4[e] = pack_bf16x2(lo * eca[t8 + 2 * e], hi * eca[t8 + 2 * e + 1]);
            }
            *reinterpret_cast<uint4 *>(Oe + f * kPadP + t8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
        }

        // dU = ed (K dS') + P' dO : rows t = 16 mt + g (+8), columns 16 nh + 8 nt + 2 t4 (+1)
        {
            float acc[2][4] = {}, pd[2][4] = {};
#pragma unroll
            for (int k0 = 0; k0 < kDK; k0 += 16) {
                uint32_t af[4], bf[4];
                ldsm_x4(af, swz(Kt, 16 * mt + plain_r, k0 + plain_c));
                ldsm_x4_trans(bf, Sb + (k0 + plain_r) * kPadB + 16 * nh + plain_c);
                mma_bf16(acc[0], af, bf[0], bf[1]);
                mma_bf16(acc[1], af, bf[2], bf[3]);
                if ((k0 & 16) == 0) {   // P' dO between them: four steps over the chunk's positions
                    const int s0 = k0 >> 1;
                    uint32_t ap[4], bo[4];
                    ldsm_x4_trans(ap, swz_row128(Pt, s0 + flip_r, 16 * mt + flip_c));
                    ldsm_x4(bo, swz_row128(Ot, 16 * nh + flip_r, s0 + flip_c));
                    mma_bf16(pd[0], ap, bo[0], bo[1]);
                    mma_bf16(pd[1], ap, bo[2], bo[3]);
                }
            }
            const float e0 = ekd[16 * mt + g], e1 = ekd[16 * mt + g + 8];
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const int col = 16 * nh + 8 * nt + 2 * t4;
                *reinterpret_cast<uint32_t *>(Ub + (16 * mt + g) * kPadB + col) =
                    pack_bf16x2(fmaf(acc[nt][0], e0, pd[nt][0]), fmaf(acc[nt][1], e0, pd[nt][1]));
                *reinterpret_cast<uint32_t *>(Ub + (16 * mt + g + 8) * kPadB + col) =
                    pack_bf16x2(fmaf(acc[nt][2], e1, pd[nt][2]), fmaf(acc[nt][3], e1, pd[nt][3]));
            }
        }
        __syncthreads();

        // dZ = Minv' dU : A[t][s] = Minv[s][t]
        {
            float z[2][4] = {};
#pragma unroll
            for (int k0 = 0; k0 < kC; k0 += 16) {
                uint32_t af[4], bf[4];
                ldsm_x4_trans(af, swz_row128(Mt, k0 + flip_r, 16 * mt + flip_c));
                ldsm_x4_trans(bf, Ub + (k0 + plain_r) * kPadB + 16 * nh + plain_c);
                mma_bf16(z[0], af, bf[0], bf[1]);
                mma_bf16(z[1], af, bf[2], bf[3]);
            }
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int hr = 0; hr < 2; hr++) {
                    const int t = 16 * mt + g + 8 * hr, col = 16 * nh + 8 * nt + 2 * t4;
                    const float2 z2 = make_float2(z[nt][2 * hr], z[nt][2 * hr + 1]);
                    *reinterpret_cast<uint32_t *>(dz_save + (row0 + t) * kDV + part * kDVP + col) = pack_bf16x2(z2.x, z2.y);
                    const float b = be[t], eb = -eca[t] * b;
                    *reinterpret_cast<uint32_t *>(Zs + t * kPadB + col) = pack_bf16x2(eb * z2.x, eb * z2.y);
                    *reinterpret_cast<uint32_t *>(dv_out + (row0 + t) * kDV + part * kDVP + col) = pack_bf16x2(b * z2.x, b * z2.y);
                }
        }
        __syncthreads();

        // dS = g dS' + Q' (e dO) + K' (-e beta dZ) : warp -> state rows 16 warp + g (+8), all 32 features
        {
            const float gamma = eca[3 * kC];
#pragma unroll
            for (int nt = 0; nt < 4; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) state[nt][e] *= gamma;
#pragma unroll
            for (int k0 = 0; k0 < kC; k0 += 16) {
                uint32_t aq[4], ak[4], bo0[4], bo1[4], bz0[4], bz1[4];
                ldsm_x4_trans(aq, swz(Qt, k0 + flip_r, 16 * warp + flip_c));
                ldsm_x4(bo0, Oe + flip_r * kPadP + k0 + flip_c);
                ldsm_x4(bo1, Oe + (16 + flip_r) * kPadP + k0 + flip_c);
                mma_bf16(state[0], aq, bo0[0], bo0[1]);
                mma_bf16(state[1], aq, bo0[2], bo0[3]);
                mma_bf16(state[2], aq, bo1[0], bo1[1]);
                mma_bf16(state[3], aq, bo1[2], bo1[3]);
                ldsm_x4_trans(ak, swz(Kt, k0 + flip_r, 16 * warp + flip_c));
                ldsm_x4_trans(bz0, Zs + (k0 + plain_r) * kPadB + plain_c);
                ldsm_x4_trans(bz1, Zs + (k0 + plain_r) * kPadB + 16 + plain_c);
                mma_bf16(state[0], ak, bz0[0], bz0[1]);
                mma_bf16(state[1], ak, bz0[2], bz0[3]);
                mma_bf16(state[2], ak, bz1[0], bz1[1]);
                mma_bf16(state[3], ak, bz1[2], bz1[3]);
            }
            put_state(Sb2 + ((step + 1) & 1) * kDK * kPadB, state);
        }
    }
}

// X = tril(dO U') .* D and G = -stril(dZ U') .* D, one block per (head, chunk): two 64 x 64 x 128 products as
// BFloat16 MMAs (U and dZ arrive rounded from the scans; dO is read as it lies, [feature][position], as a transposed A
// operand).  Warp w takes rows 16 (w % 4) .. + 15 and columns 32 (w / 4) .. + 31; tiles wholly above the diagonal
// are skipped.
__global__ void __launch_bounds__(256) deltanet_bwd_xg_kernel(const float *a, const __nv_bfloat16 *dout,
                                                              const __nv_bfloat16 *u_save, const __nv_bfloat16 *dz_save,
                                                              __nv_bfloat16 *x_out, __nv_bfloat16 *g_out, int T) {
    extern __shared__ float sm[];
    float *ca = sm;                                                        // [64]
    __nv_bfloat16 *Ot = reinterpret_cast<__nv_bfloat16 *>(ca + kC);        // [128 features][72]
    __nv_bfloat16 *Uh = Ot + kDV * kPadP;                                  // [64][136]
    __nv_bfloat16 *Zh = Uh + kC * kPadH;                                   // [64][136]
    const int chunks = T / kC;
    const int head = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const long long row0 = static_cast<long long>(head) * T + static_cast<long long>(chunk) * kC;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int plain_r = (lane & 7) + 8 * ((lane >> 3) & 1), plain_c = 8 * (lane >> 4);
    const int flip_r = (lane & 7) + 8 * (lane >> 4), flip_c = 8 * ((lane >> 3) & 1);
    for (int i = tid; i < kDV * kC / 8; i += 256) {
        const int f = i >> 3, t8 = (i & 7) * 8;
        *reinterpret_cast<uint4 *>(Ot + f * kPadP + t8) = __ldg(reinterpret_cast<const uint4 *>(
            dout + (static_cast<long long>(head) * kDV + f) * T + static_cast<long long>(chunk) * kC + t8));
    }
    for (int i = tid; i < kC * kDV / 8; i += 256) {
        const int r = i / (kDV / 8), c = (i % (kDV / 8)) * 8;
        *reinterpret_cast<uint4 *>(Uh + r * kPadH + c) = __ldg(reinterpret_cast<const uint4 *>(u_save + (row0 + r) * kDV + c));
        *reinterpret_cast<uint4 *>(Zh + r * kPadH + c) = __ldg(reinterpret_cast<const uint4 *>(dz_save + (row0 + r) * kDV + c));
    }
    if (tid < 32) {
        float lo, hi;
        chunk_cumsum(a + row0, tid, lo, hi);
        ca[tid] = lo;
        ca[tid + 32] = hi;
    }
    __syncthreads();
    const int m0 = 16 * (warp & 3), n0 = 32 * (warp >> 2);
    float xo[4][4] = {}, zo[4][4] = {};
    const int live = n0 > m0 + 15 ? 0 : (m0 + 15 - n0) / 8 + 1;   // 8-column tiles that reach the diagonal
    if (live > 0) {
#pragma unroll 2
        for (int d = 0; d < kDV; d += 16) {
            uint32_t ao[4], az[4], b0[4], b1[4];
            ldsm_x4_trans(ao, Ot + (d + flip_r) * kPadP + m0 + flip_c);         // A[t][f] = dO stored [f][t]
            ldsm_x4(az, Zh + (m0 + plain_r) * kPadH + d + plain_c);
            ldsm_x4(b0, Uh + (n0 + flip_r) * kPadH + d + flip_c);               // B[f][s] = U stored [s][f]
            ldsm_x4(b1, Uh + (n0 + 16 + flip_r) * kPadH + d + flip_c);
            mma_bf16(xo[0], ao, b0[0], b0[1]); mma_bf16(zo[0], az, b0[0], b0[1]);
            if (live > 1) { mma_bf16(xo[1], ao, b0[2], b0[3]); mma_bf16(zo[1], az, b0[2], b0[3]); }
            if (live > 2) { mma_bf16(xo[2], ao, b1[0], b1[1]); mma_bf16(zo[2], az, b1[0], b1[1]); }
            if (live > 3) { mma_bf16(xo[3], ao, b1[2], b1[3]); mma_bf16(zo[3], az, b1[2], b1[3]); }
        }
    }
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
        for (int e = 0; e < 4; e += 2) {
            const int t = m0 + g + 8 * (e >> 1), s = n0 + 8 * j + 2 * t4;
            const float d0 = t >= s ? __expf(ca[t] - ca[s]) : 0.0f, d1 = t >= s + 1 ? __expf(ca[t] - ca[s + 1]) : 0.0f;
            *reinterpret_cast<uint32_t *>(x_out + (row0 + t) * kC + s) = pack_bf16x2(d0 * xo[j][e], d1 * xo[j][e + 1]);
            *reinterpret_cast<uint32_t *>(g_out + (row0 + t) * kC + s) =
                pack_bf16x2(t > s ? -d0 * zo[j][e] : 0.0f, t > s + 1 ? -d1 * zo[j][e + 1] : 0.0f);
        }
}

// sum over a row's columns held by the four lanes that share g
__device__ __forceinline__ float sum_quad(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}

// dQ, dK, da, dbeta of one chunk; one block per (head, chunk), two blocks per SM.  The eight products of the chunk
// are BFloat16 m16n8k16 MMAs whose fragments come through ldmatrix: what the scans and the X/G kernel left (the state,
// its gradient, U, dZ, X, G) was rounded to BFloat16 where it was written -- the rounding the reference gives the
// Float32 factor of a mixed product (ext/cuTileExt/emit.jl:914-921) -- and Q, K, dO are BFloat16 already.
// (As TF32 MMAs with one scalar load and one conversion per fragment element this kernel took half the pullback's
// time: the warp-level MMA issues once in about 16 cycles per SM quarter on this part, whatever its operand type,
// so halving the number of MMAs and dropping the conversions is what pays.)  Warp w takes positions
// 16 (w % 4) .. + 15 and features 64 (w / 4) .. + 63 of every (position, feature) result, i.e. eight 16 x 8
// accumulator tiles per product; a thread holds rows g, g + 8 and columns 2 t, 2 t + 1 of each tile.  Row sums of
// products of results with Q or K (the gate and beta gradients) are taken on the accumulators and meet through
// shared memory.  X, G and beta .* G take the state's place once the products with the state are done.
__global__ void __launch_bounds__(256, 2) deltanet_bwd_out_kernel(
    const __nv_bfloat16 *q, const __nv_bfloat16 *k, const __nv_bfloat16 *v, const float *a, const float *beta,
    const __nv_bfloat16 *dout, const __nv_bfloat16 *s_save, const __nv_bfloat16 *dsin_save, const __nv_bfloat16 *u_save,
    const __nv_bfloat16 *dz_save, const __nv_bfloat16 *x_in, const __nv_bfloat16 *g_in, __nv_bfloat16 *dq, __nv_bfloat16 *dk, float *da, float *dbeta, int T) {
    extern __shared__ float sm[];
    float *vec = sm;
    float *eca = vec, *ekd = vec + 64, *be = vec + 128;
    float *part = vec + 192;               // [7 sums][2 feature halves][64 rows]
    float *red = part + 7 * 128;           // [8]
    __nv_bfloat16 *Sh = reinterpret_cast<__nv_bfloat16 *>(red + 8);   // [128][136]: S, then dS'; then X, G, beta G [64][72] each
    __nv_bfloat16 *M0 = Sh + kDK * kPadH;   // [64][136]: dO, then U, then the dQ staging
    __nv_bfloat16 *M1 = M0 + kC * kPadH;    // [64][136]: dZ, then the dK staging
    __nv_bfloat16 *Qh = M1 + kC * kPadH;    // [64][136]
    __nv_bfloat16 *Kh = Qh + kC * kPadH;
    __nv_bfloat16 *Xh = Sh, *Gh = Xh + kC * kPadP, *Gb = Gh + kC * kPadP;
    __shared__ float gamma_sm;
    enum { DE = 0, DED, RQ, RK, CQ, CK, RDZ };

    const int chunks = T / kC;
    const int head = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const long long row0 = static_cast<long long>(head) * T + static_cast<long long>(chunk) * kC;
    const long long cidx = static_cast<long long>(head) * chunks + chunk;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int m0 = 16 * (warp & 3), nh = warp >> 2, n0 = 64 * nh;
    const int plain_r = (lane & 7) + 8 * ((lane >> 3) & 1), plain_c = 8 * (lane >> 4);
    const int flip_r = (lane & 7) + 8 * (lane >> 4), flip_c = 8 * ((lane >> 3) & 1);

    auto piece = [](const __nv_bfloat16 *src) { return __ldg(reinterpret_cast<const uint4 *>(src)); };   // eight values
    for (int i = tid; i < kDK * kDV / 8; i += 256) {
        const int r = i / (kDV / 8), c = (i % (kDV / 8)) * 8;
        *reinterpret_cast<uint4 *>(Sh + r * kPadH + c) = piece(s_save + cidx * kDK * kDV + r * kDV + c);
    }
    for (int i = tid; i < kDV * kC / 8; i += 256) {   // dO arrives [feature][position]: turned as it is staged
        const int f = i >> 3, t8 = (i & 7) * 8;
        const uint4 d8 = __ldg(reinterpret_cast<const uint4 *>(dout + (static_cast<long long>(head) * kDV + f) * T +
                                                               static_cast<long long>(chunk) * kC + t8));
        const uint32_t w4[4] = {d8.x, d8.y, d8.z, d8.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            reinterpret_cast<unsigned short *>(M0)[(t8 + 2 * e) * kPadH + f] = static_cast<unsigned short>(w4[e] & 0xffffu);
            reinterpret_cast<unsigned short *>(M0)[(t8 + 2 * e + 1) * kPadH + f] = static_cast<unsigned short>(w4[e] >> 16);
        }
    }
    for (int i = tid; i < kC * kDV / 8; i += 256) {
        const int r = i / (kDV / 8), c = (i % (kDV / 8)) * 8;
        *reinterpret_cast<uint4 *>(M1 + r * kPadH + c) = piece(dz_save + (row0 + r) * kDV + c);
    }
    for (int i = tid; i < kC * kDK / 8; i += 256) {
        const int r = i / (kDK / 8), c = (i % (kDK / 8)) * 8;
        *reinterpret_cast<uint4 *>(Qh + r * kPadH + c) = __ldg(reinterpret_cast<const uint4 *>(q + (row0 + r) * kDK + c));
        *reinterpret_cast<uint4 *>(Kh + r * kPadH + c) = __ldg(reinterpret_cast<const uint4 *>(k + (row0 + r) * kDK + c));
    }
    if (tid < kC) be[tid] = beta[row0 + tid];
    if (tid < 32) {
        float lo, hi;
        chunk_cumsum(a + row0, tid, lo, hi);
        const float last = __shfl_sync(0xffffffffu, hi, 31);
        eca[tid] = __expf(lo); eca[tid + 32] = __expf(hi);
        ekd[tid] = __expf(last - lo); ekd[tid + 32] = __expf(last - hi);
        if (tid == 0) gamma_sm = __expf(last);
    }
    __syncthreads();

    const int t0 = m0 + g, t1 = t0 + 8;   // this thread's two positions
    // Q or K at the accumulator's positions: columns n0 + 8 nt + 2 t4 (+1) of rows t0, t1
    auto pair_at = [&](const __nv_bfloat16 *tile, int row, int nt, float &x0, float &x1) {
        unpack_bf16x2(*reinterpret_cast<const uint32_t *>(tile + row * kPadH + n0 + 8 * nt + 2 * t4), x0, x1);
    };
    // sum_i tile[row][i] * acc[.][row half] over this thread's columns
    auto dot_rows = [&](const __nv_bfloat16 *tile, const float (&acc)[8][4], float &r0, float &r1) {
        r0 = r1 = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            float a0, a1, b0, b1;
            pair_at(tile, t0, nt, a0, a1);
            pair_at(tile, t1, nt, b0, b1);
            r0 += a0 * acc[nt][0] + a1 * acc[nt][1];
            r1 += b0 * acc[nt][2] + b1 * acc[nt][3];
        }
    };
    auto put_rows = [&](int which, float r0, float r1) {   // this warp's share of a row sum
        r0 = sum_quad(r0);
        r1 = sum_quad(r1);
        if (t4 == 0) { part[(which * 2 + nh) * 64 + t0] = r0; part[(which * 2 + nh) * 64 + t1] = r1; }
    };
    // acc += A B over k0 .. k0 + 15 for this warp's eight feature tiles.  B stored [n][k] (rows of features, the summed
    // axis contiguous) is read as it lies; B stored [k][n] is read transposed.
    auto step_nk = [&](float (&acc)[8][4], const uint32_t (&af)[4], const __nv_bfloat16 *tile, int pitch, int k0) {
#pragma unroll
        for (int np = 0; np < 4; np++) {
            uint32_t bf[4];
            ldsm_x4(bf, tile + (n0 + 16 * np + flip_r) * pitch + k0 + flip_c);
            mma_bf16(acc[2 * np], af, bf[0], bf[1]);
            mma_bf16(acc[2 * np + 1], af, bf[2], bf[3]);
        }
    };
    auto step2_nk = [&](float (&acc0)[8][4], float (&acc1)[8][4], const uint32_t (&a0)[4], const uint32_t (&a1)[4],
                        const __nv_bfloat16 *tile, int pitch, int k0) {
#pragma unroll
        for (int np = 0; np < 4; np++) {
            uint32_t bf[4];
            ldsm_x4(bf, tile + (n0 + 16 * np + flip_r) * pitch + k0 + flip_c);
            mma_bf16(acc0[2 * np], a0, bf[0], bf[1]);
            mma_bf16(acc0[2 * np + 1], a0, bf[2], bf[3]);
            mma_bf16(acc1[2 * np], a1, bf[0], bf[1]);
            mma_bf16(acc1[2 * np + 1], a1, bf[2], bf[3]);
        }
    };
    auto step_kn = [&](float (&acc)[8][4], const uint32_t (&af)[4], const __nv_bfloat16 *tile, int pitch, int k0) {
#pragma unroll
        for (int np = 0; np < 4; np++) {
            uint32_t bf[4];
            ldsm_x4_trans(bf, tile + (k0 + plain_r) * pitch + n0 + 16 * np + plain_c);
            mma_bf16(acc[2 * np], af, bf[0], bf[1]);
            mma_bf16(acc[2 * np + 1], af, bf[2], bf[3]);
        }
    };

    float dqa[8][4], dka[8][4];
    // phase 1: T1 = dO S', T2 = dZ S' (one sweep over the state's rows for both)
    {
        float t1a[8][4] = {}, t2a[8][4] = {};
#pragma unroll 2
        for (int k0 = 0; k0 < kDV; k0 += 16) {
            uint32_t a0[4], a1[4];
            ldsm_x4(a0, M0 + (m0 + plain_r) * kPadH + k0 + plain_c);
            ldsm_x4(a1, M1 + (m0 + plain_r) * kPadH + k0 + plain_c);
            step2_nk(t1a, t2a, a0, a1, Sh, kPadH, k0);
        }
        float q0, q1, k0s, k1s;
        dot_rows(Qh, t1a, q0, q1);
        dot_rows(Kh, t2a, k0s, k1s);
        put_rows(DE, q0 - be[t0] * k0s, q1 - be[t1] * k1s);
        const float e0 = eca[t0], e1 = eca[t1], b0 = -e0 * be[t0], b1 = -e1 * be[t1];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            dqa[nt][0] = e0 * t1a[nt][0]; dqa[nt][1] = e0 * t1a[nt][1]; dqa[nt][2] = e1 * t1a[nt][2]; dqa[nt][3] = e1 * t1a[nt][3];
            dka[nt][0] = b0 * t2a[nt][0]; dka[nt][1] = b0 * t2a[nt][1]; dka[nt][2] = b1 * t2a[nt][2]; dka[nt][3] = b1 * t2a[nt][3];
        }
    }
    // K S at (position, value feature), then rowsum(dZ .* (V - e K S)) for dbeta
    {
        float ks[8][4] = {};
#pragma unroll 2
        for (int k0 = 0; k0 < kDK; k0 += 16) {
            uint32_t af[4];
            ldsm_x4(af, Kh + (m0 + plain_r) * kPadH + k0 + plain_c);
            step_kn(ks, af, Sh, kPadH, k0);
        }
        const float e0 = eca[t0], e1 = eca[t1];
        float r0 = 0.0f, r1 = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            const int col = n0 + 8 * nt + 2 * t4;
            float v00, v01, v10, v11, z00, z01, z10, z11;
            unpack_bf16x2(__ldg(reinterpret_cast<const uint32_t *>(v + (row0 + t0) * kDV + col)), v00, v01);
            unpack_bf16x2(__ldg(reinterpret_cast<const uint32_t *>(v + (row0 + t1) * kDV + col)), v10, v11);
            unpack_bf16x2(*reinterpret_cast<const uint32_t *>(M1 + t0 * kPadH + col), z00, z01);
            unpack_bf16x2(*reinterpret_cast<const uint32_t *>(M1 + t1 * kPadH + col), z10, z11);
            r0 += z00 * (v00 - e0 * ks[nt][0]) + z01 * (v01 - e0 * ks[nt][1]);
            r1 += z10 * (v10 - e1 * ks[nt][2]) + z11 * (v11 - e1 * ks[nt][3]);
        }
        put_rows(RDZ, r0, r1);
    }
    __syncthreads();

    // phase 2: dS' replaces S (their inner product is the gradient of g), U replaces dO; T3 = U dS''
    {
        float dgp = 0.0f;
        for (int i = tid; i < kDK * kDV / 8; i += 256) {
            const int r = i / (kDV / 8), c = (i % (kDV / 8)) * 8;
            const uint4 nw = piece(dsin_save + cidx * kDK * kDV + r * kDV + c);
            uint4 *slot = reinterpret_cast<uint4 *>(Sh + r * kPadH + c);
            const uint4 old = *slot;
            float o8[8], n8[8];
            unpack_bf16x2(old.x, o8[0], o8[1]); unpack_bf16x2(old.y, o8[2], o8[3]);
            unpack_bf16x2(old.z, o8[4], o8[5]); unpack_bf16x2(old.w, o8[6], o8[7]);
            unpack_bf16x2(nw.x, n8[0], n8[1]); unpack_bf16x2(nw.y, n8[2], n8[3]);
            unpack_bf16x2(nw.z, n8[4], n8[5]); unpack_bf16x2(nw.w, n8[6], n8[7]);
#pragma unroll
            for (int e = 0; e < 8; e++) dgp = fmaf(o8[e], n8[e], dgp);
            *slot = nw;
        }
        for (int i = tid; i < kC * kDV / 8; i += 256) {
            const int r = i / (kDV / 8), c = (i % (kDV / 8)) * 8;
            *reinterpret_cast<uint4 *>(M0 + r * kPadH + c) = piece(u_save + (row0 + r) * kDV + c);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dgp += __shfl_xor_sync(0xffffffffu, dgp, o);
        if (lane == 0) red[warp] = dgp;
    }
    __syncthreads();
    {
        float t3[8][4] = {};
#pragma unroll 2
        for (int k0 = 0; k0 < kDV; k0 += 16) {
            uint32_t af[4];
            ldsm_x4(af, M0 + (m0 + plain_r) * kPadH + k0 + plain_c);
            step_nk(t3, af, Sh, kPadH, k0);
        }
        float r0, r1;
        dot_rows(Kh, t3, r0, r1);
        put_rows(DED, r0, r1);
        const float e0 = ekd[t0], e1 = ekd[t1];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            dka[nt][0] = fmaf(e0, t3[nt][0], dka[nt][0]); dka[nt][1] = fmaf(e0, t3[nt][1], dka[nt][1]);
            dka[nt][2] = fmaf(e1, t3[nt][2], dka[nt][2]); dka[nt][3] = fmaf(e1, t3[nt][3], dka[nt][3]);
        }
    }
    __syncthreads();   // the state's place is free: X, G and beta .* G move in
    for (int i = tid; i < kC * kC / 8; i += 256) {
        const int r = i / (kC / 8), c = (i % (kC / 8)) * 8;
        *reinterpret_cast<uint4 *>(Xh + r * kPadP + c) = piece(x_in + row0 * kC + r * kC + c);
        const uint4 g8 = piece(g_in + row0 * kC + r * kC + c);
        *reinterpret_cast<uint4 *>(Gh + r * kPadP + c) = g8;
        const float b = be[r];
        const uint32_t w4[4] = {g8.x, g8.y, g8.z, g8.w};
        uint32_t s4[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            float lo, hi;
            unpack_bf16x2(w4[e], lo, hi);
            s4[e] = pack_bf16x2(b * lo, b * hi);
        }
        *reinterpret_cast<uint4 *>(Gb + r * kPadP + c) = make_uint4(s4[0], s4[1], s4[2], s4[3]);
    }
    __syncthreads();

    // phase 3: the four products over the chunk's own positions (B[k][n] = K[s][i] or Q[s][i])
    {   // X K -> dQ and its row sum with Q
        float xk[8][4] = {};
#pragma unroll
        for (int k0 = 0; k0 < kC; k0 += 16) {
            uint32_t af[4];
            ldsm_x4(af, Xh + (m0 + plain_r) * kPadP + k0 + plain_c);
            step_kn(xk, af, Kh, kPadH, k0);
        }
        float r0, r1;
        dot_rows(Qh, xk, r0, r1);
        put_rows(RQ, r0, r1);
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) dqa[nt][e] += xk[nt][e];
    }
    {   // X' Q -> dK and its row sum with K
        float xq[8][4] = {};
#pragma unroll
        for (int k0 = 0; k0 < kC; k0 += 16) {
            uint32_t af[4];
            ldsm_x4_trans(af, Xh + (k0 + flip_r) * kPadP + m0 + flip_c);
            step_kn(xq, af, Qh, kPadH, k0);
        }
        float r0, r1;
        dot_rows(Kh, xq, r0, r1);
        put_rows(CQ, r0, r1);
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) dka[nt][e] += xq[nt][e];
    }
    {   // G K -> beta-scaled into dK, its row sum with K feeds dbeta and the gate gradient
        float gk[8][4] = {};
#pragma unroll
        for (int k0 = 0; k0 < kC; k0 += 16) {
            uint32_t af[4];
            ldsm_x4(af, Gh + (m0 + plain_r) * kPadP + k0 + plain_c);
            step_kn(gk, af, Kh, kPadH, k0);
        }
        float r0, r1;
        dot_rows(Kh, gk, r0, r1);
        put_rows(RK, r0, r1);
        const float b0 = be[t0], b1 = be[t1];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            dka[nt][0] = fmaf(b0, gk[nt][0], dka[nt][0]); dka[nt][1] = fmaf(b0, gk[nt][1], dka[nt][1]);
            dka[nt][2] = fmaf(b1, gk[nt][2], dka[nt][2]); dka[nt][3] = fmaf(b1, gk[nt][3], dka[nt][3]);
        }
    }
    {   // G' (beta K) = (beta .* G)' K
        float gb[8][4] = {};
#pragma unroll
        for (int k0 = 0; k0 < kC; k0 += 16) {
            uint32_t af[4];
            ldsm_x4_trans(af, Gb + (k0 + flip_r) * kPadP + m0 + flip_c);
            step_kn(gb, af, Kh, kPadH, k0);
        }
        float r0, r1;
        dot_rows(Kh, gb, r0, r1);
        put_rows(CK, r0, r1);
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) dka[nt][e] += gb[nt][e];
    }
    __syncthreads();   // every reader of U (M0) and dZ (M1) is done; the row sums are visible

#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
        const int col = n0 + 8 * nt + 2 * t4;
        *reinterpret_cast<uint32_t *>(M0 + t0 * kPadH + col) = pack_bf16x2(dqa[nt][0], dqa[nt][1]);
        *reinterpret_cast<uint32_t *>(M0 + t1 * kPadH + col) = pack_bf16x2(dqa[nt][2], dqa[nt][3]);
        *reinterpret_cast<uint32_t *>(M1 + t0 * kPadH + col) = pack_bf16x2(dka[nt][0], dka[nt][1]);
        *reinterpret_cast<uint32_t *>(M1 + t1 * kPadH + col) = pack_bf16x2(dka[nt][2], dka[nt][3]);
    }
    auto row_sum = [&](int which, int t) { return part[(which * 2) * 64 + t] + part[(which * 2 + 1) * 64 + t]; };
    if (tid == 0) {
        // the gradient of ca, then da = its reverse cumulative sum inside the chunk
        float dg = 0.0f;
        for (int w = 0; w < 8; w++) dg += red[w];
        float tail = dg * gamma_sm;
        for (int t = 0; t < kC; t++) tail += row_sum(DED, t) * ekd[t];
        float run = 0.0f;
        for (int t = kC - 1; t >= 0; t--) {
            float dca = row_sum(RQ, t) + be[t] * row_sum(RK, t) - row_sum(CQ, t) - row_sum(CK, t) + row_sum(DE, t) * eca[t] -
                        row_sum(DED, t) * ekd[t];
            if (t == kC - 1) dca += tail;
            run += dca;
            da[row0 + t] = run;
        }
    }
    if (tid >= 32 && tid < 32 + kC) {
        const int t = tid - 32;
        dbeta[row0 + t] = row_sum(RDZ, t) + row_sum(RK, t);
    }
    __syncthreads();
    for (int i = tid; i < kC * kDK / 8; i += 256) {
        const int r = i / (kDK / 8), c = (i % (kDK / 8)) * 8;
        *reinterpret_cast<uint4 *>(dq + (row0 + r) * kDK + c) = *reinterpret_cast<const uint4 *>(M0 + r * kPadH + c);
        *reinterpret_cast<uint4 *>(dk + (row0 + r) * kDK + c) = *reinterpret_cast<const uint4 *>(M1 + r * kPadH + c);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A [rows][cols] BFloat16 array as a tensor map of boxes of 64 columns x box_rows rows, 128-byte swizzle.
int scan_tmap(CUtensorMap *map, const void *base, long long rows, long long cols, int box_rows = kC) {
    static std::mutex lock;
    static EncodeTiledFn fn = nullptr;
    {
        std::lock_guard<std::mutex> hold(lock);
        if (!fn) {
            void *sym = nullptr;
            cudaDriverEntryPointQueryResult qres;
            TB200_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres));
            if (!sym || qres != cudaDriverEntryPointSuccess) return TB200_ERR_UNSUPPORTED;
            fn = reinterpret_cast<EncodeTiledFn>(sym);
        }
    }
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
    cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TB200_OK : TB200_ERR_UNSUPPORTED;
}

// The forward scan's launch: tensor maps over W (scratch), Q, K and P (scratch), one block per (head, 64 features).
int launch_scan(const tb200_deltanet_desc *d, const void *q, const void *k, const float *gates, const __nv_bfloat16 *w,
                const __nv_bfloat16 *u, const __nv_bfloat16 *pw, __nv_bfloat16 *o, __nv_bfloat16 *s_save,
                __nv_bfloat16 *u_save, cudaStream_t stream);

constexpr size_t kChunkSmem = (2 * kC * kPadA + 3 * kC) * sizeof(float) + 2 * kC * kPadH * sizeof(__nv_bfloat16);
constexpr size_t kScanSmem = 1024 + 2 * kTileSetBytes + 2 * kGateFloats * sizeof(float) +
                             (kDVB / kDVP) * (2 * kDK * kPadB + 2 * kC * kPadB + kDVP * kPadP) * sizeof(__nv_bfloat16);
constexpr size_t kBwdScanSmem = 1024 + 2 * kBwdSetBytes + 2 * kGateFloats * sizeof(float) +
                                (kDVB / kDVP) * (2 * kDK * kPadB + 2 * kC * kPadB + kDVP * kPadP) * sizeof(__nv_bfloat16);
constexpr size_t kBwdXgSmem = kC * sizeof(float) + (kDV * kPadP + 2 * kC * kPadH) * sizeof(__nv_bfloat16);
constexpr size_t kBwdOutSmem = (3 * kC + 7 * 2 * kC + 8) * sizeof(float) + (kDK * kPadH + 4 * kC * kPadH) * sizeof(__nv_bfloat16);

}  // namespace
}  // namespace tb200

using namespace tb200;

namespace {
int check_deltanet(const tb200_deltanet_desc *d) {
    if (!d) return TB200_ERR_NULL;
    if (d->heads < 0 || d->positions < 0) return TB200_ERR_SHAPE;
    if (d->dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (d->dk != kDK || d->dv != kDV || d->chunk != kC || d->positions % kC != 0) return TB200_ERR_UNSUPPORTED;
    // the scans address rows of [heads * positions] arrays (and heads * 128 feature rows) by 32-bit tile coordinates,
    // and the chunk kernels take one block per chunk
    if (static_cast<long long>(d->heads) * d->positions >= (1ll << 31) || static_cast<long long>(d->heads) * kDV >= (1ll << 31))
        return TB200_ERR_SHAPE;
    return TB200_OK;
}

int configure_deltanet(int device) {
    static std::mutex lock;
    static bool configured[64] = {};
    std::lock_guard<std::mutex> hold(lock);
    if (configured[device]) return TB200_OK;
    TB200_CUDA(cudaFuncSetAttribute(deltanet_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kChunkSmem)));
    TB200_CUDA(cudaFuncSetAttribute(deltanet_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kScanSmem)));
    TB200_CUDA(cudaFuncSetAttribute(deltanet_bwd_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kBwdScanSmem)));
    TB200_CUDA(cudaFuncSetAttribute(deltanet_bwd_xg_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kBwdXgSmem)));
    TB200_CUDA(cudaFuncSetAttribute(deltanet_bwd_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kBwdOutSmem)));
    configured[device] = true;
    return TB200_OK;
}

// bytes per position of the backward's workspace, after the forward's part
constexpr size_t kBwdRowBytes = (kC /*Minv*/ + kDK * kDV / kC /*S*/ + kDV /*U*/ + kDK * kDV / kC /*dS'*/ + kDV /*dZ*/ +
                                 2 * kC /*X, G*/) * sizeof(__nv_bfloat16);
}  // namespace

extern "C" size_t tb200_deltanet_workspace_bytes(const tb200_deltanet_desc *d) {
    if (check_deltanet(d) != TB200_OK) return 0;
    const size_t rows = static_cast<size_t>(d->heads) * d->positions;
    return rows * (kDK + kDV + kC) * sizeof(__nv_bfloat16) + rows / kC * kGateFloats * sizeof(float);
}

namespace tb200 {
namespace {
int launch_scan(const tb200_deltanet_desc *d, const void *q, const void *k, const float *gates, const __nv_bfloat16 *w,
                const __nv_bfloat16 *u, const __nv_bfloat16 *pw, __nv_bfloat16 *o, __nv_bfloat16 *s_save,
                __nv_bfloat16 *u_save, cudaStream_t stream) {
    const long long rows = static_cast<long long>(d->heads) * d->positions;
    ScanMaps maps;
    int st = scan_tmap(&maps.w, w, rows, kDK);
    if (!st) st = scan_tmap(&maps.q, q, rows, kDK);
    if (!st) st = scan_tmap(&maps.k, k, rows, kDK);
    if (!st) st = scan_tmap(&maps.p, pw, rows, kC);
    if (st) return st;
    dim3 grid(static_cast<unsigned>(d->heads), kDV / kDVB);
    deltanet_scan_kernel<<<grid, kScanThreads, kScanSmem, stream>>>(maps, gates, u, o, s_save, u_save, d->positions);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}
}  // namespace
}  // namespace tb200

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
    if ((st = configure_deltanet(dev.device))) return st;
    const size_t rows = static_cast<size_t>(d->heads) * d->positions;
    __nv_bfloat16 *w = static_cast<__nv_bfloat16 *>(workspace);
    __nv_bfloat16 *u = w + rows * kDK;
    __nv_bfloat16 *pw = u + rows * kDV;
    float *gates = reinterpret_cast<float *>(pw + rows * kC);
    const int T = d->positions;
    const unsigned chunks = static_cast<unsigned>(d->heads) * (T / kC);
    deltanet_chunk_kernel<<<chunks, 256, kChunkSmem, stream>>>(
        static_cast<const __nv_bfloat16 *>(q), static_cast<const __nv_bfloat16 *>(k),
        static_cast<const __nv_bfloat16 *>(v), a, beta, w, u, pw, nullptr, gates, T);
    TB200_CUDA(cudaGetLastError());
    return launch_scan(d, q, k, gates, w, u, pw, static_cast<__nv_bfloat16 *>(o), nullptr, nullptr, stream);
}

extern "C" size_t tb200_deltanet_bwd_workspace_bytes(const tb200_deltanet_desc *d) {
    if (check_deltanet(d) != TB200_OK) return 0;
    const size_t rows = static_cast<size_t>(d->heads) * d->positions;
    return tb200_deltanet_workspace_bytes(d) + rows * kBwdRowBytes;
}

extern "C" int tb200_deltanet_bwd(const tb200_deltanet_desc *d, const void *q, const void *k, const void *v,
                                  const float *a, const float *beta, const void *dout, void *dq, void *dk, void *dv,
                                  float *da, float *dbeta, void *workspace, size_t workspace_bytes, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int st = check_deltanet(d);
    if (st) return st;
    if (d->heads == 0 || d->positions == 0) return TB200_OK;
    if (!q || !k || !v || !a || !beta || !dout || !dq || !dk || !dv || !da || !dbeta) return TB200_ERR_NULL;
    const void *wide[] = {q, k, v, dout, dq, dk, dv};
    for (const void *p : wide)
        if (!aligned_to(p, 16)) return TB200_ERR_ALIGN;
    if (!aligned_to(a, 4) || !aligned_to(beta, 4) || !aligned_to(da, 4) || !aligned_to(dbeta, 4)) return TB200_ERR_ALIGN;
    const size_t need = tb200_deltanet_bwd_workspace_bytes(d);
    if (!workspace || workspace_bytes < need || !aligned_to(workspace, 16)) return TB200_ERR_WORKSPACE;
    DeviceInfo dev;
    if ((st = current_device(&dev))) return st;
    if ((st = configure_deltanet(dev.device))) return st;

    const size_t rows = static_cast<size_t>(d->heads) * d->positions;
    __nv_bfloat16 *w = static_cast<__nv_bfloat16 *>(workspace);
    __nv_bfloat16 *u = w + rows * kDK;
    __nv_bfloat16 *pw = u + rows * kDV;
    float *gates = reinterpret_cast<float *>(pw + rows * kC);
    // what the pullback keeps between its launches, all BFloat16 (every consumer takes it as an MMA operand)
    __nv_bfloat16 *minv = reinterpret_cast<__nv_bfloat16 *>(gates + rows / kC * kGateFloats);   // (I + A)^-1
    __nv_bfloat16 *s_save = minv + rows * kC;                       // the state at every chunk start
    __nv_bfloat16 *u_save = s_save + rows * (kDK * kDV / kC);
    __nv_bfloat16 *dsin = u_save + rows * kDV;                      // the state gradient arriving at every chunk
    __nv_bfloat16 *dz = dsin + rows * (kDK * kDV / kC);
    __nv_bfloat16 *xw = dz + rows * kDV;
    __nv_bfloat16 *gw = xw + rows * kC;
    const int T = d->positions;
    const unsigned chunks = static_cast<unsigned>(d->heads) * (T / kC);
    const __nv_bfloat16 *qb = static_cast<const __nv_bfloat16 *>(q), *kb = static_cast<const __nv_bfloat16 *>(k),
                        *vb = static_cast<const __nv_bfloat16 *>(v), *dob = static_cast<const __nv_bfloat16 *>(dout);
    dim3 grid(static_cast<unsigned>(d->heads), kDV / kDVP);

    // the forward again, keeping what the pullback needs: (I + A)^-1, the state at every chunk start, U
    deltanet_chunk_kernel<<<chunks, 256, kChunkSmem, stream>>>(qb, kb, vb, a, beta, w, u, pw, minv, gates, T);
    TB200_CUDA(cudaGetLastError());
    // no result pointer: the scan only carries the state
    if ((st = launch_scan(d, q, k, gates, w, u, pw, nullptr, s_save, u_save, stream))) return st;
    {
        BwdScanMaps maps;
        if ((st = scan_tmap(&maps.k, k, static_cast<long long>(rows), kDK))) return st;
        if ((st = scan_tmap(&maps.q, q, static_cast<long long>(rows), kDK))) return st;
        if ((st = scan_tmap(&maps.p, pw, static_cast<long long>(rows), kC))) return st;
        if ((st = scan_tmap(&maps.minv, minv, static_cast<long long>(rows), kC))) return st;
        if ((st = scan_tmap(&maps.dout, dout, static_cast<long long>(d->heads) * kDV, T, kDVP))) return st;
        deltanet_bwd_scan_kernel<<<dim3(static_cast<unsigned>(d->heads), kDV / kDVB), kScanThreads, kBwdScanSmem, stream>>>(
            maps, gates, dsin, dz, static_cast<__nv_bfloat16 *>(dv), T);
        TB200_CUDA(cudaGetLastError());
    }
    deltanet_bwd_xg_kernel<<<chunks, 256, kBwdXgSmem, stream>>>(a, dob, u_save, dz, xw, gw, T);
    TB200_CUDA(cudaGetLastError());
    deltanet_bwd_out_kernel<<<chunks, 256, kBwdOutSmem, stream>>>(qb, kb, vb, a, beta, dob, s_save, dsin, u_save, dz, xw,
                                                                 gw, static_cast<__nv_bfloat16 *>(dq),
                                                                 static_cast<__nv_bfloat16 *>(dk), da, dbeta, T);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

// As tb200_device_error, for the DeltaNet scans (their tiles arrive by bulk copies on an mbarrier): 0, or 1 when a
// wait gave up.
extern "C" int tb200_deltanet_device_error(void) {
    int code = 0, zero = 0;
    TB200_CUDA(cudaDeviceSynchronize());
    TB200_CUDA(cudaMemcpyFromSymbol(&code, tb200::g_deltanet_error, sizeof(int)));
    if (code) TB200_CUDA(cudaMemcpyToSymbol(tb200::g_deltanet_error, &zero, sizeof(int)));
    return code;
}
