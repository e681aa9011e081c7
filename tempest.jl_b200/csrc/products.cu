// Products alike by arrays of their operands' addresses: one launch for `count` products of the same shape,
// layouts and element types whose matrices lie anywhere in device memory.  The reference's `Products`
// (ext/cuBLASExt.jl:273-306, cublasGemmBatchedEx on device arrays of pointers) is what it runs for the many small
// alike products of a recurrence's chunks (DeltaNet's 64 x 64 x 128 blocks); a strided batch (tb200_gemm with
// `batch`) covers only operands that lie at equal distances.
//
// Half-precision operands (BFloat16 or Float16): one block of four warps per (member, 64 x 64 tile of the result).
// The operands' tiles are staged in shared memory as they lie -- K-major ([m][k], [n][k]) or MN-major ([k][m],
// [k][n]) -- and read through ldmatrix, transposed where the m16n8k16 fragment wants the other axis contiguous, so all
// four of cuBLAS's transposes are one kernel; Float32 accumulation, one rounding at the store.  Edges (extents that
// are not multiples of 64, leading dimensions or addresses that rule out 16-byte loads) are staged element by
// element with zeros outside.  Float32 operands take a plain tiled kernel on the CUDA cores (exact Float32).
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kPT = 64;        // tile of the result and step along k
constexpr int kPPad = 72;      // row pitch of a staged tile, elements: ldmatrix rows hit 32 banks

struct PointerArgs {
    const void *const *a, *const *b;
    void *const *c;
    long long count;
    int m, n, k;
    long long lda, ldb, ldc;
    int a_mn, b_mn;
    int in_dtype, out_dtype;
    float alpha;
};

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void *row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(row))));
}
__device__ __forceinline__ void ldsm4_trans(uint32_t (&r)[4], const void *row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(row))));
}
template <bool F16>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (F16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A 64 x 64 tile of a half-precision operand into shared memory as it lies: `rows` x `cols` of it exist from
// (r0, c0) on, the rest is zero.  `cols` runs along the operand's contiguous axis.
__device__ __forceinline__ void stage_tile(unsigned short *dst, const unsigned short *src, long long ld, int r0, int c0, int rows,
                                           int cols, bool wide) {
    const int tid = threadIdx.x;
    if (wide && rows >= kPT && cols >= kPT) {
        for (int i = tid; i < kPT * kPT / 8; i += 128) {
            const int r = i >> 3, c = (i & 7) * 8;
            *reinterpret_cast<uint4 *>(dst + r * kPPad + c) =
                __ldg(reinterpret_cast<const uint4 *>(src + (r0 + r) * ld + c0 + c));
        }
    } else {
        for (int i = tid; i < kPT * kPT; i += 128) {
            const int r = i >> 6, c = i & 63;
            dst[r * kPPad + c] = (r < rows && c < cols) ? __ldg(src + (r0 + r) * ld + c0 + c) : static_cast<unsigned short>(0);
        }
    }
}

template <bool F16>
__global__ void __launch_bounds__(128) products_mma_kernel(const PointerArgs p) {
    __shared__ __align__(16) unsigned short As[kPT * kPPad];
    __shared__ __align__(16) unsigned short Bs[kPT * kPPad];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int plain_r = (lane & 7) + 8 * ((lane >> 3) & 1), plain_c = 8 * (lane >> 4);
    const int flip_r = (lane & 7) + 8 * (lane >> 4), flip_c = 8 * ((lane >> 3) & 1);
    const int m0 = blockIdx.y * kPT, n0 = blockIdx.x * kPT;
    for (long long member = blockIdx.z; member < p.count; member += gridDim.z) {
        const unsigned short *a = static_cast<const unsigned short *>(p.a[member]);
        const unsigned short *b = static_cast<const unsigned short *>(p.b[member]);
        const bool wide_a = (reinterpret_cast<uintptr_t>(a) & 15) == 0 && p.lda % 8 == 0;
        const bool wide_b = (reinterpret_cast<uintptr_t>(b) & 15) == 0 && p.ldb % 8 == 0;
        float acc[8][4] = {};
        for (int k0 = 0; k0 < p.k; k0 += kPT) {
            // staged as they lie: K-major operands [m or n][k], MN-major operands [k][m or n]
            if (p.a_mn) stage_tile(As, a, p.lda, k0, m0, p.k - k0, p.m - m0, wide_a);
            else stage_tile(As, a, p.lda, m0, k0, p.m - m0, p.k - k0, wide_a);
            if (p.b_mn) stage_tile(Bs, b, p.ldb, k0, n0, p.k - k0, p.n - n0, wide_b);
            else stage_tile(Bs, b, p.ldb, n0, k0, p.n - n0, p.k - k0, wide_b);
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < kPT; kk += 16) {
                uint32_t af[4];
                if (p.a_mn) ldsm4_trans(af, As + (kk + flip_r) * kPPad + 16 * warp + flip_c);
                else ldsm4(af, As + (16 * warp + plain_r) * kPPad + kk + plain_c);
#pragma unroll
                for (int np = 0; np < 4; np++) {
                    uint32_t bf[4];
                    if (p.b_mn) ldsm4_trans(bf, Bs + (kk + plain_r) * kPPad + 16 * np + plain_c);
                    else ldsm4(bf, Bs + (16 * np + flip_r) * kPPad + kk + flip_c);
                    mma16816<F16>(acc[2 * np], af, bf[0], bf[1]);
                    mma16816<F16>(acc[2 * np + 1], af, bf[2], bf[3]);
                }
            }
            __syncthreads();
        }
        void *c = p.c[member];
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int m = m0 + 16 * warp + g + 8 * (e >> 1), n = n0 + 8 * nt + 2 * t4 + (e & 1);
                if (m < p.m && n < p.n) store_elem(c, static_cast<long long>(m) * p.ldc + n, p.alpha * acc[nt][e], p.out_dtype);
            }
    }
}

// Any element types, any alignment: 64 x 64 tiles, sixteen results a thread, Float32 arithmetic.
__global__ void __launch_bounds__(256) products_simt_kernel(const PointerArgs p) {
    __shared__ float sa[16][65];
    __shared__ float sb[16][65];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    for (long long member = blockIdx.z; member < p.count; member += gridDim.z) {
        const void *a = p.a[member], *b = p.b[member];
        float acc[4][4] = {};
        for (int k0 = 0; k0 < p.k; k0 += 16) {
            for (int i = threadIdx.x; i < 64 * 16; i += 256) {
                int mm, kk;
                if (p.a_mn) { mm = i & 63; kk = i >> 6; } else { kk = i & 15; mm = i >> 4; }
                const int gm = m0 + mm, gk = k0 + kk;
                sa[kk][mm] = (gm < p.m && gk < p.k)
                                 ? load_elem(a, p.a_mn ? static_cast<long long>(gk) * p.lda + gm : static_cast<long long>(gm) * p.lda + gk, p.in_dtype)
                                 : 0.0f;
                int nn;
                if (p.b_mn) { nn = i & 63; kk = i >> 6; } else { kk = i & 15; nn = i >> 4; }
                const int gn = n0 + nn, gk2 = k0 + kk;
                sb[kk][nn] = (gn < p.n && gk2 < p.k)
                                 ? load_elem(b, p.b_mn ? static_cast<long long>(gk2) * p.ldb + gn : static_cast<long long>(gn) * p.ldb + gk2, p.in_dtype)
                                 : 0.0f;
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
        void *c = p.c[member];
        for (int i = 0; i < 4; i++)
            for (int j = 0; j < 4; j++) {
                const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
                if (m < p.m && n < p.n) store_elem(c, static_cast<long long>(m) * p.ldc + n, p.alpha * acc[i][j], p.out_dtype);
            }
    }
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" int tb200_gemm_pointers(const tb200_gemm_desc *d, const void *const *a, const void *const *b, void *const *c,
                                   int64_t count, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!d) return TB200_ERR_NULL;
    if (d->m < 0 || d->n < 0 || d->k < 0 || count < 0) return TB200_ERR_SHAPE;
    if (d->m > (1 << 30) || d->n > (1 << 30) || d->k > (1 << 30)) return TB200_ERR_SHAPE;
    if (ceil_div(d->m, 64) > 65535) return TB200_ERR_SHAPE;   // rows of 64 x 64 tiles are the grid's second axis
    const bool a_mn = d->a_layout == TB200_MN_MAJOR, b_mn = d->b_layout == TB200_MN_MAJOR;
    if ((d->a_layout != TB200_K_MAJOR && !a_mn) || (d->b_layout != TB200_K_MAJOR && !b_mn)) return TB200_ERR_UNSUPPORTED;
    if (d->lda < (a_mn ? d->m : d->k) || d->ldb < (b_mn ? d->n : d->k) || d->ldc < d->n) return TB200_ERR_SHAPE;
    if (d->in_dtype != TB200_F32 && d->in_dtype != TB200_BF16 && d->in_dtype != TB200_F16) return TB200_ERR_DTYPE;
    if (d->out_dtype != TB200_F32 && d->out_dtype != TB200_BF16 && d->out_dtype != TB200_F16) return TB200_ERR_DTYPE;
    if (d->epilogue != TB200_EPI_NONE) return TB200_ERR_UNSUPPORTED;   // plain products, as the reference's call
    if (count == 0 || d->m == 0 || d->n == 0) return TB200_OK;
    if (!a || !b || !c) return TB200_ERR_NULL;
    PointerArgs p{};
    p.a = a; p.b = b; p.c = c; p.count = count;
    p.m = static_cast<int>(d->m); p.n = static_cast<int>(d->n); p.k = static_cast<int>(d->k);
    p.lda = d->lda; p.ldb = d->ldb; p.ldc = d->ldc;
    p.a_mn = a_mn; p.b_mn = b_mn; p.in_dtype = d->in_dtype; p.out_dtype = d->out_dtype;
    p.alpha = d->alpha == 0.0f ? 1.0f : d->alpha;
    const dim3 grid(static_cast<unsigned>(ceil_div(d->n, 64)), static_cast<unsigned>(ceil_div(d->m, 64)),
                    static_cast<unsigned>(count < 32768 ? count : 32768));
    if (d->in_dtype == TB200_F32 || d->force_simt) products_simt_kernel<<<grid, 256, 0, stream>>>(p);
    else if (d->in_dtype == TB200_F16) products_mma_kernel<true><<<grid, 128, 0, stream>>>(p);
    else products_mma_kernel<false><<<grid, 128, 0, stream>>>(p);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}
