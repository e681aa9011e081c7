// Pointwise maps and the folds that are not row reductions, for sm_100a:
//   * squared-error loss with its gradient (a full reduction merged in a fixed order),
//   * column sums over the rows of a matrix (bias gradients: a fold over the other axis),
//   * y += alpha * x (the gradient-descent update).
// All are HBM-bound streams: 128-bit accesses, grids sized to the SM count,
// Float32 arithmetic, one rounding at the store, results that repeat bit for bit.
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kThreads = 256;

// Sum over a block in a fixed order; the result is valid in thread 0.
__device__ __forceinline__ float block_sum(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.0f;
    if (threadIdx.x == 0)
        for (int w = 0; w < (blockDim.x >> 5); w++) s += red[w];
    __syncthreads();
    return s;
}

// loss = scale * sum((a - b)^2) ; grad = grad_scale * 2 (a - b) [* (1 - a^2) through a tanh].
// Each block folds a contiguous span and writes one partial; the block that finishes last adds the
// partials in index order, so the sum does not depend on scheduling.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads) squared_error_kernel(const T *a, const T *b, T *grad, float *loss,
                                                                 float *partials, unsigned int *ticket,
                                                                 long long count, float scale, float grad_scale,
                                                                 int through_tanh) {
    __shared__ float red[kThreads / 32];
    __shared__ bool last;
    constexpr int EPV = Access<T, VEC>::EPV;
    const long long nvec = count / EPV;
    float s = 0.0f;
    for (long long i = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * kThreads) {
        float av[EPV], bv[EPV], gv[EPV];
        Access<T, VEC>::load(a + i * EPV, av);
        if (b) Access<T, VEC>::load(b + i * EPV, bv);
#pragma unroll
        for (int e = 0; e < EPV; e++) {
            const float d = b ? av[e] - bv[e] : av[e];
            s = fmaf(d, d, s);
            float g = grad_scale * (2.0f * d);
            if (through_tanh) g *= 1.0f - av[e] * av[e];
            gv[e] = g;
        }
        if (grad) Access<T, VEC>::store(grad + i * EPV, gv);
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = s;
        __threadfence();
        last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (last) {
        __threadfence();
        float t = 0.0f;
        for (int i = threadIdx.x; i < static_cast<int>(gridDim.x); i += kThreads)
            t += reinterpret_cast<volatile float *>(partials)[i];
        t = block_sum(t, red);
        if (threadIdx.x == 0) {
            *loss = scale * t;
            *ticket = 0;   // ready for the next call
        }
    }
}

// Column sums over the rows of x[rows][n]: a block covers 32 x EPV columns (one 128-bit access per
// thread per row when VEC) and one slab of rows; its 8 row lanes stride the slab's rows in order and
// merge in a fixed tree.  partial[slab][n] in Float32; colsum_merge_kernel adds the slabs in order.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) colsum_slab_kernel(const T *x, float *partial, long long rows, int n,
                                                          long long ld, int slabs) {
    constexpr int EPV = Access<T, VEC>::EPV;
    __shared__ float sm[8][32 * EPV + 1];
    const int tx = threadIdx.x & 31;
    const int col = (blockIdx.x * 32 + tx) * EPV;
    const int lane = threadIdx.x >> 5;
    const int slab = blockIdx.y;
    const long long per = (rows + slabs - 1) / slabs;
    const long long r0 = slab * per, r1 = min(rows, r0 + per);
    float s0[EPV], s1[EPV];
#pragma unroll
    for (int e = 0; e < EPV; e++) s0[e] = s1[e] = 0.0f;
    if (col < n) {
        long long r = r0 + lane;
        for (; r + 8 < r1; r += 16) {   // two rows in flight per thread
            float v0[EPV], v1[EPV];
            Access<T, VEC>::load(x + r * ld + col, v0);
            Access<T, VEC>::load(x + (r + 8) * ld + col, v1);
#pragma unroll
            for (int e = 0; e < EPV; e++) { s0[e] += v0[e]; s1[e] += v1[e]; }
        }
        for (; r < r1; r += 8) {
            float v0[EPV];
            Access<T, VEC>::load(x + r * ld + col, v0);
#pragma unroll
            for (int e = 0; e < EPV; e++) s0[e] += v0[e];
        }
    }
#pragma unroll
    for (int e = 0; e < EPV; e++) sm[lane][tx * EPV + e] = s0[e] + s1[e];
    __syncthreads();
    for (int c = threadIdx.x; c < 32 * EPV; c += 256) {
        const int gc = blockIdx.x * 32 * EPV + c;
        if (gc < n) {
            float t = 0.0f;
#pragma unroll
            for (int l = 0; l < 8; l++) t += sm[l][c];
            partial[static_cast<long long>(slab) * n + gc] = t;
        }
    }
}

// Eight lanes a column, each over every eighth slab in order, then the lanes in a fixed tree: the same sum whatever
// the grid, and 32 columns a block so that a narrow array still spreads over many SMs.
template <typename T>
__global__ void __launch_bounds__(256) colsum_merge_kernel(const float *partial, T *out, int n, int slabs,
                                                           float scale) {
    __shared__ float sm[8][33];
    const int tx = threadIdx.x & 31, lane = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + tx;
    float t = 0.0f;
    if (col < n)
        for (int s = lane; s < slabs; s += 8) t += partial[static_cast<long long>(s) * n + col];
    sm[lane][tx] = t;
    __syncthreads();
    if (lane == 0 && col < n) {
        const float sum = ((sm[0][tx] + sm[1][tx]) + (sm[2][tx] + sm[3][tx])) + ((sm[4][tx] + sm[5][tx]) + (sm[6][tx] + sm[7][tx]));
        float o[1] = {sum * scale};
        Access<T, false>::store(out + col, o);
    }
}

// y = y + alpha * x, elementwise; x may have another element type than y (BFloat16 gradients
// into Float32 or BFloat16 weights).  VEC: both arrays 16-byte aligned, eight elements a thread in one
// or two 128-bit accesses per array and the ragged end one element a thread; otherwise (a view that
// starts at an odd element) every element goes alone.
template <typename TY, typename TX, bool VEC>
__global__ void __launch_bounds__(kThreads) axpy_kernel(TY *y, const TX *x, float alpha, long long count) {
    const long long first = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
    const long long stride = static_cast<long long>(gridDim.x) * kThreads;
    if constexpr (!VEC) {
        for (long long i = first; i < count; i += stride) {
            float yv[1], xv[1];
            Access<TY, false>::load(y + i, yv);
            Access<TX, false>::load(x + i, xv);
            yv[0] = fmaf(alpha, xv[0], yv[0]);
            Access<TY, false>::store(y + i, yv);
        }
        return;
    }
    constexpr int EPV = 8;
    const long long nvec = count / EPV;
    for (long long i = first; i < nvec; i += stride) {
        float yv[EPV], xv[EPV];
#pragma unroll
        for (int j = 0; j < EPV; j += Access<TY, true>::EPV) Access<TY, true>::load(y + i * EPV + j, yv + j);
#pragma unroll
        for (int j = 0; j < EPV; j += Access<TX, true>::EPV) Access<TX, true>::load(x + i * EPV + j, xv + j);
#pragma unroll
        for (int e = 0; e < EPV; e++) yv[e] = fmaf(alpha, xv[e], yv[e]);
#pragma unroll
        for (int j = 0; j < EPV; j += Access<TY, true>::EPV) Access<TY, true>::store(y + i * EPV + j, yv + j);
    }
    const long long tail = nvec * EPV + first;
    if (tail < count && first < EPV) {
        float yv[1], xv[1];
        Access<TY, false>::load(y + tail, yv);
        Access<TX, false>::load(x + tail, xv);
        yv[0] = fmaf(alpha, xv[0], yv[0]);
        Access<TY, false>::store(y + tail, yv);
    }
}

int stream_grid(const DeviceInfo &dev, long long work_items) {
    long long g = static_cast<long long>(dev.sms) * 8;
    const long long need = ceil_div(work_items, kThreads);
    if (g > need) g = need;
    return static_cast<int>(g < 1 ? 1 : g);
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" size_t tb200_squared_error_workspace_bytes(void) {
    // one partial per block (at most 8 blocks per SM on up to 512 SMs) and the ticket
    return 4096 * sizeof(float) + 16;
}

extern "C" int tb200_squared_error(const void *a, const void *b, void *grad, float *loss, int64_t count,
                                   float scale, float grad_scale, int through_tanh, int dtype, void *workspace,
                                   size_t workspace_bytes, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (dtype != TB200_F32 && dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (count < 0) return TB200_ERR_SHAPE;
    if (!loss) return TB200_ERR_NULL;
    if (count > 0 && !a) return TB200_ERR_NULL;
    if (!workspace || workspace_bytes < tb200_squared_error_workspace_bytes() || !aligned_to(workspace, 16))
        return TB200_ERR_WORKSPACE;
    const size_t es = dtype_size(dtype);
    if (!aligned_to(a, es) || !aligned_to(b, es) || !aligned_to(grad, es) || !aligned_to(loss, 4))
        return TB200_ERR_ALIGN;
    DeviceInfo dev;
    int st = current_device(&dev);
    if (st) return st;
    float *partials = static_cast<float *>(workspace);
    unsigned int *ticket = reinterpret_cast<unsigned int *>(partials + 4096);
    const bool vec = aligned_to(a, 16) && aligned_to(b, 16) && aligned_to(grad, 16) && count % (16 / es) == 0;
    int grid = stream_grid(dev, count / (vec ? 16 / es : 1));
    if (grid > 4096) grid = 4096;
    // The ticket must start at zero: the first call on a workspace clears it; every call leaves it zero.
#define TB200_SQERR(T, V)                                                                                         \
    squared_error_kernel<T, V><<<grid, kThreads, 0, stream>>>(static_cast<const T *>(a), static_cast<const T *>(b), \
                                                              static_cast<T *>(grad), loss, partials, ticket, count, \
                                                              scale, grad_scale, through_tanh)
    if (dtype == TB200_F32) { if (vec) TB200_SQERR(float, true); else TB200_SQERR(float, false); }
    else { if (vec) TB200_SQERR(__nv_bfloat16, true); else TB200_SQERR(__nv_bfloat16, false); }
#undef TB200_SQERR
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

extern "C" int tb200_workspace_clear(void *workspace, size_t workspace_bytes, void *stream_) {
    if (!workspace) return TB200_ERR_NULL;
    TB200_CUDA(cudaMemsetAsync(workspace, 0, workspace_bytes, static_cast<cudaStream_t>(stream_)));
    return TB200_OK;
}

namespace {
// Row slabs of the column sum: enough blocks to fill the device, at least 64 rows each.
int colsum_slabs(const DeviceInfo &dev, int64_t rows, int64_t n, int epv) {
    const int64_t col_blocks = ceil_div(n, 32 * epv);
    int64_t slabs = ceil_div(static_cast<int64_t>(dev.sms) * 4, col_blocks);
    const int64_t most = ceil_div(rows, 64);
    if (slabs > most) slabs = most;
    return static_cast<int>(slabs < 1 ? 1 : slabs);
}
}  // namespace

extern "C" size_t tb200_colsum_workspace_bytes(int64_t rows, int64_t n) {
    if (rows <= 0 || n <= 0) return 0;
    DeviceInfo dev;
    if (current_device(&dev) != TB200_OK) return 0;
    // the scalar schedule has the most column blocks' worth of slabs: cover it
    const int slabs = colsum_slabs(dev, rows, n, 8) > colsum_slabs(dev, rows, n, 1) ? colsum_slabs(dev, rows, n, 8)
                                                                                    : colsum_slabs(dev, rows, n, 1);
    return static_cast<size_t>(slabs) * n * sizeof(float);
}

extern "C" int tb200_colsum(const void *x, void *out, int64_t rows, int64_t n, int64_t ld, float scale, int dtype,
                            void *workspace, size_t workspace_bytes, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (dtype != TB200_F32 && dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (rows < 0 || n < 0 || ld < n || n > INT32_MAX) return TB200_ERR_SHAPE;
    if (n == 0) return TB200_OK;
    if (!out || (rows > 0 && !x)) return TB200_ERR_NULL;
    const size_t es = dtype_size(dtype);
    if (!aligned_to(x, es) || !aligned_to(out, es)) return TB200_ERR_ALIGN;
    if (rows == 0) {
        TB200_CUDA(cudaMemsetAsync(out, 0, n * es, stream));
        return TB200_OK;
    }
    DeviceInfo dev;
    int st = current_device(&dev);
    if (st) return st;
    const int epv_vec = static_cast<int>(16 / es);
    const bool vec = aligned_to(x, 16) && n % epv_vec == 0 && ld % epv_vec == 0;
    const int epv = vec ? epv_vec : 1;
    const int slabs = colsum_slabs(dev, rows, n, epv);
    const size_t need = static_cast<size_t>(slabs) * n * sizeof(float);
    if (!workspace || workspace_bytes < need || !aligned_to(workspace, 16)) return TB200_ERR_WORKSPACE;
    float *partial = static_cast<float *>(workspace);
    dim3 grid(static_cast<unsigned>(ceil_div(n, 32 * epv)), static_cast<unsigned>(slabs));
    const unsigned merge_blocks = static_cast<unsigned>(ceil_div(n, 32));
    const int ni = static_cast<int>(n);
    if (dtype == TB200_F32) {
        const float *xp = static_cast<const float *>(x);
        if (vec) colsum_slab_kernel<float, true><<<grid, 256, 0, stream>>>(xp, partial, rows, ni, ld, slabs);
        else colsum_slab_kernel<float, false><<<grid, 256, 0, stream>>>(xp, partial, rows, ni, ld, slabs);
        colsum_merge_kernel<float><<<merge_blocks, 256, 0, stream>>>(partial, static_cast<float *>(out), ni, slabs,
                                                                     scale);
    } else {
        const __nv_bfloat16 *xp = static_cast<const __nv_bfloat16 *>(x);
        if (vec) colsum_slab_kernel<__nv_bfloat16, true><<<grid, 256, 0, stream>>>(xp, partial, rows, ni, ld, slabs);
        else colsum_slab_kernel<__nv_bfloat16, false><<<grid, 256, 0, stream>>>(xp, partial, rows, ni, ld, slabs);
        colsum_merge_kernel<__nv_bfloat16><<<merge_blocks, 256, 0, stream>>>(
            partial, static_cast<__nv_bfloat16 *>(out), ni, slabs, scale);
    }
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

extern "C" int tb200_axpy(void *y, const void *x, float alpha, int64_t count, int y_dtype, int x_dtype,
                          void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if ((y_dtype != TB200_F32 && y_dtype != TB200_BF16) || (x_dtype != TB200_F32 && x_dtype != TB200_BF16))
        return TB200_ERR_DTYPE;
    if (count < 0) return TB200_ERR_SHAPE;
    if (count == 0) return TB200_OK;
    if (!y || !x) return TB200_ERR_NULL;
    if (!aligned_to(y, dtype_size(y_dtype)) || !aligned_to(x, dtype_size(x_dtype))) return TB200_ERR_ALIGN;
    DeviceInfo dev;
    int st = current_device(&dev);
    if (st) return st;
    // the vector path needs 16-byte alignment; unaligned views go one element a thread
    const bool vec = aligned_to(y, 16) && aligned_to(x, 16);
    const int grid = stream_grid(dev, vec ? ceil_div(count, 8) : count);
#define TB200_AXPY(TY, TX)                                                                                              \
    do {                                                                                                                \
        if (vec) axpy_kernel<TY, TX, true><<<grid, kThreads, 0, stream>>>(static_cast<TY *>(y), static_cast<const TX *>(x), alpha, count);  \
        else axpy_kernel<TY, TX, false><<<grid, kThreads, 0, stream>>>(static_cast<TY *>(y), static_cast<const TX *>(x), alpha, count); \
    } while (0)
    if (y_dtype == TB200_F32 && x_dtype == TB200_F32) TB200_AXPY(float, float);
    else if (y_dtype == TB200_F32) TB200_AXPY(float, __nv_bfloat16);
    else if (x_dtype == TB200_F32) TB200_AXPY(__nv_bfloat16, float);
    else TB200_AXPY(__nv_bfloat16, __nv_bfloat16);
#undef TB200_AXPY
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}
