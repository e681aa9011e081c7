// Shared device and host helpers of the B200 backend: status plumbing, 128-bit
// element access for Float32 and BFloat16 rows, and the warp / row-group
// reductions the fused row kernels are built from.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/tempest_b200.h"

namespace tb200 {

// ---------------------------------------------------------------- host side --

// Records the CUDA error behind a TB200_ERR_CUDA for tb200_last_cuda_error().
int cuda_failed(cudaError_t e);

#define TB200_CUDA(call)                                   \
    do {                                                   \
        cudaError_t e__ = (call);                          \
        if (e__ != cudaSuccess) return ::tb200::cuda_failed(e__); \
    } while (0)

struct DeviceInfo {
    int device = -1;
    int sms = 0;
    int cc_major = 0;
    int cc_minor = 0;
    size_t smem_optin = 0;
};

// Properties of the current device (queried once per device per process).
// Returns TB200_OK, TB200_ERR_CUDA, or TB200_ERR_DEVICE when the device is not
// compute capability 10.x: the library holds sm_100a code only.
int current_device(DeviceInfo *out);

inline bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline size_t dtype_size(int dtype) { return dtype == TB200_F32 ? 4 : (dtype == TB200_BF16 || dtype == TB200_F16) ? 2 : 0; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int next_pow2(int64_t x) {
    int p = 1;
    while (p < x) p <<= 1;
    return p;
}

// -------------------------------------------------------------- device side --

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// exp(x) on the special-function unit: one multiply and one ex2.approx.
__device__ __forceinline__ float fast_exp(float x) { return fast_exp2(x * kLog2e); }

template <typename T, bool VEC>
struct Access;

// Float32, one 128-bit access = 4 elements.
template <>
struct Access<float, true> {
    static constexpr int EPV = 4;
    static __device__ __forceinline__ void load(const float *p, float *v) {
        float4 q = __ldcs(reinterpret_cast<const float4 *>(p));
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
    static __device__ __forceinline__ void load_cached(const float *p, float *v) {
        float4 q = __ldg(reinterpret_cast<const float4 *>(p));
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
    static __device__ __forceinline__ void store(float *p, const float *v) {
        __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
    }
};
template <>
struct Access<float, false> {
    static constexpr int EPV = 1;
    static __device__ __forceinline__ void load(const float *p, float *v) { v[0] = __ldcs(p); }
    static __device__ __forceinline__ void load_cached(const float *p, float *v) { v[0] = __ldg(p); }
    static __device__ __forceinline__ void store(float *p, const float *v) { __stcs(p, v[0]); }
};

__device__ __forceinline__ void unpack_bf16x2(uint32_t w, float &lo, float &hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);  // .x = lo (low half), round to nearest even
    return *reinterpret_cast<uint32_t *>(&h);
}

// BFloat16, one 128-bit access = 8 elements, widened to Float32 in registers.
template <>
struct Access<__nv_bfloat16, true> {
    static constexpr int EPV = 8;
    static __device__ __forceinline__ void unpack(uint4 q, float *v) {
        unpack_bf16x2(q.x, v[0], v[1]);
        unpack_bf16x2(q.y, v[2], v[3]);
        unpack_bf16x2(q.z, v[4], v[5]);
        unpack_bf16x2(q.w, v[6], v[7]);
    }
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float *v) {
        unpack(__ldcs(reinterpret_cast<const uint4 *>(p)), v);
    }
    static __device__ __forceinline__ void load_cached(const __nv_bfloat16 *p, float *v) {
        unpack(__ldg(reinterpret_cast<const uint4 *>(p)), v);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float *v) {
        uint4 q;
        q.x = pack_bf16x2(v[0], v[1]);
        q.y = pack_bf16x2(v[2], v[3]);
        q.z = pack_bf16x2(v[4], v[5]);
        q.w = pack_bf16x2(v[6], v[7]);
        __stcs(reinterpret_cast<uint4 *>(p), q);
    }
};
template <>
struct Access<__nv_bfloat16, false> {
    static constexpr int EPV = 1;
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float *v) {
        v[0] = __uint_as_float(static_cast<uint32_t>(__ldcs(reinterpret_cast<const unsigned short *>(p))) << 16);
    }
    static __device__ __forceinline__ void load_cached(const __nv_bfloat16 *p, float *v) {
        v[0] = __uint_as_float(static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned short *>(p))) << 16);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float *v) {
        __nv_bfloat16 h = __float2bfloat16_rn(v[0]);
        __stcs(reinterpret_cast<unsigned short *>(p), *reinterpret_cast<unsigned short *>(&h));
    }
};

// A statistic stored in Float32 or, where the plan's value is half precision,
// rounded once to BFloat16.
__device__ __forceinline__ void store_stat(void *base, int64_t i, float v, int as_bf16) {
    if (as_bf16) reinterpret_cast<__nv_bfloat16 *>(base)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float *>(base)[i] = v;
}
__device__ __forceinline__ float load_stat(const void *base, int64_t i, int as_bf16) {
    return as_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(base)[i])
                   : reinterpret_cast<const float *>(base)[i];
}

struct SumOp {
    __device__ __forceinline__ float operator()(float a, float b) const { return a + b; }
};
struct MaxOp {
    __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); }
};

// Where a thread sits among the `tpr` threads that share one row.  A block
// holds blockDim.x / tpr rows ("slots"); tpr is a power of two.
struct RowCtx {
    int tpr;    // threads per row
    int slot;   // which of the block's rows
    int t;      // index among the row's threads
    int wpr;    // warps per row (tpr / 32, at least 1 when tpr >= 32)
    int lane, warp;
    float *red; // shared scratch: 2 phases x 32 warps x kRedWidth floats
    int phase;
};
constexpr int kRedWidth = 2;

__device__ __forceinline__ RowCtx make_row_ctx(int tpr, float *red) {
    RowCtx c;
    c.tpr = tpr;
    c.slot = threadIdx.x / tpr;
    c.t = threadIdx.x - c.slot * tpr;
    c.wpr = tpr >> 5;
    c.lane = threadIdx.x & 31;
    c.warp = threadIdx.x >> 5;
    c.red = red;
    c.phase = 0;
    return c;
}

// All-reduce of NV values over the threads of one row.  Up to 32 threads: xor
// shuffles inside the warp.  More: shuffles, then one shared-memory exchange
// between the row's warps with a single __syncthreads (two alternating
// buffers make a second barrier unnecessary).  Every thread of the block must
// call it the same number of times.  The order of combination is fixed, so
// results do not vary from run to run.
template <int NV, typename Op>
__device__ __forceinline__ void row_allreduce(float (&v)[NV], RowCtx &c, Op op) {
    static_assert(NV <= kRedWidth, "widen kRedWidth");
    if (c.tpr <= 32) {
        for (int o = c.tpr >> 1; o > 0; o >>= 1)
#pragma unroll
            for (int i = 0; i < NV; i++) v[i] = op(v[i], __shfl_xor_sync(0xffffffffu, v[i], o));
        return;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int i = 0; i < NV; i++) v[i] = op(v[i], __shfl_xor_sync(0xffffffffu, v[i], o));
    float *buf = c.red + c.phase * (32 * kRedWidth);
    if (c.lane == 0)
#pragma unroll
        for (int i = 0; i < NV; i++) buf[c.warp * kRedWidth + i] = v[i];
    __syncthreads();
    const float *mine = buf + c.slot * c.wpr * kRedWidth;
#pragma unroll
    for (int i = 0; i < NV; i++) v[i] = mine[i];
    for (int w = 1; w < c.wpr; w++)
#pragma unroll
        for (int i = 0; i < NV; i++) v[i] = op(v[i], mine[w * kRedWidth + i]);
    c.phase ^= 1;
}

template <typename Op>
__device__ __forceinline__ float row_allreduce1(float x, RowCtx &c, Op op) {
    float v[1] = {x};
    row_allreduce<1>(v, c, op);
    return v[0];
}

// One element of an array of any of the three element types, as Float32.
__device__ __forceinline__ float load_elem(const void *p, long long i, int dtype) {
    if (dtype == TB200_F32) return static_cast<const float *>(p)[i];
    if (dtype == TB200_F16) return __half2float(static_cast<const __half *>(p)[i]);
    return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
}
__device__ __forceinline__ void store_elem(void *p, long long i, float v, int dtype) {
    if (dtype == TB200_F32) static_cast<float *>(p)[i] = v;
    else if (dtype == TB200_F16) static_cast<__half *>(p)[i] = __float2half_rn(v);
    else static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
}

}  // namespace tb200
