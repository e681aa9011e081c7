// Data-parallel update: the replicas' gradient sum and the SGD step as ONE kernel over NVLink.
//
// The reference spells the exchange of a data-parallel step as `r .+ s` over the devices' gradients
// followed by the update on every device, realised by peer copies and sums
// (src/Compiler/plan/devices.jl:7-11, test/fixtures/devices.jl `shards_sgd!`), and states the property
// that matters: replicas hold the same bits after every step.  Here rank r owns the r-th slice of a
// range of the flat parameter buffer.  For its slice it takes the sum of every replica's gradients --
// `multimem.ld_reduce` (the NVSwitch adds the replicas' values on the way, Float32 accumulation) where
// the buffers are bound to a multicast object, plain loads from each peer's memory otherwise -- forms
// w - rate * sum once, and writes the new weights into EVERY replica's parameter buffer
// (`multimem.st`, or one store per peer).  Each value is computed by exactly one rank and broadcast, so
// the replicas are bit-equal by construction, the summed gradient is never written anywhere, and the
// bytes a GPU puts on its links are about its own gradients once (the all-gather half of a ring
// all-reduce disappears into the switch's broadcast).
//
// Ranks meet twice inside the launch: before the first load (every replica's gradients are complete
// and none of them still reads the old weights) and after the last store (every replica holds the
// new weights).  A meeting is one counter per (block, peer) in each rank's signal pad: a block adds 1
// to its slot in every peer's pad (release) and waits until every peer's slot in its own pad has
// reached the block's own count (acquire).  Block b of a rank only ever waits for block b of the
// other ranks, so no two blocks of one GPU wait on one another and nothing needs to be co-resident.
// Every wait is bounded (two seconds): on expiry the block records an error and returns.
//
// No TMA, no bulk copy and no cluster multicast load touches a peer's memory here.
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kMaxRanks = 16;
constexpr int kDpThreads = 512;
constexpr int kDpMaxBlocks = 128;

__device__ int g_dp_error = 0;

struct DpArgs {
    const uint4 *grads[kMaxRanks];   // every rank's gradient range as mapped into this process (entry `rank`: local)
    uint4 *params[kMaxRanks];
    uint32_t *pads[kMaxRanks];       // signal pads: [block][rank] counters, zero before the first launch
    const uint4 *grads_mc;           // the same ranges through the multicast mapping, or null
    uint4 *params_mc;
    uint32_t *counts;                // local: how many meetings each block has been to
    long long vectors;               // 16-byte vectors (8 BFloat16) in the range
    float alpha;
    int rank, world;
    unsigned long long wait_ns;
};

__device__ __forceinline__ uint64_t now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// All ranks' block `blockIdx.x` meet.  Returns false if a peer did not arrive in time.
__device__ __forceinline__ bool meet(const DpArgs &a, int *failed) {
    __syncthreads();
    __shared__ uint32_t target;
    if (threadIdx.x == 0) {
        target = a.counts[blockIdx.x] + 1;
        a.counts[blockIdx.x] = target;
    }
    // everything this block wrote (to any replica) is ordered before its arrival
    __threadfence_system();
    __syncthreads();
    const uint32_t want = target;
    if (threadIdx.x < a.world && threadIdx.x != a.rank) {
        uint32_t *there = a.pads[threadIdx.x] + blockIdx.x * kMaxRanks + a.rank;
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(there) : "memory");
        const uint32_t *here = a.pads[a.rank] + blockIdx.x * kMaxRanks + threadIdx.x;
        const uint64_t t0 = now_ns();
        uint32_t seen = 0;
        while (true) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(here) : "memory");
            if (static_cast<int32_t>(seen - want) >= 0) break;
            if (*reinterpret_cast<volatile int *>(failed) || now_ns() - t0 > a.wait_ns) {
                *reinterpret_cast<volatile int *>(failed) = 1;
                atomicCAS(&g_dp_error, 0, 1 + a.rank * 16 + static_cast<int>(threadIdx.x));
                break;
            }
        }
    }
    __syncthreads();
    return *reinterpret_cast<volatile int *>(failed) == 0;
}

__device__ __forceinline__ uint4 mc_sum(const uint4 *p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mc_store(uint4 *p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
                 ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 peer_load(const uint4 *p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void peer_store(uint4 *p, uint4 v) {
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};"
                 ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// w - rate * g on eight BFloat16 values, Float32 arithmetic, one rounding
__device__ __forceinline__ uint4 step8(uint4 w, uint4 g, float alpha) {
    float wf[8], gf[8];
    Access<__nv_bfloat16, true>::unpack(w, wf);
    Access<__nv_bfloat16, true>::unpack(g, gf);
#pragma unroll
    for (int i = 0; i < 8; i++) wf[i] = fmaf(alpha, gf[i], wf[i]);
    return make_uint4(pack_bf16x2(wf[0], wf[1]), pack_bf16x2(wf[2], wf[3]), pack_bf16x2(wf[4], wf[5]),
                      pack_bf16x2(wf[6], wf[7]));
}

template <bool MULTIMEM>
__global__ void __launch_bounds__(kDpThreads) dp_update_kernel(const DpArgs a) {
    __shared__ int failed;
    if (threadIdx.x == 0) failed = 0;
    if (!meet(a, &failed)) return;
    // this rank's slice of the range, spread over its blocks
    const long long first = a.vectors * a.rank / a.world, last = a.vectors * (a.rank + 1) / a.world;
    const long long stride = static_cast<long long>(gridDim.x) * kDpThreads;
    constexpr int U = 8;   // vectors in flight per thread: a load through the switch takes microseconds
    for (long long v0 = first + blockIdx.x * static_cast<long long>(kDpThreads) + threadIdx.x; v0 < last; v0 += U * stride) {
        uint4 g[U], w[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const long long v = v0 + u * stride;
            if (v < last) {
                if constexpr (MULTIMEM) {
                    g[u] = mc_sum(a.grads_mc + v);
                } else {
                    // replicas in rank order, Float32 sums, rounded once as the switch's result is
                    float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
                    for (int r = 0; r < a.world; r++) {
                        float f[8];
                        Access<__nv_bfloat16, true>::unpack(peer_load(a.grads[r] + v), f);
#pragma unroll
                        for (int i = 0; i < 8; i++) acc[i] += f[i];
                    }
                    g[u] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                      pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
                }
                w[u] = a.params[a.rank][v];
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const long long v = v0 + u * stride;
            if (v < last) {
                const uint4 next = step8(w[u], g[u], a.alpha);
                if constexpr (MULTIMEM) {
                    mc_store(a.params_mc + v, next);
                } else {
                    for (int r = 0; r < a.world; r++) peer_store(a.params[r] + v, next);
                }
            }
        }
    }
    meet(a, &failed);
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" size_t tb200_dp_signal_bytes(void) { return static_cast<size_t>(kDpMaxBlocks) * kMaxRanks * sizeof(uint32_t); }
extern "C" size_t tb200_dp_state_bytes(void) { return static_cast<size_t>(kDpMaxBlocks) * sizeof(uint32_t); }

extern "C" int tb200_dp_update(const tb200_dp_desc *d, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!d) return TB200_ERR_NULL;
    if (d->dtype != TB200_BF16) return TB200_ERR_DTYPE;
    if (d->world < 1 || d->world > kMaxRanks || d->rank < 0 || d->rank >= d->world) return TB200_ERR_SHAPE;
    if (d->count < 0 || d->count % 8 != 0) return TB200_ERR_SHAPE;
    if (d->count == 0) return TB200_OK;
    if (!d->state) return TB200_ERR_WORKSPACE;
    const bool multimem = d->grads_multicast != nullptr && d->params_multicast != nullptr;
    DpArgs a{};
    for (int r = 0; r < d->world; r++) {
        if (!d->signals[r] || !aligned_to(d->signals[r], 4)) return TB200_ERR_NULL;
        if (!multimem || r == d->rank) {
            if (!d->grads[r] || !d->params[r]) return TB200_ERR_NULL;
            if (!aligned_to(d->grads[r], 16) || !aligned_to(d->params[r], 16)) return TB200_ERR_ALIGN;
        }
        a.grads[r] = static_cast<const uint4 *>(d->grads[r]);
        a.params[r] = static_cast<uint4 *>(d->params[r]);
        a.pads[r] = static_cast<uint32_t *>(d->signals[r]);
    }
    if (multimem && (!aligned_to(d->grads_multicast, 16) || !aligned_to(d->params_multicast, 16))) return TB200_ERR_ALIGN;
    a.grads_mc = static_cast<const uint4 *>(d->grads_multicast);
    a.params_mc = static_cast<uint4 *>(d->params_multicast);
    a.counts = static_cast<uint32_t *>(d->state);
    a.vectors = d->count / 8;
    a.alpha = d->alpha;
    a.rank = d->rank; a.world = d->world;
    a.wait_ns = 2000000000ull;
    DeviceInfo dev;
    int st = current_device(&dev);
    if (st) return st;
    // every rank must launch the same number of blocks (block b meets block b): a function of the
    // descriptor alone, not of the device
    // (measured on 8 B200s, 84 MB of gradients: 48 blocks 0.289 ms, 16 blocks 0.261 ms, 8 blocks 0.236 ms -- more
    // blocks take SMs from the products that run beside the exchange without moving the bytes any faster)
    int blocks = d->blocks > 0 ? d->blocks : 8;
    if (blocks > kDpMaxBlocks) blocks = kDpMaxBlocks;
    if (multimem) dp_update_kernel<true><<<blocks, kDpThreads, 0, stream>>>(a);
    else dp_update_kernel<false><<<blocks, kDpThreads, 0, stream>>>(a);
    TB200_CUDA(cudaGetLastError());
    return TB200_OK;
}

extern "C" int tb200_dp_error(void) {
    int code = 0, zero = 0;
    TB200_CUDA(cudaDeviceSynchronize());
    TB200_CUDA(cudaMemcpyFromSymbol(&code, g_dp_error, sizeof(int)));
    if (code) TB200_CUDA(cudaMemcpyToSymbol(g_dp_error, &zero, sizeof(int)));
    return code;
}
