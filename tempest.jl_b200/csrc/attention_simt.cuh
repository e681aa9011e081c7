// CUDA-core attention for head dimensions the tensor-core kernels do not take (attention_simt.cu).
#pragma once
#include <cuda_runtime.h>

#include "../../include/tempest_b200.h"

namespace tb200 {
// features of the values (v, o, dout, dv): the queries' and keys' unless the descriptor gives them their own
inline int attention_value_dim(const tb200_attn_desc *d) { return d->value_dim > 0 ? d->value_dim : d->head_dim; }
// what the tensor-core kernels take: 128 features for the queries, keys and values alike
inline bool attention_tensor_geometry(const tb200_attn_desc *d) { return d->head_dim == 128 && attention_value_dim(d) == 128; }
bool attention_simt_takes(const tb200_attn_desc *d);
int attention_simt_fwd(const tb200_attn_desc *d, const void *q, const void *k, const void *v, void *o, float *lse,
                       cudaStream_t stream, const tb200_attn_mask *mask = nullptr);
int attention_simt_bwd(const tb200_attn_desc *d, const void *q, const void *k, const void *v, const void *o,
                       const float *lse, const void *dout, void *dq, void *dk, void *dv, cudaStream_t stream,
                       const tb200_attn_mask *mask = nullptr);
// The tensor-core forward (attention_fwd.cu; 128 features) with masks the device holds and operands at other strides.
// TB200_ERR_UNSUPPORTED where the TMA unit cannot describe the strides.
int attention_tensor_fwd(const tb200_attn_desc *d, const tb200_attn_mask *mask, const void *q, const void *k, const void *v,
                         void *o, float *lse, cudaStream_t stream);
}  // namespace tb200
