// Shared declarations of the attention kernels (generic warp-per-row path and tensor-core path).
#pragma once
#include "common.cuh"

namespace cgpt {

struct AttnDims {
    int batch, sq, sk, hq, hkv, d;
    int causal;   // 1: key k is visible to query q iff k <= offset + q
    int offset;   // query_position_offset
    float scale;  // resolved: attention_scale > 0 ? attention_scale : 1/sqrt(d)
};

int attention_forward_generic_launch(void* out, float* lse, const void* q, const void* k, const void* v,
                                     const AttnDims& dm, int dtype, cudaStream_t s);
int attention_backward_generic_launch(void* dq, void* dk, void* dv, const void* dout, const void* out,
                                      const float* lse, const void* q, const void* k, const void* v,
                                      const AttnDims& dm, int accumulate, int dtype, cudaStream_t s);

// Tensor-core (tcgen05) path: 16-bit dtypes, head_dim 64 or 128. Return CGPT_ERR_UNSUPPORTED when the
// shape is outside what they handle so that the caller falls back to the generic kernels.
int attention_forward_tc_launch(void* out, float* lse, const void* q, const void* k, const void* v,
                                const AttnDims& dm, int dtype, cudaStream_t s);
int attention_backward_tc_launch(void* dq, void* dk, void* dv, const void* dout, const void* out,
                                 const float* lse, const void* q, const void* k, const void* v,
                                 const AttnDims& dm, int accumulate, int dtype, cudaStream_t s);

}  // namespace cgpt
