// Tensor-core attention kernels (placeholder dispatch until the tcgen05 kernels land in this file).
#include "attention.h"

namespace cgpt {

int attention_forward_tc_launch(void*, float*, const void*, const void*, const void*, const AttnDims&, int, cudaStream_t) {
    return CGPT_ERR_UNSUPPORTED;
}
int attention_backward_tc_launch(void*, void*, void*, const void*, const void*, const float*, const void*, const void*,
                                 const void*, const AttnDims&, int, int, cudaStream_t) {
    return CGPT_ERR_UNSUPPORTED;
}

}  // namespace cgpt
