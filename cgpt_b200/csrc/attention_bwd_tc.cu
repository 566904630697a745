// Tensor-core attention backward (stub until the kernels below are filled in).
#include "attention.h"

namespace cgpt {

int attention_backward_tc_launch(void*, void*, void*, const void*, const void*, const float*, const void*, const void*,
                                 const void*, const AttnDims&, int, int, cudaStream_t) {
    return CGPT_ERR_UNSUPPORTED;
}

}  // namespace cgpt
