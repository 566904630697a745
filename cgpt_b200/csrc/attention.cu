// C ABI of causal GQA attention forward (with saved log-sum-exp) and backward; validation follows
// the reference (src/ops/backward/attention_backward.cu:1868-1893) and dispatches to the tensor-core
// kernels when they apply, else to the generic kernels.
#include <cmath>

#include "attention.h"

namespace cgpt {
namespace {

int resolve(AttnDims* dm, size_t batch, size_t sq, size_t sk, size_t hq, size_t hkv, size_t d, float scale, int causal,
            size_t offset) {
    if (batch == 0 || sq == 0 || sk == 0 || hq == 0 || hkv == 0 || d == 0 || hq % hkv != 0) return CGPT_ERR_SHAPE;
    if (d > 256) return CGPT_ERR_UNSUPPORTED;
    const size_t lim = 0x7fffffffull;
    if (batch > lim || sq > lim || sk > lim || hq > lim || hkv > lim || offset > lim) return CGPT_ERR_SHAPE;
    if (!std::isfinite(scale) || scale < 0.f) return CGPT_ERR_OPTION;
    if (causal && offset + sq > sk) return CGPT_ERR_OPTION;
    *dm = AttnDims{static_cast<int>(batch), static_cast<int>(sq), static_cast<int>(sk), static_cast<int>(hq),
                   static_cast<int>(hkv), static_cast<int>(d), causal ? 1 : 0, static_cast<int>(offset),
                   scale > 0.f ? scale : 1.0f / std::sqrt(static_cast<float>(d))};
    return CGPT_OK;
}

}  // namespace
}  // namespace cgpt

using namespace cgpt;

extern "C" int cgpt_attention_forward(void* out, float* lse, const void* q, const void* k, const void* v, size_t batch,
                                      size_t sq, size_t sk, size_t hq, size_t hkv, size_t head_dim, float scale,
                                      int causal, size_t offset, int dtype, int force_generic, cgpt_stream_t stream) {
    if (!out || !q || !k || !v) return CGPT_ERR_NULL;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    AttnDims dm;
    CGPT_TRY(resolve(&dm, batch, sq, sk, hq, hkv, head_dim, scale, causal, offset));
    auto s = static_cast<cudaStream_t>(stream);
    if (!force_generic) {
        const int rc = attention_forward_tc_launch(out, lse, q, k, v, dm, dtype, s);
        if (rc != CGPT_ERR_UNSUPPORTED) return rc;
    }
    return attention_forward_generic_launch(out, lse, q, k, v, dm, dtype, s);
}

extern "C" int cgpt_attention_backward(void* dq, void* dk, void* dv, const void* dout, const void* out,
                                       const float* lse, const void* q, const void* k, const void* v, size_t batch,
                                       size_t sq, size_t sk, size_t hq, size_t hkv, size_t head_dim, float scale,
                                       int causal, size_t offset, int accumulate, int dtype, int force_generic,
                                       cgpt_stream_t stream) {
    if (!dq || !dk || !dv || !dout || !q || !k || !v) return CGPT_ERR_NULL;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    AttnDims dm;
    CGPT_TRY(resolve(&dm, batch, sq, sk, hq, hkv, head_dim, scale, causal, offset));
    auto s = static_cast<cudaStream_t>(stream);
    if (!force_generic && out != nullptr && lse != nullptr) {
        const int rc = attention_backward_tc_launch(dq, dk, dv, dout, out, lse, q, k, v, dm, accumulate, dtype, s);
        if (rc != CGPT_ERR_UNSUPPORTED) return rc;
    }
    return attention_backward_generic_launch(dq, dk, dv, dout, out, lse, q, k, v, dm, accumulate, dtype, s);
}
