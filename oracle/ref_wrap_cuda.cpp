// TEST INFRASTRUCTURE: a flat C wrapper around the reference's own CUDA operators.
//
// Compiled together with the reference's untouched GPU sources (src/ops/*.cu, src/ops/backward/*.cu except the
// cuBLASLt-based linear files, src/core/tensor.cu) by oracle/build_ref.py into oracle/_ref/libcgpt_ref_cuda.so,
// for sm_100a. It contains no arithmetic of its own: every function wraps the caller's device pointers in
// non-owning Tensor::device_view objects, calls one reference entry point on the given stream and returns.
// The GPU parity tests run the reference's kernels and this repository's kernels on the same device inputs.
//
// dtype codes follow the reference's Dtype enum (include/core/dtype.h:12-21): 0 = F16, 1 = BF16, 2 = F32.
#include <cuda_runtime.h>

#include <exception>
#include <string>
#include <vector>

#include "core/tensor.h"
#include "ops/attention.h"
#include "ops/backward/attention_backward.h"
#include "ops/backward/embedding_backward.h"
#include "ops/backward/rmsnorm_backward.h"
#include "ops/backward/rope_backward.h"
#include "ops/backward/swiglu_backward.h"
#include "ops/cross_entropy.h"
#include "ops/cut_cross_entropy.h"
#include "ops/embedding.h"
#include "ops/rmsnorm.h"
#include "ops/rope.h"
#include "ops/swiglu.h"

namespace {

std::string g_error;
using Shape = std::vector<std::size_t>;

Tensor view(const void* p, Shape shape, int dtype) {
    return Tensor::device_view(std::move(shape), const_cast<void*>(p), static_cast<Dtype>(dtype));
}

template <typename F>
int guarded(F&& f) {
    try {
        f();
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            g_error = cudaGetErrorString(e);
            return -2;
        }
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    } catch (...) {
        g_error = "unknown exception";
        return -1;
    }
}

FlashAttentionOptions attn_options(std::size_t hq, std::size_t hkv, std::size_t d, int causal, std::size_t offset, float scale) {
    FlashAttentionOptions o{};
    o.num_query_heads = hq;
    o.num_kv_heads = hkv;
    o.head_dim = d;
    o.causal = causal != 0;
    o.query_position_offset = offset;
    o.attention_scale = scale;
    return o;
}

}  // namespace

extern "C" {

const char* ref_cuda_last_error() { return g_error.c_str(); }

int ref_cuda_rmsnorm_forward(void* y, const void* x, const void* w, std::size_t rows, std::size_t hidden, float eps, int dtype,
                             cudaStream_t s) {
    return guarded([&] {
        Tensor ty = view(y, {rows, hidden}, dtype);
        rmsnorm_forward(ty, view(x, {rows, hidden}, dtype), view(w, {hidden}, dtype), eps, s);
    });
}

int ref_cuda_rmsnorm_backward(void* dx, void* dw, const void* dy, const void* x, const void* w, std::size_t rows,
                              std::size_t hidden, float eps, int dtype, cudaStream_t s) {
    return guarded([&] {
        Tensor tdx = view(dx, {rows, hidden}, dtype), tdw = view(dw, {hidden}, dtype);
        rmsnorm_backward(tdx, tdw, view(dy, {rows, hidden}, dtype), view(x, {rows, hidden}, dtype), view(w, {hidden}, dtype), eps, s);
    });
}

int ref_cuda_rope_forward(void* q, void* k, const void* cos_t, const void* sin_t, std::size_t batch, std::size_t seq,
                          std::size_t hq, std::size_t hkv, std::size_t d, std::size_t rotary, std::size_t offset,
                          std::size_t max_seq, int dtype, cudaStream_t s) {
    return guarded([&] {
        Tensor tq = view(q, {batch, seq, hq, d}, dtype), tk = view(k, {batch, seq, hkv, d}, dtype);
        const std::size_t half = (rotary ? rotary : d) / 2;
        RopeOptions o{};
        o.rotary_dim = rotary;
        o.position_offset = offset;
        rope_forward(tq, tk, view(cos_t, {max_seq, half}, dtype), view(sin_t, {max_seq, half}, dtype), s, o);
    });
}

int ref_cuda_rope_backward(void* dq, void* dk, const void* dq_rot, const void* dk_rot, const void* cos_t, const void* sin_t,
                           std::size_t batch, std::size_t seq, std::size_t hq, std::size_t hkv, std::size_t d,
                           std::size_t rotary, std::size_t offset, std::size_t max_seq, int dtype, cudaStream_t s) {
    return guarded([&] {
        Tensor tdq = view(dq, {batch, seq, hq, d}, dtype), tdk = view(dk, {batch, seq, hkv, d}, dtype);
        const std::size_t half = (rotary ? rotary : d) / 2;
        RopeOptions o{};
        o.rotary_dim = rotary;
        o.position_offset = offset;
        rope_backward(tdq, tdk, view(dq_rot, {batch, seq, hq, d}, dtype), view(dk_rot, {batch, seq, hkv, d}, dtype),
                      view(cos_t, {max_seq, half}, dtype), view(sin_t, {max_seq, half}, dtype), s, o);
    });
}

int ref_cuda_swiglu_forward(void* y, const void* gate, const void* up, std::size_t rows, std::size_t inter, int dtype,
                            cudaStream_t s) {
    return guarded([&] {
        Tensor ty = view(y, {rows, inter}, dtype);
        swiglu_forward(ty, view(gate, {rows, inter}, dtype), view(up, {rows, inter}, dtype), s);
    });
}

int ref_cuda_swiglu_backward(void* dgate, void* dup, const void* dy, const void* gate, const void* up, std::size_t rows,
                             std::size_t inter, int dtype, cudaStream_t s) {
    return guarded([&] {
        Tensor tg = view(dgate, {rows, inter}, dtype), tu = view(dup, {rows, inter}, dtype);
        swiglu_backward(tg, tu, view(dy, {rows, inter}, dtype), view(gate, {rows, inter}, dtype), view(up, {rows, inter}, dtype), s);
    });
}

int ref_cuda_embedding_backward(void* gw, const void* dy, const std::uint32_t* ids, std::size_t tokens, std::size_t vocab,
                                std::size_t hidden, int accumulate, int dtype, cudaStream_t s) {
    return guarded([&] {
        Tensor tg = view(gw, {vocab, hidden}, dtype);
        EmbeddingBackwardOptions o{};
        o.accumulate_weight = accumulate != 0;
        embedding_backward(tg, view(dy, {tokens, hidden}, dtype), ids, tokens, s, o);
    });
}

int ref_cuda_cross_entropy(float* loss, void* grad, const void* logits, const std::uint32_t* targets, std::size_t rows,
                           std::size_t vocab, float gradient_scale, int dtype, cudaStream_t s) {
    return guarded([&] {
        Tensor tl = view(loss, {1}, 2), tg = view(grad, {rows, vocab}, dtype);
        cross_entropy_forward_backward(tl, tg, view(logits, {rows, vocab}, dtype), targets, rows, s, gradient_scale);
    });
}

int ref_cuda_cut_cross_entropy(float* loss, void* gx, void* gc, const void* x, const void* c, const std::uint32_t* targets,
                               std::size_t rows, std::size_t vocab, std::size_t hidden, int dtype, cudaStream_t s) {
    return guarded([&] {
        Tensor tl = view(loss, {1}, 2), tgx = view(gx, {rows, hidden}, dtype), tgc = view(gc, {vocab, hidden}, dtype);
        cut_cross_entropy_forward_backward(tl, tgx, tgc, view(x, {rows, hidden}, dtype), view(c, {vocab, hidden}, dtype), targets, rows, s);
    });
}

int ref_cuda_attention_forward(void* out, float* lse, const void* q, const void* k, const void* v, std::size_t batch,
                               std::size_t sq, std::size_t sk, std::size_t hq, std::size_t hkv, std::size_t d, int causal,
                               std::size_t offset, float scale, int dtype, cudaStream_t s) {
    return guarded([&] {
        Tensor to = view(out, {batch, sq, hq, d}, dtype), tl = view(lse, {batch, sq, hq}, 2);
        flash_gqa_attention_forward_with_lse(to, tl, view(q, {batch, sq, hq, d}, dtype), view(k, {batch, sk, hkv, d}, dtype),
                                             view(v, {batch, sk, hkv, d}, dtype), s, attn_options(hq, hkv, d, causal, offset, scale));
    });
}

int ref_cuda_attention_backward(void* dq, void* dk, void* dv, const void* dout, const void* out, const float* lse, const void* q,
                                const void* k, const void* v, std::size_t batch, std::size_t sq, std::size_t sk, std::size_t hq,
                                std::size_t hkv, std::size_t d, int causal, std::size_t offset, float scale, int dtype,
                                cudaStream_t s) {
    return guarded([&] {
        Tensor tdq = view(dq, {batch, sq, hq, d}, dtype), tdk = view(dk, {batch, sk, hkv, d}, dtype),
               tdv = view(dv, {batch, sk, hkv, d}, dtype);
        flash_gqa_attention_backward_with_lse(tdq, tdk, tdv, view(dout, {batch, sq, hq, d}, dtype), view(out, {batch, sq, hq, d}, dtype),
                                              view(lse, {batch, sq, hq}, 2), view(q, {batch, sq, hq, d}, dtype),
                                              view(k, {batch, sk, hkv, d}, dtype), view(v, {batch, sk, hkv, d}, dtype), s,
                                              attn_options(hq, hkv, d, causal, offset, scale), false);
    });
}

}  // extern "C"
