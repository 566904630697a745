// TEST INFRASTRUCTURE: a flat C wrapper around the reference's own CPU operators.
//
// This file is compiled together with the reference's untouched sources (src/ops/cpu/**, src/core/tensor.cu,
// src/optim/adamw.cu) by oracle/build_ref.py into oracle/_ref/libcgpt_ref_cpu.so. It contains no
// arithmetic of its own: every function builds CPU `Tensor`s from host float arrays (rounding to the
// requested storage dtype exactly as Tensor::copy_from_host does), calls one reference function and
// copies the result back as float. It exists so that the numpy oracle can be validated against the
// reference's real CPU code, and so that bench.py can time the reference's CPU forward.
//
// dtype codes follow the reference's Dtype enum (include/core/dtype.h:12-21): 0 = F16, 1 = BF16, 2 = F32.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <exception>
#include <span>
#include <string>
#include <vector>

#include "core/tensor.h"
#include "ops/attention.h"
#include "ops/backward/attention_backward.h"
#include "ops/backward/embedding_backward.h"
#include "ops/backward/linear_backward.h"
#include "ops/backward/swiglu_backward.h"
#include "ops/cpu/attention_cpu.h"
#include "ops/cpu/backward/attention_backward_cpu.h"
#include "ops/cpu/backward/cross_entropy_backward_cpu.h"
#include "ops/cpu/backward/embedding_backward_cpu.h"
#include "ops/cpu/backward/linear_backward_cpu.h"
#include "ops/cpu/backward/rmsnorm_backward_cpu.h"
#include "ops/cpu/cross_entropy_cpu.h"
#include "ops/cpu/embedding_cpu.h"
#include "ops/cpu/linear_cpu.h"
#include "ops/cpu/rmsnorm_cpu.h"
#include "ops/cpu/rope_backward_cpu.h"
#include "ops/cpu/rope_cpu.h"
#include "ops/cpu/swiglu_backward_cpu.h"
#include "ops/cpu/swiglu_cpu.h"
#include "ops/rope.h"
#include "optim/adamw.h"

namespace {

std::string g_error;

using Shape = std::vector<std::size_t>;

Tensor make(const float* src, Shape shape, int dtype) {
    Tensor t(std::move(shape), DeviceType::CPU, static_cast<Dtype>(dtype));
    if (src != nullptr) t.copy_from_host(std::span<const float>(src, t.numel()));
    return t;
}

void fetch(float* dst, const Tensor& t) { t.copy_to_host(std::span<float>(dst, t.numel())); }

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    } catch (...) {
        g_error = "unknown exception";
        return -1;
    }
}

FlashAttentionOptions attn_options(std::size_t hq, std::size_t hkv, std::size_t d, int causal, std::size_t offset,
                                   float scale) {
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

const char* ref_last_error() { return g_error.c_str(); }

int ref_rmsnorm_forward(float* y, const float* x, const float* w, std::size_t rows, std::size_t hidden, float eps,
                        int dtype) {
    return guarded([&] {
        Tensor tx = make(x, {rows, hidden}, dtype), tw = make(w, {hidden}, dtype), ty = make(nullptr, {rows, hidden}, dtype);
        rmsnorm_forward_cpu(ty, tx, tw, eps);
        fetch(y, ty);
    });
}

int ref_rmsnorm_backward(float* dx, float* dw, const float* dy, const float* x, const float* w, std::size_t rows,
                         std::size_t hidden, float eps, int dtype) {
    return guarded([&] {
        Tensor tdy = make(dy, {rows, hidden}, dtype), tx = make(x, {rows, hidden}, dtype), tw = make(w, {hidden}, dtype);
        Tensor tdx = make(nullptr, {rows, hidden}, dtype), tdw = make(nullptr, {hidden}, dtype);
        rmsnorm_backward_cpu(tdx, tdw, tdy, tx, tw, eps);
        fetch(dx, tdx);
        fetch(dw, tdw);
    });
}

int ref_rope_forward(float* q, float* k, const float* cos_t, const float* sin_t, std::size_t b, std::size_t s,
                     std::size_t hq, std::size_t hkv, std::size_t d, std::size_t rotary, std::size_t offset,
                     std::size_t max_seq, int dtype) {
    return guarded([&] {
        const std::size_t r = rotary == 0 ? d : rotary;
        Tensor tq = make(q, {b, s, hq, d}, dtype), tk = make(k, {b, s, hkv, d}, dtype);
        Tensor tc = make(cos_t, {max_seq, r / 2}, dtype), ts = make(sin_t, {max_seq, r / 2}, dtype);
        rope_forward_cpu(tq, tk, tc, ts, RopeOptions{rotary, offset});
        fetch(q, tq);
        fetch(k, tk);
    });
}

int ref_rope_backward(float* dq, float* dk, const float* dq_rot, const float* dk_rot, const float* cos_t,
                      const float* sin_t, std::size_t b, std::size_t s, std::size_t hq, std::size_t hkv, std::size_t d,
                      std::size_t rotary, std::size_t offset, std::size_t max_seq, int dtype) {
    return guarded([&] {
        const std::size_t r = rotary == 0 ? d : rotary;
        Tensor tq = make(dq_rot, {b, s, hq, d}, dtype), tk = make(dk_rot, {b, s, hkv, d}, dtype);
        Tensor oq = make(nullptr, {b, s, hq, d}, dtype), ok = make(nullptr, {b, s, hkv, d}, dtype);
        Tensor tc = make(cos_t, {max_seq, r / 2}, dtype), ts = make(sin_t, {max_seq, r / 2}, dtype);
        rope_backward_cpu(oq, ok, tq, tk, tc, ts, RopeOptions{rotary, offset});
        fetch(dq, oq);
        fetch(dk, ok);
    });
}

int ref_swiglu_forward(float* y, const float* gate, const float* up, std::size_t rows, std::size_t cols, int dtype) {
    return guarded([&] {
        Tensor tg = make(gate, {rows, cols}, dtype), tu = make(up, {rows, cols}, dtype), ty = make(nullptr, {rows, cols}, dtype);
        swiglu_forward_cpu(ty, tg, tu);
        fetch(y, ty);
    });
}

int ref_swiglu_backward(float* dgate, float* dup, const float* dy, const float* gate, const float* up, std::size_t rows,
                        std::size_t cols, int dtype) {
    return guarded([&] {
        Tensor tg = make(gate, {rows, cols}, dtype), tu = make(up, {rows, cols}, dtype), td = make(dy, {rows, cols}, dtype);
        Tensor og = make(nullptr, {rows, cols}, dtype), ou = make(nullptr, {rows, cols}, dtype);
        swiglu_backward_cpu(og, ou, td, tg, tu);
        fetch(dgate, og);
        fetch(dup, ou);
    });
}

int ref_embedding_forward(float* out, const std::uint32_t* ids, const float* weight, std::size_t tokens, std::size_t vocab,
                          std::size_t hidden, int dtype) {
    return guarded([&] {
        Tensor tw = make(weight, {vocab, hidden}, dtype), to = make(nullptr, {tokens, hidden}, dtype);
        embedding_forward_cpu(to, ids, tokens, tw);
        fetch(out, to);
    });
}

int ref_embedding_backward(float* grad_weight, const float* grad_output, const std::uint32_t* ids, std::size_t tokens,
                           std::size_t vocab, std::size_t hidden, int accumulate, int dtype) {
    return guarded([&] {
        Tensor tg = make(grad_weight, {vocab, hidden}, dtype), td = make(grad_output, {tokens, hidden}, dtype);
        EmbeddingBackwardOptions o{};
        o.accumulate_weight = accumulate != 0;
        embedding_backward_cpu(tg, td, ids, tokens, o);
        fetch(grad_weight, tg);
    });
}

int ref_linear_forward(float* y, const float* x, const float* w, std::size_t rows, std::size_t in, std::size_t out,
                       int dtype) {
    return guarded([&] {
        Tensor tx = make(x, {rows, in}, dtype), tw = make(w, {out, in}, dtype), ty = make(nullptr, {rows, out}, dtype);
        linear_forward_cpu(ty, tx, tw);
        fetch(y, ty);
    });
}

int ref_linear_backward(float* dx, float* dw, float* db, const float* dy, const float* x, const float* w,
                        std::size_t rows, std::size_t in, std::size_t out, int acc_input, int acc_weight, int acc_bias,
                        int dtype) {
    return guarded([&] {
        Tensor tdy = make(dy, {rows, out}, dtype), tx = make(x, {rows, in}, dtype), tw = make(w, {out, in}, dtype);
        Tensor tdx = make(dx, {rows, in}, dtype), tdw = make(dw, {out, in}, dtype), tdb = make(db, {out}, dtype);
        LinearBackwardOptions o{};
        o.accumulate_input = acc_input != 0;
        o.accumulate_weight = acc_weight != 0;
        o.accumulate_bias = acc_bias != 0;
        linear_backward_cpu(tdx, tdw, tdb, tdy, tx, tw, o);
        fetch(dx, tdx);
        fetch(dw, tdw);
        fetch(db, tdb);
    });
}

int ref_attention_forward_lse(float* out, float* lse, const float* q, const float* k, const float* v, std::size_t b,
                              std::size_t sq, std::size_t sk, std::size_t hq, std::size_t hkv, std::size_t d, int causal,
                              std::size_t offset, float scale, int dtype) {
    return guarded([&] {
        Tensor tq = make(q, {b, sq, hq, d}, dtype), tk = make(k, {b, sk, hkv, d}, dtype), tv = make(v, {b, sk, hkv, d}, dtype);
        Tensor to = make(nullptr, {b, sq, hq, d}, dtype), tl = make(nullptr, {b, sq, hq}, 2);
        flash_gqa_attention_forward_with_lse_cpu(to, tl, tq, tk, tv, attn_options(hq, hkv, d, causal, offset, scale));
        fetch(out, to);
        fetch(lse, tl);
    });
}

int ref_attention_backward_lse(float* dq, float* dk, float* dv, const float* dout, const float* out, const float* lse,
                               const float* q, const float* k, const float* v, std::size_t b, std::size_t sq,
                               std::size_t sk, std::size_t hq, std::size_t hkv, std::size_t d, int causal,
                               std::size_t offset, float scale, int dtype) {
    return guarded([&] {
        Tensor tq = make(q, {b, sq, hq, d}, dtype), tk = make(k, {b, sk, hkv, d}, dtype), tv = make(v, {b, sk, hkv, d}, dtype);
        Tensor tdo = make(dout, {b, sq, hq, d}, dtype), to = make(out, {b, sq, hq, d}, dtype), tl = make(lse, {b, sq, hq}, 2);
        Tensor odq = make(nullptr, {b, sq, hq, d}, dtype), odk = make(nullptr, {b, sk, hkv, d}, dtype),
               odv = make(nullptr, {b, sk, hkv, d}, dtype);
        flash_gqa_attention_backward_with_lse_cpu(odq, odk, odv, tdo, to, tl, tq, tk, tv,
                                                  attn_options(hq, hkv, d, causal, offset, scale));
        fetch(dq, odq);
        fetch(dk, odk);
        fetch(dv, odv);
    });
}

int ref_attention_backward(float* dq, float* dk, float* dv, const float* dout, const float* q, const float* k,
                           const float* v, std::size_t b, std::size_t sq, std::size_t sk, std::size_t hq,
                           std::size_t hkv, std::size_t d, int causal, std::size_t offset, float scale, int dtype) {
    return guarded([&] {
        Tensor tq = make(q, {b, sq, hq, d}, dtype), tk = make(k, {b, sk, hkv, d}, dtype), tv = make(v, {b, sk, hkv, d}, dtype);
        Tensor tdo = make(dout, {b, sq, hq, d}, dtype);
        Tensor odq = make(nullptr, {b, sq, hq, d}, dtype), odk = make(nullptr, {b, sk, hkv, d}, dtype),
               odv = make(nullptr, {b, sk, hkv, d}, dtype);
        flash_gqa_attention_backward_cpu(odq, odk, odv, tdo, tq, tk, tv, attn_options(hq, hkv, d, causal, offset, scale));
        fetch(dq, odq);
        fetch(dk, odk);
        fetch(dv, odv);
    });
}

int ref_cross_entropy(float* loss, float* grad, const float* logits, const std::uint32_t* targets, std::size_t rows,
                      std::size_t vocab, float gradient_scale, int dtype) {
    return guarded([&] {
        Tensor tl = make(logits, {rows, vocab}, dtype), tloss = make(nullptr, {1}, 2);
        if (grad != nullptr) {
            Tensor tg = make(nullptr, {rows, vocab}, dtype);
            cross_entropy_forward_backward_cpu(tloss, tg, tl, targets, rows, gradient_scale);
            fetch(grad, tg);
        } else {
            cross_entropy_forward_cpu(tloss, tl, targets, rows);
        }
        fetch(loss, tloss);
    });
}

// One adamw_step on CPU tensors (src/optim/adamw.cu:405-435, CPU branch :193-225). `step` is in/out.
// Returns 1 if the update was applied, 0 if it was skipped, -1 on exception.
int ref_adamw_step_cpu(float* param, const float* grad, float* master, float* m, float* v, std::size_t n,
                       unsigned long long* step, float lr, float beta1, float beta2, float eps, float wd,
                       float loss_scale, float max_grad_norm, int dtype) {
    int applied = 0;
    const int rc = guarded([&] {
        Tensor tp = make(param, {n}, dtype), tg = make(grad, {n}, dtype);
        AdamWState st{make(master, {n}, 2), make(m, {n}, 2), make(v, {n}, 2), *step};
        AdamWOptions o{};
        o.learning_rate = lr; o.beta1 = beta1; o.beta2 = beta2; o.epsilon = eps; o.weight_decay = wd;
        o.loss_scale = loss_scale; o.max_grad_norm = max_grad_norm;
        applied = adamw_step(tp, tg, st, o) ? 1 : 0;
        fetch(param, tp);
        fetch(master, st.master_parameter);
        fetch(m, st.first_moment);
        fetch(v, st.second_moment);
        *step = st.step;
    });
    return rc != 0 ? -1 : applied;
}

// Reference CPU forward + cross-entropy loss of the whole model on fp32 CPU tensors, composed from the
// public CPU operators in the order of src/core/generation_cpu.cpp:323-379 (that function has internal
// linkage), with the block structure of src/core/transformer_block.cu:466-595. Weights are passed as one
// flat fp32 array laid out as: token_embedding [V,d], then per layer {attention_norm[d], q[Hq*D,d],
// k[Hkv*D,d], q_norm[D], k_norm[D], v[Hkv*D,d], o[d,Hq*D], ffn_norm[d], gate[I,d], up[I,d], down[d,I]},
// then final_norm [d]; the LM head is tied to the embedding. Returns the wall-clock seconds of the
// forward+loss (median of `repeats`), writes the loss to *loss_out; negative on error.
double ref_cpu_forward_loss(float* loss_out, const float* weights, const std::uint32_t* ids,
                            const std::uint32_t* targets, std::size_t batch, std::size_t seq, std::size_t layers,
                            std::size_t d, std::size_t hq, std::size_t hkv, std::size_t hd, std::size_t inter,
                            std::size_t vocab, float eps, int repeats) {
    double result = -1.0;
    guarded([&] {
        const std::size_t rows = batch * seq;
        const float* p = weights;
        auto take = [&](Shape shape) {
            Tensor t(shape, DeviceType::CPU, Dtype::F32);
            t.copy_from_host(std::span<const float>(p, t.numel()));
            p += t.numel();
            return t;
        };
        struct Layer { Tensor an, q, k, qn, kn, v, o, fn, gate, up, down; };
        Tensor embedding = take({vocab, d});
        std::vector<Layer> lw;
        for (std::size_t l = 0; l < layers; ++l) {
            lw.push_back(Layer{take({d}), take({hq * hd, d}), take({hkv * hd, d}), take({hd}), take({hd}),
                               take({hkv * hd, d}), take({d, hq * hd}), take({d}), take({inter, d}), take({inter, d}),
                               take({d, inter})});
        }
        Tensor final_norm = take({d});
        std::vector<float> cosv(seq * hd / 2), sinv(seq * hd / 2);
        for (std::size_t pos = 0; pos < seq; ++pos)
            for (std::size_t i = 0; i < hd / 2; ++i) {
                const float theta = static_cast<float>(pos) /
                                    std::pow(10000.0F, 2.0F * static_cast<float>(i) / static_cast<float>(hd));
                cosv[pos * (hd / 2) + i] = std::cos(theta);
                sinv[pos * (hd / 2) + i] = std::sin(theta);
            }
        Tensor cos_cache = make(cosv.data(), {seq, hd / 2}, 2), sin_cache = make(sinv.data(), {seq, hd / 2}, 2);

        std::vector<double> times;
        for (int rep = 0; rep < (repeats < 1 ? 1 : repeats); ++rep) {
            const auto t0 = std::chrono::steady_clock::now();
            Tensor hidden({rows, d}, DeviceType::CPU, Dtype::F32), norm({rows, d}, DeviceType::CPU, Dtype::F32);
            embedding_forward_cpu(hidden, ids, rows, embedding);
            for (std::size_t l = 0; l < layers; ++l) {
                const Layer& w = lw[l];
                Tensor q({rows, hq * hd}, DeviceType::CPU, Dtype::F32), k({rows, hkv * hd}, DeviceType::CPU, Dtype::F32),
                    v({rows, hkv * hd}, DeviceType::CPU, Dtype::F32);
                rmsnorm_forward_cpu(norm, hidden, w.an, eps);
                linear_forward_cpu(q, norm, w.q);
                linear_forward_cpu(k, norm, w.k);
                linear_forward_cpu(v, norm, w.v);
                q.reshape({rows * hq, hd});
                k.reshape({rows * hkv, hd});
                Tensor qn({rows * hq, hd}, DeviceType::CPU, Dtype::F32), kn({rows * hkv, hd}, DeviceType::CPU, Dtype::F32);
                rmsnorm_forward_cpu(qn, q, w.qn, eps);
                rmsnorm_forward_cpu(kn, k, w.kn, eps);
                qn.reshape({batch, seq, hq, hd});
                kn.reshape({batch, seq, hkv, hd});
                v.reshape({batch, seq, hkv, hd});
                rope_forward_cpu(qn, kn, cos_cache, sin_cache, RopeOptions{hd, 0});
                Tensor attn({batch, seq, hq, hd}, DeviceType::CPU, Dtype::F32), lse({batch, seq, hq}, DeviceType::CPU, Dtype::F32);
                flash_gqa_attention_forward_with_lse_cpu(attn, lse, qn, kn, v, attn_options(hq, hkv, hd, 1, 0, 0.0F));
                attn.reshape({rows, hq * hd});
                Tensor proj({rows, d}, DeviceType::CPU, Dtype::F32);
                linear_forward_cpu(proj, attn, w.o);
                rmsnorm_forward_cpu(norm, hidden, w.fn, eps);
                Tensor gate({rows, inter}, DeviceType::CPU, Dtype::F32), up({rows, inter}, DeviceType::CPU, Dtype::F32),
                    act({rows, inter}, DeviceType::CPU, Dtype::F32), ffn({rows, d}, DeviceType::CPU, Dtype::F32);
                linear_forward_cpu(gate, norm, w.gate);
                linear_forward_cpu(up, norm, w.up);
                swiglu_forward_cpu(act, gate, up);
                linear_forward_cpu(ffn, act, w.down);
                float* h = hidden.data();
                const float* a = proj.data();
                const float* f = ffn.data();
                for (std::size_t i = 0; i < rows * d; ++i) h[i] = (h[i] + a[i]) + f[i];
            }
            rmsnorm_forward_cpu(norm, hidden, final_norm, eps);
            Tensor logits({rows, vocab}, DeviceType::CPU, Dtype::F32), loss({1}, DeviceType::CPU, Dtype::F32);
            linear_forward_cpu(logits, norm, embedding);
            cross_entropy_forward_cpu(loss, logits, targets, rows);
            const auto t1 = std::chrono::steady_clock::now();
            times.push_back(std::chrono::duration<double>(t1 - t0).count());
            *loss_out = loss.data()[0];
        }
        std::sort(times.begin(), times.end());
        result = times[times.size() / 2];
    });
    return result;
}

}  // extern "C"
