// TEST INFRASTRUCTURE: a flat C wrapper around the reference's own transformer block / model / optimizer CUDA code.
//
// Compiled by oracle/build_ref.py together with the reference's untouched sources (src/core/transformer_block.cu,
// src/core/transformer_model.cu, src/ops/backward/linear_backward.cu, src/optim/adamw.cu, src/core/cuda_graph.cu, the
// forward and backward operators and a build-time copy of src/ops/linear.cu) into oracle/_ref/libcgpt_ref_cuda.so for
// sm_100a. It contains no arithmetic of its own. It owns the tensors the reference's trainer owns
// (train/train.cpp:251-300 ModelStorage with tied embedding, :427-457 workspaces, logits, optimizer state) and runs the
// trainer's step (train/train.cpp:536-556): transformer_model_forward -> cross_entropy_forward_backward ->
// transformer_model_backward, then adamw_step_many_async; optionally captured into the reference's CudaGraph as the
// trainer does (:545-548). The GPU parity tests feed the same weights and token ids to this and to the library and
// compare gradients, updated weights and losses; bench.py times it as an informational baseline.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <exception>
#include <memory>
#include <string>
#include <vector>

#include "core/cuda_graph.h"
#include "core/tensor.h"
#include "core/transformer_block.h"
#include "core/transformer_model.h"
#include "core/weight_initialization.h"
#include "ops/backward/linear_backward.h"
#include "ops/cross_entropy.h"
#include "optim/adamw.h"

namespace {

std::string g_error;

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

constexpr int kBlockTensors = 11;
const char* const kBlockNames[kBlockTensors] = {"attention_norm", "q_projection", "k_projection", "q_norm", "k_norm", "v_projection",
                                                "o_projection",   "ffn_norm",     "gate_proj",    "up_proj", "down_proj"};

std::vector<std::vector<std::size_t>> block_shapes(const TransformerBlockOptions& o) {
    const std::size_t kv = o.num_kv_heads * o.head_dim, qd = o.num_query_heads * o.head_dim;
    return {{o.hidden_size},      {qd, o.hidden_size}, {kv, o.hidden_size},
            {o.head_dim},         {o.head_dim},        {kv, o.hidden_size},
            {o.hidden_size, qd},  {o.hidden_size},     {o.intermediate_size, o.hidden_size},
            {o.intermediate_size, o.hidden_size},      {o.hidden_size, o.intermediate_size}};
}

// The eleven tensors of a block, as weights and as gradients (the trainer's LayerStorage, train/train.cpp:251-272).
struct Layer {
    std::vector<Tensor> w, g;
    Layer(const TransformerBlockOptions& o, Dtype dt) {
        for (const auto& s : block_shapes(o)) {
            w.emplace_back(s, dt);
            g.emplace_back(s, dt);
        }
    }
    TransformerBlockWeights weights() const { return {w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7], w[8], w[9], w[10]}; }
    MutableTransformerBlockWeights mutable_weights() { return {w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7], w[8], w[9], w[10]}; }
    TransformerBlockGradients gradients() { return {g[0], g[1], g[2], g[3], g[4], g[5], g[6], g[7], g[8], g[9], g[10]}; }
};

struct Model {
    TransformerModelOptions options;
    std::size_t batch, seq;
    Tensor embedding, final_norm, g_embedding, g_final_norm;
    std::vector<std::unique_ptr<Layer>> layers;
    std::vector<TransformerBlockWeights> weight_layers;
    std::vector<MutableTransformerBlockWeights> mutable_layers;
    std::vector<TransformerBlockGradients> gradient_layers;
    Tensor cos_cache, sin_cache;
    TransformerModelWorkspace forward_ws;
    TransformerModelBackwardWorkspace backward_ws;
    Tensor logits, grad_logits, loss;
    std::vector<std::pair<Tensor*, Tensor*>> parameters;   // trainer's order, train/train.cpp:302-320
    std::vector<std::string> names;
    std::vector<AdamWState> optimizer;
    std::vector<AdamWBatchEntry> entries;
    std::unique_ptr<AdamWWorkspace> optimizer_ws;
    CublasLtContext cublas;
    CudaGraph graph;
    const std::uint32_t* captured_ids = nullptr;
    const std::uint32_t* captured_targets = nullptr;
    float captured_scale = 0.f;

    Model(const TransformerModelOptions& o, std::size_t b, std::size_t s)
        : options(o), batch(b), seq(s),
          embedding({o.vocabulary_size, o.block_options.hidden_size}, Dtype::F16), final_norm({o.block_options.hidden_size}, Dtype::F16),
          g_embedding({o.vocabulary_size, o.block_options.hidden_size}, Dtype::F16), g_final_norm({o.block_options.hidden_size}, Dtype::F16),
          cos_cache({s, o.block_options.rotary_dim / 2}, Dtype::F16), sin_cache({s, o.block_options.rotary_dim / 2}, Dtype::F16),
          forward_ws(o, b, s, Dtype::F16), backward_ws(o, b, s, Dtype::F16),
          logits({b * s, o.vocabulary_size}, Dtype::F16), grad_logits({b * s, o.vocabulary_size}, Dtype::F16), loss({1}, Dtype::F32) {
        for (std::size_t i = 0; i < o.num_layers; ++i) layers.push_back(std::make_unique<Layer>(o.block_options, Dtype::F16));
        for (auto& l : layers) {
            weight_layers.push_back(l->weights());
            mutable_layers.push_back(l->mutable_weights());
            gradient_layers.push_back(l->gradients());
        }
        parameters.emplace_back(&embedding, &g_embedding);
        names.emplace_back("token_embedding");
        parameters.emplace_back(&final_norm, &g_final_norm);
        names.emplace_back("final_norm");
        for (std::size_t li = 0; li < layers.size(); ++li)
            for (int t = 0; t < kBlockTensors; ++t) {
                parameters.emplace_back(&layers[li]->w[t], &layers[li]->g[t]);
                names.push_back("layers." + std::to_string(li) + "." + kBlockNames[t]);
            }
    }
    TransformerModelWeights weights() const { return {embedding, weight_layers, final_norm, embedding}; }
    TransformerModelGradients gradients() { return {g_embedding, gradient_layers, g_final_norm, g_embedding}; }

    // Fresh optimizer state from the current weights (AdamWState::for_parameter copies the parameter into the fp32 master).
    void reset_optimizer() {
        optimizer.clear();
        entries.clear();
        for (auto& [p, g] : parameters) optimizer.push_back(AdamWState::for_parameter(*p));
        for (std::size_t i = 0; i < parameters.size(); ++i) entries.push_back({parameters[i].first, parameters[i].second, &optimizer[i]});
        optimizer_ws = std::make_unique<AdamWWorkspace>();
    }

    void enqueue_model_step(const std::uint32_t* ids, const std::uint32_t* targets, float loss_scale, cudaStream_t stream) {
        transformer_model_forward(logits, ids, batch, seq, weights(), forward_ws, cos_cache, sin_cache, cublas, stream, options);
        cross_entropy_forward_backward(loss, grad_logits, logits, targets, batch * seq, stream, loss_scale);
        transformer_model_backward(grad_logits, ids, batch, seq, weights(), gradients(), forward_ws, backward_ws, cos_cache, sin_cache,
                                   cublas, stream, options);
    }
};

Model* M(void* h) { return static_cast<Model*>(h); }

AdamWOptions adamw_options(float lr, float b1, float b2, float eps, float wd, float loss_scale, float max_norm) {
    AdamWOptions o;
    o.learning_rate = lr;
    o.beta1 = b1;
    o.beta2 = b2;
    o.epsilon = eps;
    o.weight_decay = wd;
    o.loss_scale = loss_scale;
    o.max_grad_norm = max_norm;
    return o;
}

}  // namespace

extern "C" {

const char* ref_model_last_error() { return g_error.c_str(); }

// Allocates the trainer's tensors for a tied-embedding fp16 model and a fixed (batch, seq); cos/sin are copied from the
// caller's fp16 device tables [seq, rotary/2]. Weights are uninitialised until ref_model_init or ref_model_set_param.
void* ref_model_create(std::size_t vocab, std::size_t num_layers, std::size_t hidden, std::size_t intermediate, std::size_t hq,
                       std::size_t hkv, std::size_t head_dim, std::size_t rotary, float eps, std::size_t batch, std::size_t seq,
                       const void* cos_table, const void* sin_table) {
    Model* m = nullptr;
    const int rc = guarded([&] {
        TransformerModelOptions o;
        o.vocabulary_size = vocab;
        o.num_layers = num_layers;
        o.block_options.hidden_size = hidden;
        o.block_options.intermediate_size = intermediate;
        o.block_options.num_query_heads = hq;
        o.block_options.num_kv_heads = hkv;
        o.block_options.head_dim = head_dim;
        o.block_options.rotary_dim = rotary;
        o.block_options.rms_epsilon = eps;
        m = new Model(o, batch, seq);
        CUDA_CHECK(cudaMemcpy(m->cos_cache.raw_data(), cos_table, m->cos_cache.nbytes(), cudaMemcpyDeviceToDevice));
        CUDA_CHECK(cudaMemcpy(m->sin_cache.raw_data(), sin_table, m->sin_cache.nbytes(), cudaMemcpyDeviceToDevice));
        m->reset_optimizer();
    });
    if (rc != 0) {
        delete m;
        return nullptr;
    }
    return m;
}

void ref_model_destroy(void* h) { delete M(h); }

// The reference's own seeded initialisation (src/core/weight_initialization.cu:122-181), then fresh optimizer state.
int ref_model_init(void* h, std::uint64_t seed) {
    return guarded([&] {
        WeightInitializationOptions init;
        init.seed = seed;
        initialize_transformer_weights({M(h)->embedding, M(h)->mutable_layers, M(h)->final_norm, M(h)->embedding}, M(h)->options, init);
        M(h)->reset_optimizer();
    });
}

int ref_model_num_params(void* h) { return static_cast<int>(M(h)->parameters.size()); }

// Name (copied into `name`, at most `cap` bytes), element count and device pointers of parameter i and its gradient.
int ref_model_param(void* h, int i, char* name, std::size_t cap, std::size_t* numel, void** param, void** grad) {
    return guarded([&] {
        auto& [p, g] = M(h)->parameters.at(static_cast<std::size_t>(i));
        if (name != nullptr && cap > 0) std::snprintf(name, cap, "%s", M(h)->names[static_cast<std::size_t>(i)].c_str());
        if (numel != nullptr) *numel = p->numel();
        if (param != nullptr) *param = p->raw_data();
        if (grad != nullptr) *grad = g->raw_data();
    });
}

// After weights were written through the pointers of ref_model_param: optimizer state restarts from them.
int ref_model_reset_optimizer(void* h) {
    return guarded([&] { M(h)->reset_optimizer(); });
}

// fp32 master / first moment / second moment device pointers of parameter i (for comparing optimizer state).
int ref_model_state(void* h, int i, void** master, void** m1, void** m2) {
    return guarded([&] {
        AdamWState& s = M(h)->optimizer.at(static_cast<std::size_t>(i));
        *master = s.master_parameter.raw_data();
        *m1 = s.first_moment.raw_data();
        *m2 = s.second_moment.raw_data();
    });
}

// forward + cross-entropy (gradient_scale = loss_scale) + backward, eagerly on `stream` (train/train.cpp:536-544).
int ref_model_step(void* h, const std::uint32_t* ids, const std::uint32_t* targets, float loss_scale, cudaStream_t stream) {
    return guarded([&] { M(h)->enqueue_model_step(ids, targets, loss_scale, stream); });
}

// The same step replayed from the reference's CudaGraph; captured on first use for (ids, targets, loss_scale) after one
// eager run, as the trainer does (train/train.cpp:545-548). `stream` must be a non-default stream.
int ref_model_step_graph(void* h, const std::uint32_t* ids, const std::uint32_t* targets, float loss_scale, cudaStream_t stream) {
    return guarded([&] {
        Model* m = M(h);
        if (!m->graph.initialized() || m->captured_ids != ids || m->captured_targets != targets || m->captured_scale != loss_scale) {
            m->enqueue_model_step(ids, targets, loss_scale, stream);
            CUDA_CHECK(cudaStreamSynchronize(stream));
            m->graph.capture(stream, [&] { m->enqueue_model_step(ids, targets, loss_scale, stream); });
            m->graph.upload(stream);
            m->captured_ids = ids;
            m->captured_targets = targets;
            m->captured_scale = loss_scale;
        }
        m->graph.launch(stream);
    });
}

// adamw_step_many_async over all parameters in the trainer's order (train/train.cpp:554-556).
int ref_model_adamw(void* h, float lr, float b1, float b2, float eps, float wd, float loss_scale, float max_norm, cudaStream_t stream) {
    return guarded([&] {
        adamw_step_many_async(M(h)->entries, adamw_options(lr, b1, b2, eps, wd, loss_scale, max_norm), *M(h)->optimizer_ws, stream);
    });
}

// adamw_check: synchronises, *ok = every step since the last check had finite gradients, *step = host step counter.
int ref_model_check(void* h, int* ok, std::uint64_t* step, cudaStream_t stream) {
    return guarded([&] {
        *ok = adamw_check(*M(h)->optimizer_ws, stream) ? 1 : 0;
        *step = M(h)->optimizer.empty() ? 0 : M(h)->optimizer[0].step;
    });
}

int ref_model_loss(void* h, float* out, cudaStream_t stream) {
    return guarded([&] {
        CUDA_CHECK(cudaStreamSynchronize(stream));
        CUDA_CHECK(cudaMemcpy(out, M(h)->loss.raw_data(), sizeof(float), cudaMemcpyDeviceToHost));
    });
}

// Device pointers of the fp16 logits [batch*seq, vocab] and of their gradient written by the last step.
int ref_model_logits(void* h, void** logits, void** grad_logits) {
    return guarded([&] {
        *logits = M(h)->logits.raw_data();
        *grad_logits = M(h)->grad_logits.raw_data();
    });
}

// One transformer block through the reference: transformer_block_forward into fresh workspaces (it produces the saved
// activations the backward needs), then transformer_block_backward (src/core/transformer_block.cu:405-748). weights and
// grads are arrays of the eleven device pointers in the order of TransformerBlockWeights; fp16. Allocates and frees its
// workspaces; synchronises `stream` before returning.
int ref_block_forward_backward(void* out, void* grad_input, const void* grad_output, const void* input, void* const* weights,
                               void* const* grads, const void* cos_table, const void* sin_table, std::size_t batch, std::size_t seq,
                               std::size_t hidden, std::size_t intermediate, std::size_t hq, std::size_t hkv, std::size_t head_dim,
                               std::size_t rotary, float eps, cudaStream_t stream) {
    return guarded([&] {
        TransformerModelOptions mo;
        mo.vocabulary_size = 8;
        mo.num_layers = 1;
        TransformerBlockOptions& o = mo.block_options;
        o.hidden_size = hidden;
        o.intermediate_size = intermediate;
        o.num_query_heads = hq;
        o.num_kv_heads = hkv;
        o.head_dim = head_dim;
        o.rotary_dim = rotary;
        o.rms_epsilon = eps;
        const auto shapes = block_shapes(o);
        std::vector<Tensor> w, g;
        for (int t = 0; t < kBlockTensors; ++t) {
            w.push_back(Tensor::device_view(shapes[static_cast<std::size_t>(t)], weights[t], Dtype::F16));
            g.push_back(Tensor::device_view(shapes[static_cast<std::size_t>(t)], grads[t], Dtype::F16));
        }
        const TransformerBlockWeights bw{w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7], w[8], w[9], w[10]};
        const TransformerBlockGradients bg{g[0], g[1], g[2], g[3], g[4], g[5], g[6], g[7], g[8], g[9], g[10]};
        TransformerModelWorkspace fws(mo, batch, seq, Dtype::F16);   // its layers[0] is a block forward workspace of the right shapes
        TransformerBlockBackwardWorkspace bws(o, batch, seq, Dtype::F16);
        const std::size_t rows = batch * seq;
        const Tensor x = Tensor::device_view({rows, hidden}, const_cast<void*>(input), Dtype::F16);
        const Tensor dy = Tensor::device_view({rows, hidden}, const_cast<void*>(grad_output), Dtype::F16);
        Tensor y = Tensor::device_view({rows, hidden}, out, Dtype::F16);
        Tensor dx = Tensor::device_view({rows, hidden}, grad_input, Dtype::F16);
        const Tensor cosv = Tensor::device_view({seq, rotary / 2}, const_cast<void*>(cos_table), Dtype::F16);
        const Tensor sinv = Tensor::device_view({seq, rotary / 2}, const_cast<void*>(sin_table), Dtype::F16);
        const CublasLtContext cublas;
        transformer_block_forward(y, x, bw, fws.layers.at(0), cosv, sinv, cublas, stream, o);
        transformer_block_backward(dx, dy, x, bw, bg, fws.layers.at(0), bws, cosv, sinv, cublas, stream, o);
        CUDA_CHECK(cudaStreamSynchronize(stream));
    });
}

// linear_backward of the reference (two cuBLASLt products + the bias reduction, src/ops/backward/linear_backward.cu:268-285).
int ref_cuda_linear_backward(void* dx, void* dw, void* db, const void* dy, const void* x, const void* w, std::size_t rows,
                             std::size_t in_features, std::size_t out_features, int acc_input, int acc_weight, int acc_bias, int dtype,
                             cudaStream_t stream) {
    return guarded([&] {
        const Dtype dt = static_cast<Dtype>(dtype);
        Tensor tdx = Tensor::device_view({rows, in_features}, dx, dt), tdw = Tensor::device_view({out_features, in_features}, dw, dt),
               tdb = Tensor::device_view({out_features}, db, dt);
        LinearBackwardOptions o;
        o.accumulate_input = acc_input != 0;
        o.accumulate_weight = acc_weight != 0;
        o.accumulate_bias = acc_bias != 0;
        const CublasLtContext cublas;
        linear_backward(tdx, tdw, tdb, Tensor::device_view({rows, out_features}, const_cast<void*>(dy), dt),
                        Tensor::device_view({rows, in_features}, const_cast<void*>(x), dt),
                        Tensor::device_view({out_features, in_features}, const_cast<void*>(w), dt), cublas, stream, o);
        CUDA_CHECK(cudaStreamSynchronize(stream));
    });
}

}  // extern "C"
