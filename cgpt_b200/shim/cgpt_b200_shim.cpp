// cgpt_b200_shim.cpp -- CGPT's own C++ entry points for the training hot path, defined on top of the C ABI of
// libcgpt_b200.so (include/cgpt_b200.h).
//
// This translation unit is compiled against CGPT's UNMODIFIED public headers (its include/ directory) and takes the
// place of these source files of CGPT's `cgpt_core` library (CMakeLists.txt:36-56):
//     src/ops/backward/attention_backward.cu  src/ops/backward/linear_backward.cu  src/ops/backward/rmsnorm_backward.cu
//     src/ops/backward/rope_backward.cu       src/ops/backward/swiglu_backward.cu  src/ops/backward/embedding_backward.cu
//     src/ops/cross_entropy.cu                src/ops/cut_cross_entropy.cu         src/optim/adamw.cu
//     src/core/transformer_block.cu           src/core/transformer_model.cu
// Every symbol those files export through the headers is defined here with the same signature, the same argument
// meaning and the same exception types (std::invalid_argument for bad arguments, std::runtime_error for a workspace of
// the wrong shape; CUDA failures print and exit like CUDA_CHECK). Callers -- train/train.cpp and the tests under tests/ --
// compile and link unchanged. All other CGPT sources (Tensor, the forward operators used on their own, KV cache,
// generation, the CPU operators, the tokenizer ...) stay CGPT's.
//
// Nothing here computes on the GPU itself: each function validates like its counterpart, unpacks Tensor objects into
// raw device pointers and sizes and calls one or a few C-ABI entry points on the caller's stream. The only arithmetic in
// this file is the host loop of adamw_step for CPU tensors, which CGPT's adamw_step offers and tests
// (src/optim/adamw.cu:193-225, tests/adamw_test.cu:97-105).
#include <cuda_runtime.h>

#include <climits>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <optional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "cgpt_b200.h"

#include "core/cuda_check.h"
#include "core/tensor.h"
#include "core/transformer_block.h"
#include "core/transformer_model.h"
#include "ops/backward/attention_backward.h"
#include "ops/backward/embedding_backward.h"
#include "ops/backward/linear_backward.h"
#include "ops/backward/rmsnorm_backward.h"
#include "ops/backward/rope_backward.h"
#include "ops/backward/swiglu_backward.h"
#include "ops/cross_entropy.h"
#include "ops/cut_cross_entropy.h"
#include "ops/embedding.h"
#include "ops/linear.h"
#include "ops/rmsnorm.h"
#include "optim/adamw.h"

namespace {

using Shape = std::vector<std::size_t>;

// Dtype codes are the same on both sides (include/core/dtype.h:12-21: F16 = 0, BF16 = 1, F32 = 2).
int code(Dtype d) { return static_cast<int>(d); }

// Status of a C-ABI call -> CGPT's error conventions (include/core/cuda_check.h:19-50): an argument error class
// becomes std::invalid_argument, a CUDA error is printed and ends the process.
void check(int rc, const char* what) {
    if (rc == CGPT_OK) return;
    if (rc > 0) throw std::invalid_argument(std::string(what) + ": rejected by cgpt_b200 (argument error class " + std::to_string(rc) + ")");
    std::fprintf(stderr, "%s: CUDA error %d (%s)\n", what, -rc, cudaGetErrorString(static_cast<cudaError_t>(-rc)));
    std::exit(EXIT_FAILURE);
}

void require(bool ok, const char* message) {
    if (!ok) throw std::invalid_argument(message);
}

bool cuda_float(const Tensor& t) { return t.device_type() == DeviceType::CUDA && is_floating_point(t.dtype()); }

bool same_cuda_dtype(std::initializer_list<const Tensor*> tensors) {
    const Tensor* first = *tensors.begin();
    for (const Tensor* t : tensors)
        if (t->device_type() != DeviceType::CUDA || t->dtype() != first->dtype()) return false;
    return is_floating_point(first->dtype());
}

void* ptr(const Tensor& t) { return const_cast<void*>(t.raw_data()); }

// ---------------------------------------------------------------------------------------------------------------------
// Scratch for the entry points whose CGPT signature has no workspace argument (transformer_block_forward and
// transformer_model_forward): one grow-only device buffer per device, sized by cgpt_block_workspace_bytes. It grows
// with cudaMalloc, so the first call with a given shape must happen outside stream capture -- CGPT's trainer runs the
// step once eagerly before it captures (train/train.cpp:545-548).
struct ForwardScratch {
    void* data = nullptr;
    std::size_t bytes = 0;
};

void* forward_scratch(std::size_t bytes) {
    static std::mutex mutex;
    static std::unordered_map<int, ForwardScratch> per_device;
    int device = 0;
    CUDA_CHECK(cudaGetDevice(&device));
    std::lock_guard<std::mutex> lock(mutex);
    ForwardScratch& s = per_device[device];
    if (s.bytes < bytes) {
        if (s.data != nullptr) {
            CUDA_CHECK(cudaDeviceSynchronize());
            CUDA_CHECK(cudaFree(s.data));
        }
        CUDA_CHECK(cudaMalloc(&s.data, bytes));
        s.bytes = bytes;
    }
    return s.data;
}

void validate_block_options(const TransformerBlockOptions& o) {
    require(o.hidden_size != 0 && o.intermediate_size != 0 && o.num_query_heads != 0 && o.num_kv_heads != 0 && o.head_dim != 0,
            "transformer block dimensions must be non-zero");
}

void validate_model_options(const TransformerModelOptions& options) {
    const TransformerBlockOptions& b = options.block_options;
    require(options.vocabulary_size != 0 && options.num_layers != 0 && b.hidden_size != 0 && b.intermediate_size != 0 &&
                b.num_query_heads != 0 && b.num_kv_heads != 0 && b.head_dim != 0,
            "transformer model dimensions must be non-zero");
    require(b.num_query_heads * b.head_dim == b.hidden_size, "transformer model query heads times head_dim must equal hidden_size");
    require(b.num_kv_heads <= b.num_query_heads && b.num_query_heads % b.num_kv_heads == 0,
            "transformer model has an invalid GQA head configuration");
}

cgpt_model_config make_config(const TransformerBlockOptions& o, Dtype dtype, std::size_t max_seq, std::size_t vocab = 1,
                              std::size_t layers = 1, bool tied = false) {
    cgpt_model_config c{};
    c.vocab = vocab;
    c.layers = layers;
    c.hidden = o.hidden_size;
    c.intermediate = o.intermediate_size;
    c.q_heads = o.num_query_heads;
    c.kv_heads = o.num_kv_heads;
    c.head_dim = o.head_dim;
    c.rotary_dim = o.rotary_dim != 0 ? o.rotary_dim : o.head_dim;
    c.max_seq = max_seq;
    c.rms_epsilon = o.rms_epsilon;
    c.dtype = code(dtype);
    c.tied_embeddings = tied ? 1 : 0;
    return c;
}

cgpt_block_params params_of(const TransformerBlockWeights& w) {
    return {ptr(w.attention_norm), ptr(w.q_projection), ptr(w.k_projection), ptr(w.q_norm), ptr(w.k_norm), ptr(w.v_projection),
            ptr(w.o_projection),   ptr(w.ffn_norm),     ptr(w.gate_proj),    ptr(w.up_proj), ptr(w.down_proj)};
}

cgpt_block_params params_of(const TransformerBlockGradients& g) {
    return {ptr(g.attention_norm), ptr(g.q_projection), ptr(g.k_projection), ptr(g.q_norm), ptr(g.k_norm), ptr(g.v_projection),
            ptr(g.o_projection),   ptr(g.ffn_norm),     ptr(g.gate_proj),    ptr(g.up_proj), ptr(g.down_proj)};
}

// The saved activations are CGPT's TransformerBlockWorkspace members one to one. CGPT has no buffer for the attention
// norm's output (its backward recomputes it, transformer_block.cu:725), so that pointer stays NULL and the library
// recomputes it too.
cgpt_block_saved saved_of(const TransformerBlockWorkspace& w) {
    cgpt_block_saved s{};
    s.norm = ptr(w.norm);
    s.query = ptr(w.query);
    s.key = ptr(w.key);
    s.value = ptr(w.value);
    s.query_pre_norm = ptr(w.query_pre_norm);
    s.key_pre_norm = ptr(w.key_pre_norm);
    s.attention_output = ptr(w.attention_output);
    s.attention_logsumexp = static_cast<float*>(ptr(w.attention_logsumexp));
    s.gate = ptr(w.gate);
    s.up = ptr(w.up);
    s.activated = ptr(w.activated);
    s.attention_norm_output = nullptr;
    return s;
}

void require_shape(const Tensor& t, const Shape& shape, const char* name) {
    if (t.shape() != shape) throw std::runtime_error(std::string(name) + ": tensor shape mismatch");
}

// The model-level backward workspace constructor sets this while it builds its per-layer block workspaces: layer 0
// gets the real scratch buffer, the others a token allocation, because one buffer serves every layer in turn.
thread_local bool g_block_workspace_token_only = false;

}  // namespace

// =====================================================================================================================
// Backward operators
// =====================================================================================================================

void rmsnorm_backward(Tensor& grad_input, Tensor& grad_weight, const Tensor& grad_output, const Tensor& input, const Tensor& weight,
                      float epsilon, cudaStream_t stream) {
    require(std::isfinite(epsilon) && epsilon > 0.0F, "rmsnorm_backward: epsilon must be finite and positive");
    require(same_cuda_dtype({&input, &grad_output, &weight, &grad_input, &grad_weight}),
            "rmsnorm_backward: all tensors must be CUDA tensors of one floating dtype");
    require(input.dim() == 2 && grad_output.shape() == input.shape() && grad_input.shape() == input.shape() && weight.dim() == 1 &&
                weight.size(0) == input.size(1) && grad_weight.shape() == weight.shape() && input.numel() != 0,
            "rmsnorm_backward: incompatible tensor shapes");
    check(cgpt_rmsnorm_backward(ptr(grad_input), ptr(grad_weight), ptr(grad_output), ptr(input), ptr(weight), nullptr, nullptr,
                                input.size(0), input.size(1), epsilon, code(input.dtype()), stream),
          "rmsnorm_backward");
}

void rope_backward(Tensor& grad_query, Tensor& grad_key, const Tensor& grad_rotated_query, const Tensor& grad_rotated_key,
                   const Tensor& cos_cache, const Tensor& sin_cache, cudaStream_t stream, const RopeOptions& o) {
    require(same_cuda_dtype({&grad_query, &grad_key, &grad_rotated_query, &grad_rotated_key, &cos_cache, &sin_cache}),
            "RoPE backward: all tensors must be CUDA tensors with the same dtype");
    require(grad_query.dim() == 4 && grad_key.dim() == 4 && grad_rotated_query.shape() == grad_query.shape() &&
                grad_rotated_key.shape() == grad_key.shape() && grad_query.size(0) == grad_key.size(0) &&
                grad_query.size(1) == grad_key.size(1) && grad_query.size(3) == grad_key.size(3),
            "RoPE backward: incompatible Q/K gradient shapes");
    const std::size_t head_dim = grad_query.size(3);
    const std::size_t rotary = o.rotary_dim != 0 ? o.rotary_dim : head_dim;
    require(rotary <= head_dim && rotary % 2 == 0 && cos_cache.dim() == 2 && sin_cache.shape() == cos_cache.shape() &&
                cos_cache.size(1) == rotary / 2,
            "RoPE backward: rotary_dim must be even, at most head_dim, and match the cache width");
    require(o.position_offset + grad_query.size(1) <= cos_cache.size(0), "RoPE backward: cache does not cover the requested rotary positions");
    check(cgpt_rope_backward(ptr(grad_query), ptr(grad_key), ptr(grad_rotated_query), ptr(grad_rotated_key), ptr(cos_cache),
                             ptr(sin_cache), grad_query.size(0), grad_query.size(1), grad_query.size(2), grad_key.size(2), head_dim,
                             rotary, o.position_offset, cos_cache.size(0), code(grad_query.dtype()), stream),
          "rope_backward");
}

void swiglu_backward(Tensor& grad_gate, Tensor& grad_up, const Tensor& grad_output, const Tensor& gate, const Tensor& up,
                     cudaStream_t stream, const SwiGLUBackwardOptions& o) {
    require(same_cuda_dtype({&grad_gate, &grad_up, &grad_output, &gate, &up}),
            "swiglu_backward: all tensors must be CUDA tensors of one floating dtype");
    require(gate.numel() != 0 && up.shape() == gate.shape() && grad_output.shape() == gate.shape() && grad_gate.shape() == gate.shape() &&
                grad_up.shape() == gate.shape(),
            "swiglu_backward: all tensors must have the same non-empty shape");
    check(cgpt_swiglu_backward(ptr(grad_gate), ptr(grad_up), ptr(grad_output), ptr(gate), ptr(up), gate.numel(), o.accumulate_gate,
                               o.accumulate_up, code(gate.dtype()), stream),
          "swiglu_backward");
}

void embedding_backward(Tensor& grad_weight, const Tensor& grad_output, const bpe::TokenId* device_token_ids, std::size_t token_count,
                        cudaStream_t stream, const EmbeddingBackwardOptions& o) {
    require(device_token_ids != nullptr, "embedding_backward: token_ids cannot be null");
    require(token_count != 0, "embedding_backward: token_count must be positive");
    require(o.block_size >= 0 && o.block_size <= 1024, "embedding_backward: invalid block size");
    require(same_cuda_dtype({&grad_weight, &grad_output}), "embedding_backward: tensors must be CUDA tensors with the same dtype");
    require(grad_weight.dim() == 2 && grad_output.dim() >= 1 && grad_output.size(grad_output.dim() - 1) == grad_weight.size(1),
            "embedding_backward: hidden sizes must match");
    require(grad_output.numel() == token_count * grad_weight.size(1), "embedding_backward: grad_output must hold token_count rows");
    // bounds_check = false promises in-range ids; the library skips out-of-range ids either way instead of dereferencing them
    check(cgpt_embedding_backward(ptr(grad_weight), ptr(grad_output), device_token_ids, token_count, grad_weight.size(0),
                                  grad_weight.size(1), 1, o.accumulate_weight, code(grad_weight.dtype()), stream),
          "embedding_backward");
}

void linear_backward(Tensor& grad_input, Tensor& grad_weight, Tensor& grad_bias, const Tensor& grad_output, const Tensor& input,
                     const Tensor& weight, const CublasLtContext& context, cudaStream_t stream, const LinearBackwardOptions& o) {
    require(input.dim() >= 2, "linear_backward: input must have at least 2 dimensions");
    require(weight.dim() == 2, "linear_backward: weight must have shape [out_features, in_features]");
    require(grad_output.dim() == input.dim() && grad_input.shape() == input.shape(),
            "linear_backward: grad_output and grad_input must match input rank and leading dimensions");
    const std::size_t in_features = input.size(input.dim() - 1), out_features = weight.size(0);
    require(weight.size(1) == in_features, "linear_backward: input feature size does not match weight");
    for (std::size_t axis = 0; axis + 1 < input.dim(); ++axis)
        require(grad_output.size(axis) == input.size(axis), "linear_backward: grad_output leading dimensions must match input");
    require(grad_output.size(grad_output.dim() - 1) == out_features && grad_weight.shape() == weight.shape() &&
                grad_bias.dim() == 1 && grad_bias.size(0) == out_features,
            "linear_backward: invalid gradient shape");
    require(same_cuda_dtype({&input, &weight, &grad_output, &grad_input, &grad_weight, &grad_bias}),
            "linear_backward: all tensors must be CUDA tensors with the same floating dtype");
    require(is_valid_compute_type(o.compute_type), "linear_backward: invalid compute type");
    // The cuBLASLt handle is not used; the tensors must live on the context's device, as CGPT requires.
    int device = 0;
    CUDA_CHECK(cudaGetDevice(&device));
    require(device == context.device_index(), "linear_backward: tensors must be on the same device as the cuBLASLt context");
    const std::size_t rows = input.numel() / in_features;
    check(cgpt_linear_backward(ptr(grad_input), ptr(grad_weight), ptr(grad_bias), ptr(grad_output), ptr(input), ptr(weight), rows,
                               in_features, out_features, o.accumulate_input, o.accumulate_weight, o.accumulate_bias,
                               code(input.dtype()), stream),
          "linear_backward");
}

namespace {

void validate_attention(const Tensor& gq, const Tensor& gk, const Tensor& gv, const Tensor& go, const Tensor& q, const Tensor& k,
                        const Tensor& v, const FlashAttentionOptions& o) {
    require(same_cuda_dtype({&q, &gq, &gk, &gv, &go, &k, &v}), "flash_gqa_attention_backward: tensors must be CUDA and have one dtype");
    require(q.dim() == 4 && k.dim() == 4 && v.dim() == 4 && go.shape() == q.shape() && gq.shape() == q.shape() && gv.shape() == k.shape() &&
                gk.shape() == k.shape(),
            "flash_gqa_attention_backward: invalid gradient or operand shape");
    require(v.shape() == k.shape() && o.num_query_heads != 0 && o.num_kv_heads != 0 && o.head_dim != 0 &&
                o.num_query_heads % o.num_kv_heads == 0 && q.size(2) == o.num_query_heads && k.size(2) == o.num_kv_heads &&
                q.size(3) == o.head_dim && k.size(3) == o.head_dim && q.size(0) == k.size(0),
            "flash_gqa_attention_backward: invalid attention configuration");
    require(o.head_dim <= 128, "flash_gqa_attention_backward: head_dim must not exceed 128");
    require(std::isfinite(o.attention_scale) && o.attention_scale >= 0.0F && (!o.causal || o.query_position_offset + q.size(1) <= k.size(1)),
            "flash_gqa_attention_backward: invalid scale or causal range");
    require(q.size(0) <= INT_MAX && q.size(1) <= INT_MAX && k.size(1) <= INT_MAX, "flash_gqa_attention_backward: dimensions exceed CUDA limits");
}

void attention_backward(Tensor& gq, Tensor& gk, Tensor& gv, const Tensor& go, const Tensor* out, const Tensor* lse, const Tensor& q,
                        const Tensor& k, const Tensor& v, cudaStream_t stream, const FlashAttentionOptions& o, bool accumulate,
                        const char* what) {
    check(cgpt_attention_backward(ptr(gq), ptr(gk), ptr(gv), ptr(go), out != nullptr ? ptr(*out) : nullptr,
                                  lse != nullptr ? static_cast<const float*>(lse->raw_data()) : nullptr, ptr(q), ptr(k), ptr(v), q.size(0),
                                  q.size(1), k.size(1), o.num_query_heads, o.num_kv_heads, o.head_dim, o.attention_scale, o.causal,
                                  o.query_position_offset, accumulate, code(q.dtype()), 0, stream),
          what);
}

}  // namespace

void flash_gqa_attention_backward(Tensor& grad_query, Tensor& grad_key, Tensor& grad_value, const Tensor& grad_output,
                                  const Tensor& query, const Tensor& key, const Tensor& value, cudaStream_t stream,
                                  const FlashAttentionOptions& options, bool accumulate_grads) {
    validate_attention(grad_query, grad_key, grad_value, grad_output, query, key, value, options);
    attention_backward(grad_query, grad_key, grad_value, grad_output, nullptr, nullptr, query, key, value, stream, options,
                       accumulate_grads, "flash_gqa_attention_backward");
}

void flash_gqa_attention_backward_with_lse(Tensor& grad_query, Tensor& grad_key, Tensor& grad_value, const Tensor& grad_output,
                                           const Tensor& output, const Tensor& logsumexp, const Tensor& query, const Tensor& key,
                                           const Tensor& value, cudaStream_t stream, const FlashAttentionOptions& options,
                                           bool accumulate_grads) {
    validate_attention(grad_query, grad_key, grad_value, grad_output, query, key, value, options);
    require(output.device_type() == DeviceType::CUDA && output.dtype() == query.dtype() && output.shape() == query.shape() &&
                logsumexp.device_type() == DeviceType::CUDA && logsumexp.dtype() == Dtype::F32 &&
                logsumexp.shape() == Shape{query.size(0), query.size(1), query.size(2)},
            "flash_gqa_attention_backward_with_lse: invalid saved output or logsumexp");
    attention_backward(grad_query, grad_key, grad_value, grad_output, &output, &logsumexp, query, key, value, stream, options,
                       accumulate_grads, "flash_gqa_attention_backward_with_lse");
}

// =====================================================================================================================
// Loss layer
// =====================================================================================================================

void cross_entropy_forward_backward(Tensor& loss, Tensor& gradient, const Tensor& logits, const bpe::TokenId* device_targets,
                                    std::size_t target_count, cudaStream_t stream, float gradient_scale) {
    require(std::isfinite(gradient_scale) && gradient_scale > 0.0F, "cross_entropy: gradient scale must be finite and positive");
    require(cuda_float(logits) && logits.dim() == 2 && logits.numel() != 0 && device_targets != nullptr,
            "cross_entropy: logits and targets must be non-empty CUDA inputs");
    require(gradient.device_type() == DeviceType::CUDA && gradient.dtype() == logits.dtype() && gradient.shape() == logits.shape() &&
                target_count == logits.size(0),
            "cross_entropy: invalid gradient or target count");
    require(loss.device_type() == DeviceType::CUDA && loss.dtype() == Dtype::F32 && loss.numel() == 1,
            "cross_entropy: loss must be a CUDA F32 tensor with shape [1]");
    check(cgpt_cross_entropy(static_cast<float*>(ptr(loss)), ptr(gradient), ptr(logits), device_targets, logits.size(0), logits.size(1),
                             gradient_scale, code(logits.dtype()), stream),
          "cross_entropy_forward_backward");
}

void cross_entropy_forward(Tensor& loss, const Tensor& logits, const bpe::TokenId* device_targets, std::size_t target_count,
                           cudaStream_t stream) {
    require(cuda_float(logits) && logits.dim() == 2 && logits.numel() != 0 && device_targets != nullptr && target_count == logits.size(0),
            "cross_entropy: invalid logits or target count");
    require(loss.device_type() == DeviceType::CUDA && loss.dtype() == Dtype::F32 && loss.numel() == 1,
            "cross_entropy: loss must be a CUDA F32 tensor with shape [1]");
    check(cgpt_cross_entropy(static_cast<float*>(ptr(loss)), nullptr, ptr(logits), device_targets, logits.size(0), logits.size(1), 1.0F,
                             code(logits.dtype()), stream),
          "cross_entropy_forward");
}

// CGPT's operator takes F32 only (src/ops/cut_cross_entropy.cu:167-172); the library's also takes the 16-bit training
// dtypes, so this entry point accepts every floating dtype. There is no gradient_scale in CGPT's signature: it is 1.
void cut_cross_entropy_forward_backward(Tensor& loss, Tensor& input_gradient, Tensor& classifier_gradient, const Tensor& input,
                                        const Tensor& classifier, const bpe::TokenId* device_targets, std::size_t target_count,
                                        cudaStream_t stream) {
    require(same_cuda_dtype({&input, &classifier}) && input.dim() == 2 && classifier.dim() == 2 && input.numel() != 0 &&
                classifier.numel() != 0 && input.size(1) == classifier.size(1),
            "cut_cross_entropy: input and classifier must be non-empty CUDA matrices of one floating dtype");
    require(same_cuda_dtype({&input, &input_gradient, &classifier_gradient}) && input_gradient.shape() == input.shape() &&
                classifier_gradient.shape() == classifier.shape() && device_targets != nullptr && target_count == input.size(0),
            "cut_cross_entropy: incompatible gradient or target count");
    require(loss.device_type() == DeviceType::CUDA && loss.dtype() == Dtype::F32 && loss.numel() == 1,
            "cut_cross_entropy: loss must be a CUDA F32 tensor with shape [1]");
    check(cgpt_cut_cross_entropy(static_cast<float*>(ptr(loss)), ptr(input_gradient), ptr(classifier_gradient), ptr(input), ptr(classifier),
                                 device_targets, target_count, classifier.size(0), input.size(1), 1.0F, 0, 0, code(input.dtype()), stream),
          "cut_cross_entropy_forward_backward");
}

// =====================================================================================================================
// Transformer block
// =====================================================================================================================

// CGPT allocates seventeen tensors here, about 1 GB per layer at the 104m training shape
// (src/core/transformer_block.cu:338-362). The library's block backward carves everything it needs out of ONE buffer
// of cgpt_block_workspace_bytes() bytes; it lives in `grad_attention_norm_input` (as rows of `hidden` elements). The
// other sixteen members keep their names and dtype but hold a single element: they are scratch that callers never read.
TransformerBlockBackwardWorkspace::TransformerBlockBackwardWorkspace(const TransformerBlockOptions& options, const std::size_t batch_size,
                                                                     const std::size_t sequence_length, const Dtype dtype)
    : grad_attention_norm_input(
          [&]() -> Shape {
              if (options.hidden_size == 0 || batch_size == 0 || sequence_length == 0 || !is_floating_point(dtype) ||
                  g_block_workspace_token_only)
                  return {1};
              const cgpt_model_config cfg = make_config(options, dtype, sequence_length);
              const std::size_t bytes = cgpt_block_workspace_bytes(&cfg, batch_size, sequence_length);
              const std::size_t row_bytes = options.hidden_size * dtype_size(dtype);
              return {(bytes + row_bytes - 1) / row_bytes + 1, options.hidden_size};
          }(),
          is_floating_point(dtype) ? dtype : Dtype::F16),
      attention_norm_output({1}, Dtype::F16), grad_ffn_norm_input({1}, Dtype::F16), grad_residual({1}, Dtype::F16),
      grad_attention_projection({1}, Dtype::F16), grad_attention_output({1}, Dtype::F16), grad_query({1}, Dtype::F16),
      grad_key({1}, Dtype::F16), grad_value({1}, Dtype::F16), grad_query_pre_rope({1}, Dtype::F16), grad_key_pre_rope({1}, Dtype::F16),
      grad_gate({1}, Dtype::F16), grad_up({1}, Dtype::F16), grad_activated({1}, Dtype::F16), hidden_bias({1}, Dtype::F16),
      intermediate_bias({1}, Dtype::F16), kv_bias({1}, Dtype::F16) {
    validate_block_options(options);
    require(batch_size != 0 && sequence_length != 0 && is_floating_point(dtype),
            "transformer block backward workspace requires positive dimensions and a floating dtype");
    if (!g_block_workspace_token_only) {
        const cgpt_model_config cfg = make_config(options, dtype, sequence_length);
        require(cgpt_block_workspace_bytes(&cfg, batch_size, sequence_length) != 0,
                "transformer block backward workspace: configuration not supported (hidden must equal query heads x head_dim)");
    }
}

namespace {

struct BlockShape {
    std::size_t rows, batch, sequence;
};

// Argument checks shared by the block forward and backward: CGPT's conditions and exception types
// (src/core/transformer_block.cu:421-465).
BlockShape validate_block_call(const Tensor& output, const Tensor& input, const TransformerBlockWorkspace& workspace,
                               const TransformerBlockOptions& options) {
    validate_block_options(options);
    require(input.dim() == 2 && output.shape() == input.shape(), "transformer block input/output must be [batch * sequence, hidden]");
    const std::size_t rows = input.size(0), hidden = input.size(1);
    require(hidden == options.hidden_size, "transformer block hidden size mismatch");
    require(workspace.query.dim() == 4, "workspace.query must initially be [batch, sequence, query_heads, head_dim]");
    const std::size_t batch = workspace.query.size(0), sequence = workspace.query.size(1);
    require(batch * sequence == rows, "workspace batch * sequence must be equal input rows");
    require_shape(workspace.query, {batch, sequence, options.num_query_heads, options.head_dim}, "query");
    require_shape(workspace.key, {batch, sequence, options.num_kv_heads, options.head_dim}, "key");
    require_shape(workspace.value, {batch, sequence, options.num_kv_heads, options.head_dim}, "value");
    require_shape(workspace.query_pre_norm, {batch, sequence, options.num_query_heads, options.head_dim}, "query_pre_norm");
    require_shape(workspace.key_pre_norm, {batch, sequence, options.num_kv_heads, options.head_dim}, "key_pre_norm");
    require_shape(workspace.attention_output, {batch, sequence, options.num_query_heads, options.head_dim}, "attention_output");
    require_shape(workspace.attention_logsumexp, {batch, sequence, options.num_query_heads}, "attention_logsumexp");
    require(workspace.attention_logsumexp.dtype() == Dtype::F32, "attention_logsumexp must use F32 storage");
    require_shape(workspace.norm, {rows, hidden}, "norm");
    require_shape(workspace.attention_projection, {rows, hidden}, "attention_projection");
    require_shape(workspace.gate, {rows, options.intermediate_size}, "gate");
    require_shape(workspace.up, {rows, options.intermediate_size}, "up");
    require_shape(workspace.activated, {rows, options.intermediate_size}, "activated");
    require_shape(workspace.ffn_output, {rows, hidden}, "ffn_output");
    require(cuda_float(input) && output.device_type() == DeviceType::CUDA && output.dtype() == input.dtype() &&
                workspace.query.dtype() == input.dtype(),
            "transformer block tensors must be CUDA tensors of one floating dtype");
    require(options.num_query_heads * options.head_dim == options.hidden_size,
            "transformer block: query heads times head_dim must equal hidden_size");
    return {rows, batch, sequence};
}

// The block forward as separate operator calls, for the cases the one-call form does not cover: a KV cache (decoding)
// or non-causal attention. Same operator order as CGPT (src/core/transformer_block.cu:466-595).
void block_forward_stepwise(Tensor& output, const Tensor& input, const TransformerBlockWeights& w, TransformerBlockWorkspace& ws,
                            const Tensor& cos_cache, const Tensor& sin_cache, cudaStream_t stream, const TransformerBlockOptions& o,
                            std::size_t position_offset, Tensor* key_cache, Tensor* value_cache, std::size_t cache_length,
                            const BlockShape& s) {
    const int dt = code(input.dtype());
    const std::size_t d = o.hidden_size, qd = o.num_query_heads * o.head_dim, kvd = o.num_kv_heads * o.head_dim;
    const std::size_t rotary = o.rotary_dim != 0 ? o.rotary_dim : o.head_dim;
    check(cgpt_rmsnorm_forward(ptr(ws.norm), ptr(input), ptr(w.attention_norm), s.rows, d, o.rms_epsilon, dt, stream), "block: attention norm");
    check(cgpt_linear_forward(ptr(ws.query_pre_norm), ptr(ws.norm), ptr(w.q_projection), s.rows, d, qd, dt, stream), "block: q projection");
    check(cgpt_linear_forward(ptr(ws.key_pre_norm), ptr(ws.norm), ptr(w.k_projection), s.rows, d, kvd, dt, stream), "block: k projection");
    check(cgpt_linear_forward(ptr(ws.value), ptr(ws.norm), ptr(w.v_projection), s.rows, d, kvd, dt, stream), "block: v projection");
    check(cgpt_rmsnorm_forward(ptr(ws.query), ptr(ws.query_pre_norm), ptr(w.q_norm), s.rows * o.num_query_heads, o.head_dim, o.rms_epsilon, dt,
                               stream), "block: q norm");
    check(cgpt_rmsnorm_forward(ptr(ws.key), ptr(ws.key_pre_norm), ptr(w.k_norm), s.rows * o.num_kv_heads, o.head_dim, o.rms_epsilon, dt, stream),
          "block: k norm");
    check(cgpt_rope_forward(ptr(ws.query), ptr(ws.key), ptr(cos_cache), ptr(sin_cache), s.batch, s.sequence, o.num_query_heads, o.num_kv_heads,
                            o.head_dim, rotary, position_offset, cos_cache.size(0), dt, stream), "block: rope");
    const void* attention_key = ptr(ws.key);
    const void* attention_value = ptr(ws.value);
    std::size_t key_length = s.sequence;
    if (key_cache != nullptr || value_cache != nullptr) {
        require(key_cache != nullptr && value_cache != nullptr && key_cache->dim() == 4 && value_cache->shape() == key_cache->shape() &&
                    key_cache->size(0) == s.batch && key_cache->size(1) >= cache_length + s.sequence && key_cache->size(2) == o.num_kv_heads &&
                    key_cache->size(3) == o.head_dim && key_cache->dtype() == ws.key.dtype() && value_cache->dtype() == ws.value.dtype(),
                "invalid transformer KV cache shape");
        // append this call's keys and values behind the cached prefix of every sequence
        const std::size_t token_bytes = kvd * dtype_size(ws.key.dtype());
        for (std::size_t b = 0; b < s.batch; ++b) {
            auto* kd = static_cast<unsigned char*>(ptr(*key_cache)) + (b * key_cache->size(1) + cache_length) * token_bytes;
            auto* vd = static_cast<unsigned char*>(ptr(*value_cache)) + (b * value_cache->size(1) + cache_length) * token_bytes;
            const auto* ks = static_cast<const unsigned char*>(ptr(ws.key)) + b * s.sequence * token_bytes;
            const auto* vs = static_cast<const unsigned char*>(ptr(ws.value)) + b * s.sequence * token_bytes;
            CUDA_CHECK(cudaMemcpyAsync(kd, ks, s.sequence * token_bytes, cudaMemcpyDeviceToDevice, stream));
            CUDA_CHECK(cudaMemcpyAsync(vd, vs, s.sequence * token_bytes, cudaMemcpyDeviceToDevice, stream));
        }
        attention_key = ptr(*key_cache);
        attention_value = ptr(*value_cache);
        key_length = cache_length + s.sequence;   // CGPT views the cache as [batch, cache_length + sequence, ...] (:549-556)
    }
    check(cgpt_attention_forward(ptr(ws.attention_output), static_cast<float*>(ptr(ws.attention_logsumexp)), ptr(ws.query), attention_key,
                                 attention_value, s.batch, s.sequence, key_length, o.num_query_heads, o.num_kv_heads, o.head_dim, 0.0F,
                                 o.causal, position_offset, dt, 0, stream), "block: attention");
    check(cgpt_linear_forward(ptr(ws.attention_projection), ptr(ws.attention_output), ptr(w.o_projection), s.rows, qd, d, dt, stream),
          "block: o projection");
    check(cgpt_rmsnorm_forward(ptr(ws.norm), ptr(input), ptr(w.ffn_norm), s.rows, d, o.rms_epsilon, dt, stream), "block: ffn norm");
    check(cgpt_linear_forward(ptr(ws.gate), ptr(ws.norm), ptr(w.gate_proj), s.rows, d, o.intermediate_size, dt, stream), "block: gate");
    check(cgpt_linear_forward(ptr(ws.up), ptr(ws.norm), ptr(w.up_proj), s.rows, d, o.intermediate_size, dt, stream), "block: up");
    check(cgpt_swiglu_forward(ptr(ws.activated), ptr(ws.gate), ptr(ws.up), s.rows * o.intermediate_size, dt, stream), "block: swiglu");
    check(cgpt_linear_forward(ptr(ws.ffn_output), ptr(ws.activated), ptr(w.down_proj), s.rows, o.intermediate_size, d, dt, stream), "block: down");
    check(cgpt_add(ptr(output), ptr(input), ptr(ws.attention_projection), ptr(ws.ffn_output), s.rows * d, dt, stream), "block: residual");
}

}  // namespace

void transformer_block_forward(Tensor& output, const Tensor& input, const TransformerBlockWeights& weights,
                               TransformerBlockWorkspace& workspace, const Tensor& cos_cache, const Tensor& sin_cache,
                               const CublasLtContext&, cudaStream_t stream, const TransformerBlockOptions& options,
                               std::size_t position_offset, Tensor* key_cache, Tensor* value_cache, const std::size_t cache_length) {
    const BlockShape s = validate_block_call(output, input, workspace, options);
    require(cos_cache.dim() == 2 && sin_cache.shape() == cos_cache.shape() && cos_cache.dtype() == input.dtype(),
            "transformer block: rotary caches must be [positions, rotary_dim / 2] in the activations' dtype");
    if (key_cache != nullptr || value_cache != nullptr || !options.causal) {
        block_forward_stepwise(output, input, weights, workspace, cos_cache, sin_cache, stream, options, position_offset, key_cache,
                               value_cache, cache_length, s);
        return;
    }
    const cgpt_model_config cfg = make_config(options, input.dtype(), cos_cache.size(0));
    const std::size_t bytes = cgpt_block_workspace_bytes(&cfg, s.batch, s.sequence);
    require(bytes != 0, "transformer block: configuration not supported");
    const cgpt_block_params w = params_of(weights);
    const cgpt_block_saved saved = saved_of(workspace);
    check(cgpt_block_forward(ptr(output), ptr(input), &w, &saved, forward_scratch(bytes), ptr(cos_cache), ptr(sin_cache), &cfg, s.batch,
                             s.sequence, position_offset, stream),
          "transformer_block_forward");
}

void transformer_block_backward(Tensor& grad_input, const Tensor& grad_output, const Tensor& input, const TransformerBlockWeights& weights,
                                TransformerBlockGradients gradients, const TransformerBlockWorkspace& forward_workspace,
                                TransformerBlockBackwardWorkspace& backward_workspace, const Tensor& cos_cache, const Tensor& sin_cache,
                                const CublasLtContext&, cudaStream_t stream, const TransformerBlockOptions& options,
                                std::size_t position_offset) {
    require(grad_output.shape() == input.shape() && grad_output.dtype() == input.dtype() && grad_output.device_type() == DeviceType::CUDA,
            "transformer block backward: grad_output must match the block input");
    const BlockShape s = validate_block_call(grad_input, input, forward_workspace, options);
    require(options.causal, "transformer block backward: the training path is causal");
    const cgpt_model_config cfg = make_config(options, input.dtype(), cos_cache.size(0));
    const std::size_t bytes = cgpt_block_workspace_bytes(&cfg, s.batch, s.sequence);
    require(bytes != 0, "transformer block backward: configuration not supported");
    require(backward_workspace.grad_attention_norm_input.nbytes() >= bytes,
            "transformer block backward: workspace was built for a smaller batch, sequence or model");
    const cgpt_block_params w = params_of(weights), g = params_of(gradients);
    const cgpt_block_saved saved = saved_of(forward_workspace);
    check(cgpt_block_backward(ptr(grad_input), ptr(grad_output), ptr(input), &w, &g, &saved, ptr(backward_workspace.grad_attention_norm_input),
                              ptr(cos_cache), ptr(sin_cache), &cfg, s.batch, s.sequence, position_offset, stream),
          "transformer_block_backward");
}

// =====================================================================================================================
// Transformer model
// =====================================================================================================================

namespace {

TransformerBlockWorkspace make_block_workspace(const TransformerModelOptions& options, std::size_t batch, std::size_t sequence, Dtype dtype) {
    const TransformerBlockOptions& b = options.block_options;
    const std::size_t rows = batch * sequence;
    return {Tensor({rows, b.hidden_size}, dtype),
            Tensor({batch, sequence, b.num_query_heads, b.head_dim}, dtype),
            Tensor({batch, sequence, b.num_kv_heads, b.head_dim}, dtype),
            Tensor({batch, sequence, b.num_kv_heads, b.head_dim}, dtype),
            Tensor({batch, sequence, b.num_query_heads, b.head_dim}, dtype),
            Tensor({batch, sequence, b.num_kv_heads, b.head_dim}, dtype),
            Tensor({batch, sequence, b.num_query_heads, b.head_dim}, dtype),
            Tensor({batch, sequence, b.num_query_heads}, Dtype::F32),
            Tensor({rows, b.hidden_size}, dtype),
            Tensor({rows, b.intermediate_size}, dtype),
            Tensor({rows, b.intermediate_size}, dtype),
            Tensor({rows, b.intermediate_size}, dtype),
            Tensor({rows, b.hidden_size}, dtype)};
}

void require_cuda_tensor(const Tensor& t, const Shape& shape, Dtype dtype, const char* name) {
    if (t.device_type() != DeviceType::CUDA || t.dtype() != dtype || t.shape() != shape)
        throw std::invalid_argument(std::string("transformer model: invalid ") + name + " tensor");
}

}  // namespace

TransformerModelWorkspace::TransformerModelWorkspace(const TransformerModelOptions& options, const std::size_t batch_size,
                                                     const std::size_t sequence_length, const Dtype dtype)
    : hidden({batch_size * sequence_length, options.block_options.hidden_size}, dtype),
      layer_output({batch_size * sequence_length, options.block_options.hidden_size}, dtype),
      normalized({batch_size * sequence_length, options.block_options.hidden_size}, dtype) {
    validate_model_options(options);
    require(batch_size != 0 && sequence_length != 0 && is_floating_point(dtype),
            "transformer model workspace requires positive dimensions and a floating dtype");
    if (batch_size > std::numeric_limits<std::size_t>::max() / sequence_length)
        throw std::overflow_error("transformer model workspace row count overflows");
    layers.reserve(options.num_layers);
    for (std::size_t layer = 0; layer < options.num_layers; ++layer) {
        layers.push_back(make_block_workspace(options, batch_size, sequence_length, dtype));
        layer_inputs.emplace_back(Shape{batch_size * sequence_length, options.block_options.hidden_size}, dtype);
    }
}

// One block scratch buffer serves all layers (they run one after the other on one stream): layers[0] owns it, the
// remaining entries are token allocations. CGPT allocates a full set of seventeen tensors per layer
// (src/core/transformer_model.cu:152-166).
TransformerModelBackwardWorkspace::TransformerModelBackwardWorkspace(const TransformerModelOptions& options, const std::size_t batch_size,
                                                                     const std::size_t sequence_length, const Dtype dtype)
    : grad_normalized({batch_size * sequence_length, options.block_options.hidden_size}, dtype),
      grad_hidden({batch_size * sequence_length, options.block_options.hidden_size}, dtype),
      grad_previous({batch_size * sequence_length, options.block_options.hidden_size}, dtype),
      lm_head_bias({options.vocabulary_size}, dtype) {
    validate_model_options(options);
    require(batch_size != 0 && sequence_length != 0 && is_floating_point(dtype),
            "transformer model backward workspace requires positive dimensions and a floating dtype");
    layers.reserve(options.num_layers);
    struct TokenOnly {
        explicit TokenOnly(bool on) { g_block_workspace_token_only = on; }
        ~TokenOnly() { g_block_workspace_token_only = false; }
    };
    for (std::size_t layer = 0; layer < options.num_layers; ++layer) {
        const TokenOnly guard(layer != 0);
        layers.emplace_back(options.block_options, batch_size, sequence_length, dtype);
    }
}

void transformer_model_forward(Tensor& logits, const bpe::TokenId* const device_token_ids, const std::size_t batch_size,
                               const std::size_t sequence_length, const TransformerModelWeights& weights,
                               TransformerModelWorkspace& workspace, const Tensor& cos_cache, const Tensor& sin_cache,
                               const CublasLtContext& cublas_context, cudaStream_t stream, const TransformerModelOptions& options,
                               const std::size_t position_offset) {
    validate_model_options(options);
    require(device_token_ids != nullptr && batch_size != 0 && sequence_length != 0,
            "transformer model requires token IDs and positive batch/sequence dimensions");
    if (batch_size > std::numeric_limits<std::size_t>::max() / sequence_length) throw std::overflow_error("transformer model row count overflows");
    const std::size_t rows = batch_size * sequence_length;
    const TransformerBlockOptions& block = options.block_options;
    const Dtype dtype = weights.token_embedding.dtype();
    require(is_floating_point(dtype) && weights.layers.size() == options.num_layers, "transformer model weights have an invalid dtype or layer count");
    require_cuda_tensor(weights.token_embedding, {options.vocabulary_size, block.hidden_size}, dtype, "token_embedding");
    require_cuda_tensor(weights.final_norm, {block.hidden_size}, dtype, "final_norm");
    require_cuda_tensor(weights.lm_head, {options.vocabulary_size, block.hidden_size}, dtype, "lm_head");
    require_cuda_tensor(workspace.hidden, {rows, block.hidden_size}, dtype, "workspace.hidden");
    require_cuda_tensor(workspace.layer_output, {rows, block.hidden_size}, dtype, "workspace.layer_output");
    require_cuda_tensor(workspace.normalized, {rows, block.hidden_size}, dtype, "workspace.normalized");
    require_cuda_tensor(logits, {rows, options.vocabulary_size}, dtype, "logits");
    require(workspace.layers.size() == options.num_layers && workspace.layer_inputs.size() == options.num_layers,
            "transformer model workspace layer count mismatch");
    const int dt = code(dtype);
    // The embedding is written straight into the first layer's saved input and every block writes the next layer's
    // saved input (the last one writes workspace.hidden): CGPT's per-layer D2D copy of the hidden state
    // (src/core/transformer_model.cu:230) is not needed, and workspace.hidden ends as the last block's output as in CGPT.
    check(cgpt_embedding_forward(ptr(workspace.layer_inputs[0]), device_token_ids, ptr(weights.token_embedding), rows, options.vocabulary_size,
                                 block.hidden_size, dt, stream),
          "transformer_model_forward: embedding");
    for (std::size_t layer = 0; layer < options.num_layers; ++layer) {
        Tensor& out = layer + 1 < options.num_layers ? workspace.layer_inputs[layer + 1] : workspace.hidden;
        transformer_block_forward(out, workspace.layer_inputs[layer], weights.layers[layer], workspace.layers[layer], cos_cache, sin_cache,
                                  cublas_context, stream, block, position_offset);
    }
    check(cgpt_rmsnorm_forward(ptr(workspace.normalized), ptr(workspace.hidden), ptr(weights.final_norm), rows, block.hidden_size,
                               block.rms_epsilon, dt, stream),
          "transformer_model_forward: final norm");
    check(cgpt_linear_forward(ptr(logits), ptr(workspace.normalized), ptr(weights.lm_head), rows, block.hidden_size, options.vocabulary_size, dt,
                              stream),
          "transformer_model_forward: lm head");
}

// One-token decode against the KV cache: CGPT's own sequence of calls (src/core/transformer_model.cu:259-300) over this
// file's transformer_block_forward; the forward operators it uses on their own remain CGPT's.
void transformer_model_forward_cached(Tensor& logits, const bpe::TokenId* const device_token_ids, const TransformerModelWeights& weights,
                                      TransformerModelWorkspace& workspace, KVCache& kv_cache, const std::size_t cache_length,
                                      const Tensor& cos_cache, const Tensor& sin_cache, const CublasLtContext& cublas_context,
                                      cudaStream_t stream, const TransformerModelOptions& options) {
    const TransformerBlockOptions& block = options.block_options;
    require(device_token_ids != nullptr && workspace.layers.size() == options.num_layers &&
                workspace.hidden.shape() == Shape{1, block.hidden_size} && logits.shape() == Shape{1, options.vocabulary_size},
            "cached transformer model: invalid workspace or token IDs");
    embedding_forward(workspace.hidden, device_token_ids, 1, weights.token_embedding, stream);
    for (std::size_t layer = 0; layer < options.num_layers; ++layer) {
        const Shape cache_shape{1, kv_cache.config().max_sequence_length, block.num_kv_heads, block.head_dim};
        Tensor key_cache = Tensor::device_view(cache_shape, kv_cache.key_sequence(layer, 0), Dtype::F16);
        Tensor value_cache = Tensor::device_view(cache_shape, kv_cache.value_sequence(layer, 0), Dtype::F16);
        transformer_block_forward(workspace.layer_output, workspace.hidden, weights.layers[layer], workspace.layers[layer], cos_cache, sin_cache,
                                  cublas_context, stream, block, cache_length, &key_cache, &value_cache, cache_length);
        std::swap(workspace.hidden, workspace.layer_output);
        kv_cache.advance_sequence_length(layer, 0, 1);
    }
    rmsnorm_forward(workspace.normalized, workspace.hidden, weights.final_norm, block.rms_epsilon, stream);
    linear_forward(logits, workspace.normalized, weights.lm_head, cublas_context, stream, block.linear_options);
}

void transformer_model_backward(const Tensor& grad_logits, const bpe::TokenId* const device_token_ids, const std::size_t batch_size,
                                const std::size_t sequence_length, const TransformerModelWeights& weights,
                                const TransformerModelGradients gradients, const TransformerModelWorkspace& forward_workspace,
                                TransformerModelBackwardWorkspace& backward_workspace, const Tensor& cos_cache, const Tensor& sin_cache,
                                const CublasLtContext& cublas_context, cudaStream_t stream, const TransformerModelOptions& options,
                                const std::size_t position_offset) {
    validate_model_options(options);
    require(device_token_ids != nullptr && batch_size != 0 && sequence_length != 0 && gradients.layers.size() == options.num_layers &&
                forward_workspace.layers.size() == options.num_layers && forward_workspace.layer_inputs.size() == options.num_layers &&
                backward_workspace.layers.size() == options.num_layers,
            "transformer model backward: invalid model state or token IDs");
    const std::size_t rows = batch_size * sequence_length;
    const TransformerBlockOptions& block = options.block_options;
    const Dtype dtype = weights.token_embedding.dtype();
    require(grad_logits.device_type() == DeviceType::CUDA && grad_logits.dtype() == dtype &&
                grad_logits.shape() == Shape{rows, options.vocabulary_size} &&
                backward_workspace.grad_normalized.shape() == Shape{rows, block.hidden_size} &&
                forward_workspace.normalized.shape() == Shape{rows, block.hidden_size} &&
                forward_workspace.hidden.shape() == Shape{rows, block.hidden_size},
            "transformer model backward: invalid logits gradient or workspace shape");
    const int dt = code(dtype);
    // LM head: dX and dW. CGPT also reduces a bias gradient into a scratch buffer that nothing reads
    // (src/core/transformer_model.cu:358-361); the model has no biases, so that column sum over [rows, vocab] is left out.
    check(cgpt_linear_backward(ptr(backward_workspace.grad_normalized), ptr(gradients.lm_head), nullptr, ptr(grad_logits),
                               ptr(forward_workspace.normalized), ptr(weights.lm_head), rows, block.hidden_size, options.vocabulary_size, 0, 0,
                               0, dt, stream),
          "transformer_model_backward: lm head");
    rmsnorm_backward(backward_workspace.grad_hidden, gradients.final_norm, backward_workspace.grad_normalized, forward_workspace.hidden,
                     weights.final_norm, block.rms_epsilon, stream);
    Tensor* current = &backward_workspace.grad_hidden;
    Tensor* previous = &backward_workspace.grad_previous;
    for (std::size_t reverse = options.num_layers; reverse-- > 0;) {
        transformer_block_backward(*previous, *current, forward_workspace.layer_inputs[reverse], weights.layers[reverse],
                                   gradients.layers[reverse], forward_workspace.layers[reverse], backward_workspace.layers[0], cos_cache,
                                   sin_cache, cublas_context, stream, block, position_offset);
        std::swap(current, previous);
    }
    EmbeddingBackwardOptions embedding_options;
    embedding_options.accumulate_weight = &gradients.token_embedding == &gradients.lm_head;   // tied embedding (:375-380)
    embedding_backward(gradients.token_embedding, *current, device_token_ids, rows, stream, embedding_options);
}

// =====================================================================================================================
// AdamW
// =====================================================================================================================

namespace {

void validate_adamw_options(const AdamWOptions& o) {
    const bool ok = std::isfinite(o.learning_rate) && o.learning_rate >= 0.0F && o.beta1 >= 0.0F && o.beta1 < 1.0F && o.beta2 >= 0.0F &&
                    o.beta2 < 1.0F && std::isfinite(o.epsilon) && o.epsilon > 0.0F && std::isfinite(o.weight_decay) && o.weight_decay >= 0.0F &&
                    std::isfinite(o.loss_scale) && o.loss_scale > 0.0F && !std::isnan(o.max_grad_norm) && o.max_grad_norm > 0.0F;
    require(ok, "adamw_step: invalid optimizer options");
}

void validate_adamw_tensors(const Tensor& parameter, const Tensor& gradient, const AdamWState& state) {
    require(is_floating_point(parameter.dtype()) && gradient.dtype() == parameter.dtype() && gradient.shape() == parameter.shape() &&
                gradient.device_type() == parameter.device_type(),
            "adamw_step: parameter and gradient must have the same floating dtype, shape and device");
    for (const Tensor* t : {&state.master_parameter, &state.first_moment, &state.second_moment})
        require(t->dtype() == Dtype::F32 && t->shape() == parameter.shape() && t->device_type() == parameter.device_type(),
                "adamw_step: master parameter and moment buffers must be F32");
}

cgpt_adamw_options c_options(const AdamWOptions& o) {
    return {o.learning_rate, o.beta1, o.beta2, o.epsilon, o.weight_decay, o.loss_scale, o.max_grad_norm};
}

cgpt_adamw_tensor c_tensor(Tensor& parameter, const Tensor& gradient, AdamWState& state) {
    cgpt_adamw_tensor t{};
    t.param = ptr(parameter);
    t.grad = ptr(gradient);
    t.master = static_cast<float*>(ptr(state.master_parameter));
    t.m = static_cast<float*>(ptr(state.first_moment));
    t.v = static_cast<float*>(ptr(state.second_moment));
    t.count = parameter.numel();
    t.dtype = code(parameter.dtype());
    return t;
}

// The library's optimizer object behind each AdamWWorkspace. AdamWWorkspace has no member that could hold a host
// pointer, so the handles live in this table, keyed by the device address of the workspace's own `step_` buffer: that
// allocation belongs to exactly one live workspace and moves with it. A fresh workspace that happens to receive the
// address of a destroyed one is recognised by its `initialized_` flag being false; its predecessor's handle is then
// released.
std::mutex g_adamw_mutex;
std::unordered_map<const void*, cgpt_adamw_workspace*> g_adamw_handles;

// The host loop of CGPT's adamw_step for CPU tensors (src/optim/adamw.cu:193-225): gradients unscaled and checked,
// per-tensor norm clip, the same expression tree as the GPU update, bias corrections passed in.
bool adamw_cpu(Tensor& parameter, const Tensor& gradient, AdamWState& state, const AdamWOptions& o, float bc1, float bc2) {
    std::vector<float> grad(gradient.numel());
    gradient.copy_to_host(grad);
    double squared = 0.0;
    for (const float value : grad) {
        const float g = value / o.loss_scale;
        if (!std::isfinite(g)) return false;
        squared += static_cast<double>(g) * g;
    }
    const float norm = static_cast<float>(std::sqrt(squared));
    const float clip = norm > o.max_grad_norm ? o.max_grad_norm / norm : 1.0F;
    std::vector<float> master(parameter.numel());
    state.master_parameter.copy_to_host(master);
    auto* m = static_cast<float*>(state.first_moment.raw_data());
    auto* v = static_cast<float*>(state.second_moment.raw_data());
    for (std::size_t i = 0; i < master.size(); ++i) {
        const float g = grad[i] / o.loss_scale * clip;
        m[i] = o.beta1 * m[i] + (1.0F - o.beta1) * g;
        v[i] = o.beta2 * v[i] + (1.0F - o.beta2) * g * g;
        const float normalized = (m[i] / bc1) / (std::sqrt(v[i] / bc2) + o.epsilon);
        master[i] = master[i] * (1.0F - o.learning_rate * o.weight_decay) - o.learning_rate * normalized;
    }
    state.master_parameter.copy_from_host(master);
    parameter.copy_from_host(master);
    return true;
}

}  // namespace

AdamWWorkspace::AdamWWorkspace() : step_(sizeof(unsigned long long)) {}

void adamw_step_many_async(std::span<const AdamWBatchEntry> entries, const AdamWOptions& options, AdamWWorkspace& workspace,
                           cudaStream_t stream) {
    validate_adamw_options(options);
    require(!entries.empty(), "adamw_step_many_async: empty parameter list");
    cgpt_adamw_workspace* handle = nullptr;
    if (!workspace.initialized_) {
        std::vector<cgpt_adamw_tensor> tensors;
        tensors.reserve(entries.size());
        const std::uint64_t initial_step = entries.front().state != nullptr ? entries.front().state->step : 0;
        for (const AdamWBatchEntry& e : entries) {
            require(e.parameter != nullptr && e.gradient != nullptr && e.state != nullptr, "adamw_step_many_async: null entry");
            validate_adamw_tensors(*e.parameter, *e.gradient, *e.state);
            require(e.parameter->device_type() == DeviceType::CUDA, "adamw_step_many_async: CUDA tensors required");
            require(e.state->step == initial_step, "adamw_step_many_async: states must share one step count");
            tensors.push_back(c_tensor(*e.parameter, *e.gradient, *e.state));
        }
        check(cgpt_adamw_create(&handle, tensors.data(), tensors.size(), initial_step, stream), "adamw_step_many_async");
        {
            std::lock_guard<std::mutex> lock(g_adamw_mutex);
            cgpt_adamw_workspace*& slot = g_adamw_handles[workspace.step_.data()];
            if (slot != nullptr) cgpt_adamw_destroy(slot);   // left behind by a destroyed workspace whose buffer had this address
            slot = handle;
        }
        workspace.states_.clear();
        for (const AdamWBatchEntry& e : entries) workspace.states_.push_back(e.state);
        workspace.initialized_ = true;
    } else {
        require(workspace.states_.size() == entries.size(), "adamw_step_many_async: workspace entries changed");
        for (std::size_t i = 0; i < entries.size(); ++i)
            require(entries[i].state == workspace.states_[i], "adamw_step_many_async: workspace states changed");
        std::lock_guard<std::mutex> lock(g_adamw_mutex);
        handle = g_adamw_handles.at(workspace.step_.data());
    }
    const cgpt_adamw_options o = c_options(options);
    check(cgpt_adamw_step(handle, &o, stream), "adamw_step_many_async");
}

bool adamw_check(AdamWWorkspace& workspace, cudaStream_t stream) {
    if (!workspace.initialized_) {
        CUDA_CHECK(cudaStreamSynchronize(stream));
        return true;
    }
    cgpt_adamw_workspace* handle = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_adamw_mutex);
        handle = g_adamw_handles.at(workspace.step_.data());
    }
    std::uint64_t step = 0;
    int non_finite = 0;
    check(cgpt_adamw_check(handle, &step, &non_finite, stream), "adamw_check");
    for (AdamWState* state : workspace.states_) state->step = step;
    return non_finite == 0;
}

AdamWState AdamWState::for_parameter(const Tensor& parameter, cudaStream_t stream) {
    require(is_floating_point(parameter.dtype()), "AdamWState: parameter must have a floating dtype");
    Tensor master(parameter.shape(), parameter.device_type(), Dtype::F32);
    std::vector<float> values(parameter.numel());
    parameter.copy_to_host(values);
    master.copy_from_host(values);
    return {std::move(master), Tensor::zeros(parameter.shape(), parameter.device_type(), stream, Dtype::F32),
            Tensor::zeros(parameter.shape(), parameter.device_type(), stream, Dtype::F32), 0};
}

// Single-tensor step: per-tensor clip, synchronous, returns whether the update was applied. CUDA tensors go through a
// one-entry optimizer object of the library (the step counter lives on the device there, seeded with state.step); CPU
// tensors through the host loop above with CGPT's host-side bias corrections.
bool adamw_step(Tensor& parameter, const Tensor& gradient, AdamWState& state, const AdamWOptions& options, cudaStream_t stream) {
    validate_adamw_options(options);
    validate_adamw_tensors(parameter, gradient, state);
    if (state.step == std::numeric_limits<std::uint64_t>::max()) throw std::overflow_error("adamw_step: step counter overflow");
    if (parameter.device_type() == DeviceType::CPU) {
        const std::uint64_t next = state.step + 1;
        const auto bc1 = static_cast<float>(1.0 - std::pow(static_cast<double>(options.beta1), static_cast<double>(next)));
        const auto bc2 = static_cast<float>(1.0 - std::pow(static_cast<double>(options.beta2), static_cast<double>(next)));
        const bool updated = adamw_cpu(parameter, gradient, state, options, bc1, bc2);
        if (updated) state.step = next;
        return updated;
    }
    const cgpt_adamw_tensor tensor = c_tensor(parameter, gradient, state);
    cgpt_adamw_workspace* handle = nullptr;
    check(cgpt_adamw_create(&handle, &tensor, 1, state.step, stream), "adamw_step");
    const cgpt_adamw_options o = c_options(options);
    int rc = cgpt_adamw_step(handle, &o, stream);
    std::uint64_t step = state.step;
    int non_finite = 0;
    if (rc == CGPT_OK) rc = cgpt_adamw_check(handle, &step, &non_finite, stream);
    cgpt_adamw_destroy(handle);
    check(rc, "adamw_step");
    state.step = step;
    return non_finite == 0;
}
