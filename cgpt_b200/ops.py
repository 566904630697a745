"""Host-side mirror of CGPT's operator API for the training hot path.

Each function has the name, argument order (outputs first, then inputs, then ``stream``, then the
options object) and error behaviour of the C++ function it stands for; ``ValueError`` plays the role
of ``std::invalid_argument``. Tensors are ``torch`` CUDA tensors used purely as device-memory handles;
all arithmetic happens in ``libcgpt_b200.so`` through the C ABI.

Reference declarations: ``include/ops/backward/*.h``, ``include/ops/{rmsnorm,rope,swiglu,embedding,
cross_entropy,cut_cross_entropy}.h``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from ._lib import check, dtype_code, lib, ptr, stream_ptr


@dataclass
class RopeOptions:
    """include/ops/rope.h:6-11"""
    rotary_dim: int = 0
    position_offset: int = 0


@dataclass
class SwiGLUBackwardOptions:
    """include/ops/backward/swiglu_backward.h:6-13"""
    accumulate_gate: bool = False
    accumulate_up: bool = False
    accumulate_gate_up: bool = False


@dataclass
class EmbeddingBackwardOptions:
    """include/ops/backward/embedding_backward.h:6-14"""
    block_size: int = 0
    bounds_check: bool = True
    accumulate_weight: bool = False


def _require(cond: bool, message: str) -> None:
    if not cond:
        raise _lib.CgptInvalidArgument(message)


def _same_cuda_dtype(name: str, *tensors: torch.Tensor) -> None:
    first = tensors[0]
    for t in tensors:
        _require(t.is_cuda, f"{name}: all tensors must be CUDA tensors")
        _require(t.dtype == first.dtype, f"{name}: all tensors must share one dtype")
        _require(t.is_contiguous(), f"{name}: tensors must be contiguous")


def _ids(t: torch.Tensor, count: int, name: str) -> torch.Tensor:
    _require(t is not None and t.is_cuda, f"{name}: token ids must be a CUDA buffer")
    _require(t.dtype in (torch.int32, torch.uint32), f"{name}: token ids must be 32-bit")
    _require(t.numel() >= count, f"{name}: token id buffer too small")
    return t


# ---------------------------------------------------------------------------------------------- Linear
@dataclass
class LinearBackwardOptions:
    """include/ops/backward/linear_backward.h:10-21 (compute_type / workspace_bytes are accepted and
    ignored: accumulation is always fp32 and scratch comes from the library's arena)."""
    compute_type: str = "F32"
    workspace_bytes: int = 32 * 1024 * 1024
    accumulate_input: bool = False
    accumulate_weight: bool = False
    accumulate_bias: bool = False


def linear_forward(output, input, weight, cublas_lt_context=None, stream=None, options=None):
    """linear_forward(output, input, weight, context, stream, options): Y = X W^T (include/ops/linear.h)."""
    _same_cuda_dtype("linear_forward", output, input, weight)
    _require(weight.dim() == 2 and input.shape[-1] == weight.shape[1] and output.shape[-1] == weight.shape[0]
             and output.numel() // weight.shape[0] == input.numel() // weight.shape[1],
             "linear_forward: incompatible shapes")
    rows = input.numel() // weight.shape[1]
    check(lib.cgpt_linear_forward(ptr(output), ptr(input), ptr(weight), rows, weight.shape[1], weight.shape[0],
                                  dtype_code(input), stream_ptr(stream)), "linear_forward")


def linear_backward(grad_input, grad_weight, grad_bias, grad_output, input, weight, cublas_lt_context=None,
                    stream=None, options: LinearBackwardOptions | None = None):
    """linear_backward (include/ops/backward/linear_backward.h:36-46). Any of grad_input / grad_weight /
    grad_bias may be None to skip that product (extension; the reference always computes all three)."""
    o = options or LinearBackwardOptions()
    outs = [t for t in (grad_input, grad_weight, grad_bias) if t is not None]
    _same_cuda_dtype("linear_backward", grad_output, input, weight, *outs)
    out_f, in_f = weight.shape
    rows = input.numel() // in_f
    _require(weight.dim() == 2 and input.shape[-1] == in_f and grad_output.shape[-1] == out_f
             and grad_output.numel() == rows * out_f, "linear_backward: incompatible shapes")
    _require(grad_input is None or grad_input.shape == input.shape, "linear_backward: grad_input shape")
    _require(grad_weight is None or grad_weight.shape == weight.shape, "linear_backward: grad_weight shape")
    _require(grad_bias is None or tuple(grad_bias.shape) == (out_f,), "linear_backward: grad_bias shape")
    check(lib.cgpt_linear_backward(ptr(grad_input), ptr(grad_weight), ptr(grad_bias), ptr(grad_output), ptr(input),
                                   ptr(weight), rows, in_f, out_f, int(o.accumulate_input), int(o.accumulate_weight),
                                   int(o.accumulate_bias), dtype_code(input), stream_ptr(stream)), "linear_backward")


def linear_forward_fused(outputs, input, weights, stream=None):
    """outputs[i] = input @ weights[i].T for up to three projections of one input, as one launch
    (cgpt_linear_forward_fused; the reference calls linear_forward once per projection)."""
    import ctypes as C
    n = len(outputs)
    _require(1 <= n <= 3 and len(weights) == n, "linear_forward_fused: 1..3 projections")
    _same_cuda_dtype("linear_forward_fused", input, *outputs, *weights)
    in_f = input.shape[-1]
    rows = input.numel() // in_f
    for y, w in zip(outputs, weights):
        _require(w.dim() == 2 and w.shape[1] == in_f and y.shape[-1] == w.shape[0] and y.numel() == rows * w.shape[0],
                 "linear_forward_fused: incompatible shapes")
    ys = (C.c_void_p * n)(*[ptr(t) for t in outputs])
    ws = (C.c_void_p * n)(*[ptr(t) for t in weights])
    outs = (C.c_size_t * n)(*[w.shape[0] for w in weights])
    check(lib.cgpt_linear_forward_fused(ys, ptr(input), ws, outs, n, rows, in_f, dtype_code(input), stream_ptr(stream)),
          "linear_forward_fused")


def linear_backward_weight_fused(grad_weights, grad_outputs, input, stream=None, accumulate_weight: bool = False):
    """grad_weights[i] (+)= grad_outputs[i].T @ input for up to three projections of one input, as one launch
    (cgpt_linear_backward_weight_fused; the reference runs one linear_backward per projection)."""
    import ctypes as C
    n = len(grad_weights)
    _require(1 <= n <= 3 and len(grad_outputs) == n, "linear_backward_weight_fused: 1..3 projections")
    _same_cuda_dtype("linear_backward_weight_fused", input, *grad_weights, *grad_outputs)
    in_f = input.shape[-1]
    rows = input.numel() // in_f
    for gw, dy in zip(grad_weights, grad_outputs):
        _require(gw.dim() == 2 and gw.shape[1] == in_f and dy.shape[-1] == gw.shape[0] and dy.numel() == rows * gw.shape[0],
                 "linear_backward_weight_fused: incompatible shapes")
    gws = (C.c_void_p * n)(*[ptr(t) for t in grad_weights])
    dys = (C.c_void_p * n)(*[ptr(t) for t in grad_outputs])
    outs = (C.c_size_t * n)(*[gw.shape[0] for gw in grad_weights])
    check(lib.cgpt_linear_backward_weight_fused(gws, dys, ptr(input), outs, n, rows, in_f, int(accumulate_weight),
                                                dtype_code(input), stream_ptr(stream)), "linear_backward_weight_fused")


def linear_swiglu_forward(gate, up, activated, input, gate_weight, up_weight, stream=None):
    """gate = input @ gate_weight.T, up = input @ up_weight.T, activated = swiglu(gate, up) in one launch
    (cgpt_linear_swiglu_forward; the reference's block forward calls linear_forward twice and swiglu_forward)."""
    _same_cuda_dtype("linear_swiglu_forward", gate, up, activated, input, gate_weight, up_weight)
    inter, in_f = gate_weight.shape
    rows = input.numel() // in_f
    _require(up_weight.shape == gate_weight.shape and input.shape[-1] == in_f
             and all(t.numel() == rows * inter and t.shape[-1] == inter for t in (gate, up, activated)),
             "linear_swiglu_forward: incompatible shapes")
    check(lib.cgpt_linear_swiglu_forward(ptr(gate), ptr(up), ptr(activated), ptr(input), ptr(gate_weight), ptr(up_weight),
                                         rows, in_f, inter, dtype_code(input), stream_ptr(stream)), "linear_swiglu_forward")


def linear_backward_input_fused(grad_input, grad_outputs, weights, stream=None, accumulate_input: bool = False):
    """grad_input (+)= sum_i grad_outputs[i] @ weights[i] for up to three projections of the same input, in one
    pass (cgpt_linear_backward_input_fused; the reference runs one accumulating linear_backward per projection)."""
    import ctypes as C
    n = len(grad_outputs)
    _require(1 <= n <= 3 and len(weights) == n, "linear_backward_input_fused: 1..3 projections")
    _same_cuda_dtype("linear_backward_input_fused", grad_input, *grad_outputs, *weights)
    in_f = grad_input.shape[-1]
    rows = grad_input.numel() // in_f
    for dy, w in zip(grad_outputs, weights):
        _require(w.dim() == 2 and w.shape[1] == in_f and dy.shape[-1] == w.shape[0] and dy.numel() == rows * w.shape[0],
                 "linear_backward_input_fused: incompatible shapes")
    dys = (C.c_void_p * n)(*[ptr(t) for t in grad_outputs])
    ws = (C.c_void_p * n)(*[ptr(t) for t in weights])
    outs = (C.c_size_t * n)(*[w.shape[0] for w in weights])
    check(lib.cgpt_linear_backward_input_fused(ptr(grad_input), dys, ws, outs, n, rows, in_f, int(accumulate_input),
                                               dtype_code(grad_input), stream_ptr(stream)), "linear_backward_input_fused")


def linear_forward_sum(output, inputs, weights, residual=None, stream=None):
    """output = residual + sum_i inputs[i] @ weights[i].T for up to three projections into the same output, in one pass
    (cgpt_linear_forward_sum; the end of the reference's parallel-residual block is two projections and two adds)."""
    import ctypes as C
    n = len(inputs)
    _require(1 <= n <= 3 and len(weights) == n, "linear_forward_sum: 1..3 projections")
    _same_cuda_dtype("linear_forward_sum", output, *inputs, *weights, *([residual] if residual is not None else []))
    out_f = output.shape[-1]
    rows = output.numel() // out_f
    for x, w in zip(inputs, weights):
        _require(w.dim() == 2 and w.shape[0] == out_f and x.shape[-1] == w.shape[1] and x.numel() == rows * w.shape[1],
                 "linear_forward_sum: incompatible shapes")
    _require(residual is None or residual.shape == output.shape, "linear_forward_sum: residual must have the output's shape")
    xs = (C.c_void_p * n)(*[ptr(t) for t in inputs])
    ws = (C.c_void_p * n)(*[ptr(t) for t in weights])
    ins = (C.c_size_t * n)(*[w.shape[1] for w in weights])
    check(lib.cgpt_linear_forward_sum(ptr(output), xs, ws, ins, n, rows, out_f, ptr(residual) if residual is not None else None,
                                      dtype_code(output), stream_ptr(stream)), "linear_forward_sum")


def gemm(c, a, b, m, n, k, a_layout=0, b_layout=0, accumulate=False, force_simt=False, stream=None):
    """Raw contraction C[m,n] (+)= A B of the library (see cgpt_gemm in include/cgpt_b200.h)."""
    _same_cuda_dtype("gemm", c, a, b)
    check(lib.cgpt_gemm(ptr(c), ptr(a), ptr(b), m, n, k, a_layout, b_layout, int(accumulate), dtype_code(c),
                        int(force_simt), stream_ptr(stream)), "gemm")


# ------------------------------------------------------------------------------------------- Attention
@dataclass
class FlashAttentionOptions:
    """include/ops/attention.h:8-32 (key_tile_size, block_size and use_tensor_cores are accepted and
    ignored by the backward, as in the reference)."""
    num_query_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    attention_scale: float = 0.0
    causal: bool = True
    query_position_offset: int = 0
    key_tile_size: int = 16
    block_size: int = 128
    use_tensor_cores: bool = True


def _attn_check(name, q, k, v, o: FlashAttentionOptions, *same_as_q, same_as_k=()):
    _same_cuda_dtype(name, q, k, v, *same_as_q, *same_as_k)
    _require(q.dim() == 4 and k.dim() == 4 and v.shape == k.shape and all(t.shape == q.shape for t in same_as_q)
             and all(t.shape == k.shape for t in same_as_k), f"{name}: invalid gradient or operand shape")
    _require(o.num_query_heads > 0 and o.num_kv_heads > 0 and o.head_dim > 0
             and o.num_query_heads % o.num_kv_heads == 0 and q.shape[2] == o.num_query_heads
             and k.shape[2] == o.num_kv_heads and q.shape[3] == o.head_dim and k.shape[3] == o.head_dim
             and q.shape[0] == k.shape[0], f"{name}: invalid attention configuration")
    _require(o.attention_scale >= 0 and o.attention_scale == o.attention_scale
             and not (o.causal and o.query_position_offset + q.shape[1] > k.shape[1]),
             f"{name}: invalid scale or causal range")


def flash_gqa_attention_forward_with_lse(output, logsumexp, query, key, value, stream=None,
                                         options: FlashAttentionOptions | None = None, force_generic=False):
    """flash_gqa_attention_forward_with_lse (include/ops/attention.h:60-81)."""
    o = options or FlashAttentionOptions()
    _attn_check("flash_gqa_attention_forward", query, key, value, o, output)
    _require(logsumexp is None or (logsumexp.dtype == torch.float32 and logsumexp.is_cuda
                                   and tuple(logsumexp.shape) == tuple(query.shape[:3])),
             "flash_gqa_attention_forward: logsumexp must be F32 [batch, seq, heads]")
    b, sq, hq, d = query.shape
    check(lib.cgpt_attention_forward(ptr(output), ptr(logsumexp), ptr(query), ptr(key), ptr(value), b, sq, key.shape[1],
                                     hq, key.shape[2], d, float(o.attention_scale), int(o.causal),
                                     o.query_position_offset, dtype_code(query), int(force_generic),
                                     stream_ptr(stream)), "flash_gqa_attention_forward_with_lse")


def flash_gqa_attention_backward_with_lse(grad_query, grad_key, grad_value, grad_output, output, logsumexp, query,
                                          key, value, stream=None, options: FlashAttentionOptions | None = None,
                                          accumulate_grads=False, force_generic=False):
    """flash_gqa_attention_backward_with_lse (include/ops/backward/attention_backward.h:57-70)."""
    o = options or FlashAttentionOptions()
    _attn_check("flash_gqa_attention_backward", query, key, value, o, grad_query, grad_output, output,
                same_as_k=(grad_key, grad_value))
    _require(logsumexp.dtype == torch.float32 and tuple(logsumexp.shape) == tuple(query.shape[:3]),
             "flash_gqa_attention_backward: logsumexp must be F32 [batch, seq, heads]")
    b, sq, hq, d = query.shape
    check(lib.cgpt_attention_backward(ptr(grad_query), ptr(grad_key), ptr(grad_value), ptr(grad_output), ptr(output),
                                      ptr(logsumexp), ptr(query), ptr(key), ptr(value), b, sq, key.shape[1], hq,
                                      key.shape[2], d, float(o.attention_scale), int(o.causal),
                                      o.query_position_offset, int(accumulate_grads), dtype_code(query),
                                      int(force_generic), stream_ptr(stream)), "flash_gqa_attention_backward_with_lse")


def flash_gqa_attention_backward(grad_query, grad_key, grad_value, grad_output, query, key, value, stream=None,
                                 options: FlashAttentionOptions | None = None, accumulate_grads=False):
    """flash_gqa_attention_backward without saved statistics (attention_backward.h:24-35)."""
    o = options or FlashAttentionOptions()
    _attn_check("flash_gqa_attention_backward", query, key, value, o, grad_query, grad_output,
                same_as_k=(grad_key, grad_value))
    b, sq, hq, d = query.shape
    check(lib.cgpt_attention_backward(ptr(grad_query), ptr(grad_key), ptr(grad_value), ptr(grad_output), None, None,
                                      ptr(query), ptr(key), ptr(value), b, sq, key.shape[1], hq, key.shape[2], d,
                                      float(o.attention_scale), int(o.causal), o.query_position_offset,
                                      int(accumulate_grads), dtype_code(query), 1, stream_ptr(stream)),
          "flash_gqa_attention_backward")


# --------------------------------------------------------------------------------------------- RMSNorm
def rmsnorm_forward(output, input, weight, epsilon, stream=None):
    """rmsnorm_forward(Tensor& output, const Tensor& input, const Tensor& weight, float eps, stream)."""
    _same_cuda_dtype("rmsnorm_forward", output, input, weight)
    _require(input.dim() == 2 and output.shape == input.shape and weight.dim() == 1
             and weight.shape[0] == input.shape[1], "rmsnorm_forward: incompatible shapes")
    check(lib.cgpt_rmsnorm_forward(ptr(output), ptr(input), ptr(weight), input.shape[0], input.shape[1],
                                   float(epsilon), dtype_code(input), stream_ptr(stream)), "rmsnorm_forward")


def rmsnorm_backward(grad_input, grad_weight, grad_output, input, weight, epsilon, stream=None,
                     residual_a=None, residual_b=None):
    """rmsnorm_backward (include/ops/backward/rmsnorm_backward.h:21-29). ``residual_a/b`` are this
    library's extension: tensors added to grad_input inside the kernel."""
    extra = [t for t in (residual_a, residual_b) if t is not None]
    _same_cuda_dtype("rmsnorm_backward", grad_input, grad_weight, grad_output, input, weight, *extra)
    _require(input.dim() == 2 and grad_output.shape == input.shape and grad_input.shape == input.shape
             and weight.dim() == 1 and weight.shape[0] == input.shape[1] and grad_weight.shape == weight.shape
             and all(t.shape == input.shape for t in extra), "rmsnorm_backward: incompatible shapes")
    check(lib.cgpt_rmsnorm_backward(ptr(grad_input), ptr(grad_weight), ptr(grad_output), ptr(input), ptr(weight),
                                    ptr(residual_a), ptr(residual_b), input.shape[0], input.shape[1],
                                    float(epsilon), dtype_code(input), stream_ptr(stream)), "rmsnorm_backward")


def rmsnorm_forward_dual(output_a, output_b, input, weight_a, weight_b, epsilon, stream=None):
    """Both RMSNorms of a parallel-residual block's input in one pass over it (cgpt_rmsnorm_forward_dual)."""
    _same_cuda_dtype("rmsnorm_forward_dual", output_a, output_b, input, weight_a, weight_b)
    _require(input.dim() == 2 and output_a.shape == input.shape and output_b.shape == input.shape and weight_a.dim() == 1
             and weight_a.shape[0] == input.shape[1] and weight_b.shape == weight_a.shape, "rmsnorm_forward_dual: incompatible shapes")
    check(lib.cgpt_rmsnorm_forward_dual(ptr(output_a), ptr(output_b), ptr(input), ptr(weight_a), ptr(weight_b), input.shape[0],
                                        input.shape[1], float(epsilon), dtype_code(input), stream_ptr(stream)), "rmsnorm_forward_dual")


def rmsnorm_backward_dual(grad_input, grad_weight_a, grad_weight_b, grad_output_a, grad_output_b, input, weight_a, weight_b,
                          epsilon, residual=None, stream=None):
    """grad_input = residual + the input gradients of both norms of the same input, and both weight gradients, in one
    pass (cgpt_rmsnorm_backward_dual)."""
    extra = [residual] if residual is not None else []
    _same_cuda_dtype("rmsnorm_backward_dual", grad_input, grad_weight_a, grad_weight_b, grad_output_a, grad_output_b, input,
                     weight_a, weight_b, *extra)
    _require(input.dim() == 2 and all(t.shape == input.shape for t in (grad_input, grad_output_a, grad_output_b, *extra))
             and weight_a.dim() == 1 and weight_a.shape[0] == input.shape[1]
             and all(t.shape == weight_a.shape for t in (weight_b, grad_weight_a, grad_weight_b)),
             "rmsnorm_backward_dual: incompatible shapes")
    check(lib.cgpt_rmsnorm_backward_dual(ptr(grad_input), ptr(grad_weight_a), ptr(grad_weight_b), ptr(grad_output_a),
                                         ptr(grad_output_b), ptr(input), ptr(weight_a), ptr(weight_b), ptr(residual),
                                         input.shape[0], input.shape[1], float(epsilon), dtype_code(input), stream_ptr(stream)),
          "rmsnorm_backward_dual")


# ------------------------------------------------------------------------------------------------ RoPE
def _rope_dims(q, k, cos_cache, sin_cache, opts, name):
    _require(q.dim() == 4 and k.dim() == 4 and q.shape[0] == k.shape[0] and q.shape[1] == k.shape[1]
             and q.shape[3] == k.shape[3], f"{name}: query/key must be [batch, seq, heads, head_dim]")
    rotary = opts.rotary_dim or q.shape[3]
    _require(rotary <= q.shape[3] and rotary % 2 == 0, f"{name}: invalid rotary_dim")
    _require(cos_cache.dim() == 2 and sin_cache.shape == cos_cache.shape and cos_cache.shape[1] == rotary // 2,
             f"{name}: caches must be [max_seq, rotary_dim/2]")
    _require(opts.position_offset + q.shape[1] <= cos_cache.shape[0], f"{name}: position exceeds cache")
    return rotary


def rope_forward(query, key, cos_cache, sin_cache, stream=None, rope_options: RopeOptions | None = None):
    """rope_forward: rotates query and key in place (include/ops/rope.h:13-39)."""
    opts = rope_options or RopeOptions()
    _same_cuda_dtype("rope_forward", query, key, cos_cache, sin_cache)
    rotary = _rope_dims(query, key, cos_cache, sin_cache, opts, "rope_forward")
    b, s, hq, d = query.shape
    check(lib.cgpt_rope_forward(ptr(query), ptr(key), ptr(cos_cache), ptr(sin_cache), b, s, hq, key.shape[2], d,
                                rotary, opts.position_offset, cos_cache.shape[0], dtype_code(query),
                                stream_ptr(stream)), "rope_forward")


def rope_backward(grad_query, grad_key, grad_rotated_query, grad_rotated_key, cos_cache, sin_cache, stream=None,
                  rope_options: RopeOptions | None = None):
    """rope_backward (include/ops/backward/rope_backward.h:22-31)."""
    opts = rope_options or RopeOptions()
    _same_cuda_dtype("rope_backward", grad_query, grad_key, grad_rotated_query, grad_rotated_key, cos_cache,
                     sin_cache)
    _require(grad_query.shape == grad_rotated_query.shape and grad_key.shape == grad_rotated_key.shape,
             "rope_backward: gradient shapes differ")
    rotary = _rope_dims(grad_query, grad_key, cos_cache, sin_cache, opts, "rope_backward")
    b, s, hq, d = grad_query.shape
    check(lib.cgpt_rope_backward(ptr(grad_query), ptr(grad_key), ptr(grad_rotated_query), ptr(grad_rotated_key),
                                 ptr(cos_cache), ptr(sin_cache), b, s, hq, grad_key.shape[2], d, rotary,
                                 opts.position_offset, cos_cache.shape[0], dtype_code(grad_query),
                                 stream_ptr(stream)), "rope_backward")


# ---------------------------------------------------------------------------------------------- SwiGLU
def swiglu_forward(output, gate, up, stream=None):
    _same_cuda_dtype("swiglu_forward", output, gate, up)
    _require(output.shape == gate.shape == up.shape, "swiglu_forward: shapes differ")
    check(lib.cgpt_swiglu_forward(ptr(output), ptr(gate), ptr(up), gate.numel(), dtype_code(gate),
                                  stream_ptr(stream)), "swiglu_forward")


def swiglu_backward(grad_gate, grad_up, grad_output, gate, up, stream=None,
                    options: SwiGLUBackwardOptions | None = None):
    """swiglu_backward, separate gate/up layout (include/ops/backward/swiglu_backward.h:29-37)."""
    o = options or SwiGLUBackwardOptions()
    _same_cuda_dtype("swiglu_backward", grad_gate, grad_up, grad_output, gate, up)
    _require(grad_gate.shape == grad_up.shape == grad_output.shape == gate.shape == up.shape,
             "swiglu_backward: shapes differ")
    check(lib.cgpt_swiglu_backward(ptr(grad_gate), ptr(grad_up), ptr(grad_output), ptr(gate), ptr(up), gate.numel(),
                                   int(o.accumulate_gate), int(o.accumulate_up), dtype_code(gate),
                                   stream_ptr(stream)), "swiglu_backward")


# ------------------------------------------------------------------------------------------- Embedding
def embedding_forward(output, device_token_ids, token_count, weight, stream=None):
    _same_cuda_dtype("embedding_forward", output, weight)
    _ids(device_token_ids, token_count, "embedding_forward")
    _require(weight.dim() == 2 and output.numel() == token_count * weight.shape[1],
             "embedding_forward: output must hold token_count * hidden elements")
    check(lib.cgpt_embedding_forward(ptr(output), ptr(device_token_ids), ptr(weight), token_count, weight.shape[0],
                                     weight.shape[1], dtype_code(weight), stream_ptr(stream)), "embedding_forward")


def embedding_backward(grad_weight, grad_output, device_token_ids, token_count, stream=None,
                       options: EmbeddingBackwardOptions | None = None):
    """embedding_backward (include/ops/backward/embedding_backward.h:35-42)."""
    o = options or EmbeddingBackwardOptions()
    _same_cuda_dtype("embedding_backward", grad_weight, grad_output)
    _ids(device_token_ids, token_count, "embedding_backward")
    _require(grad_weight.dim() == 2 and grad_output.numel() == token_count * grad_weight.shape[1],
             "embedding_backward: grad_output must hold token_count * hidden elements")
    check(lib.cgpt_embedding_backward(ptr(grad_weight), ptr(grad_output), ptr(device_token_ids), token_count,
                                      grad_weight.shape[0], grad_weight.shape[1], int(o.bounds_check),
                                      int(o.accumulate_weight), dtype_code(grad_weight), stream_ptr(stream)),
          "embedding_backward")


# --------------------------------------------------------------------------------------- Residual adds
def add_tensors(output, a, b, stream=None, c=None):
    """add_tensors / add_inplace of src/core/transformer_block.cu:161-215,261-288 (output may alias a)."""
    extra = [c] if c is not None else []
    _same_cuda_dtype("add_tensors", output, a, b, *extra)
    _require(output.shape == a.shape == b.shape, "add_tensors: shapes differ")
    check(lib.cgpt_add(ptr(output), ptr(a), ptr(b), ptr(c), a.numel(), dtype_code(a), stream_ptr(stream)),
          "add_tensors")


# --------------------------------------------------------------------------------------- Cross entropy
def _ce_check(loss, logits, targets, target_count, name):
    _require(loss.is_cuda and loss.dtype == torch.float32 and tuple(loss.shape) == (1,),
             f"{name}: loss must be a CUDA F32 tensor with shape [1]")
    _require(logits.is_cuda and logits.dim() == 2 and logits.shape[0] > 0 and logits.shape[1] > 0,
             f"{name}: logits must be a non-empty CUDA matrix")
    _require(target_count == logits.shape[0], f"{name}: target count must equal logits rows")
    _ids(targets, target_count, name)


def cross_entropy_forward_backward(loss, gradient, logits, device_targets, target_count, stream=None,
                                   gradient_scale: float = 1.0):
    """cross_entropy_forward_backward (include/ops/cross_entropy.h:25-32)."""
    _ce_check(loss, logits, device_targets, target_count, "cross_entropy")
    _same_cuda_dtype("cross_entropy", gradient, logits)
    _require(gradient.shape == logits.shape, "cross_entropy: gradient shape must match logits")
    check(lib.cgpt_cross_entropy(ptr(loss), ptr(gradient), ptr(logits), ptr(device_targets), logits.shape[0],
                                 logits.shape[1], float(gradient_scale), dtype_code(logits), stream_ptr(stream)),
          "cross_entropy_forward_backward")


def cross_entropy_forward(loss, logits, device_targets, target_count, stream=None):
    """cross_entropy_forward (include/ops/cross_entropy.h:37-42)."""
    _ce_check(loss, logits, device_targets, target_count, "cross_entropy")
    check(lib.cgpt_cross_entropy(ptr(loss), None, ptr(logits), ptr(device_targets), logits.shape[0], logits.shape[1],
                                 1.0, dtype_code(logits), stream_ptr(stream)), "cross_entropy_forward")
