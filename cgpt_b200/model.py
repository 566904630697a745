"""Host-side mirror of CGPT's transformer block / model API for the training step.

Names and argument order follow ``include/core/transformer_block.h`` and ``include/core/transformer_model.h``
of the reference; tensors are ``torch`` CUDA tensors used as device-memory handles and all work happens in
``libcgpt_b200.so`` (``cgpt_block_*`` / ``cgpt_model_*`` of the C ABI). ``cut_cross_entropy_forward_backward``
mirrors ``include/ops/cut_cross_entropy.h`` with two extensions (16-bit tensors, ``gradient_scale``).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field

import torch

from . import _lib
from ._lib import (BLOCK_PARAM_FIELDS, BLOCK_SAVED_FIELDS, BlockParams, BlockSaved, ModelConfig, ModelSaved,
                   ModelTensors, check, dtype_code, lib, ptr, stream_ptr)


@dataclass
class TransformerBlockOptions:
    """include/core/transformer_block.h:10-31."""
    hidden_size: int = 0
    intermediate_size: int = 0
    num_query_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    rotary_dim: int = 0
    rms_epsilon: float = 1.0e-5
    causal: bool = True


@dataclass
class TransformerModelOptions:
    """include/core/transformer_model.h:20-27."""
    vocabulary_size: int = 0
    num_layers: int = 0
    block_options: TransformerBlockOptions = field(default_factory=TransformerBlockOptions)


def preset(name: str, vocabulary_size: int = 32000) -> TransformerModelOptions:
    """Model presets of the reference trainer (train/train.cpp:140-149) plus the tiny CPU-runnable model and a 1.3B one."""
    if name == "104m":
        b = TransformerBlockOptions(1024, 2048, 8, 2, 128, 128)
        return TransformerModelOptions(vocabulary_size, 8, b)
    if name == "small":
        return TransformerModelOptions(vocabulary_size, 4, TransformerBlockOptions(512, 1024, 4, 1, 128, 128))
    if name == "1.3b":   # the scaled-up configuration: 24 layers, d 2048, 16/4 heads of 128, SwiGLU 5632
        return TransformerModelOptions(vocabulary_size, 24, TransformerBlockOptions(2048, 5632, 16, 4, 128, 128))
    if name == "tiny":
        return TransformerModelOptions(vocabulary_size, 2, TransformerBlockOptions(256, 688, 4, 2, 64, 64))
    raise ValueError(f"unknown preset {name}")


def _validate_block(o: TransformerBlockOptions) -> None:
    """validate_options of src/core/transformer_block.cu (raises like std::invalid_argument)."""
    ok = (o.hidden_size > 0 and o.intermediate_size > 0 and o.num_query_heads > 0 and o.num_kv_heads > 0
          and o.head_dim > 0 and o.num_query_heads % o.num_kv_heads == 0
          and o.num_query_heads * o.head_dim == o.hidden_size and o.rotary_dim <= o.head_dim
          and o.rotary_dim % 2 == 0 and o.rms_epsilon > 0)
    if not ok:
        raise _lib.CgptInvalidArgument("transformer block: invalid options")


def _config(opts: TransformerModelOptions, dtype: torch.dtype, max_seq: int, tied: bool) -> ModelConfig:
    b = opts.block_options
    return ModelConfig(opts.vocabulary_size, opts.num_layers, b.hidden_size, b.intermediate_size, b.num_query_heads,
                       b.num_kv_heads, b.head_dim, b.rotary_dim or b.head_dim, max_seq, b.rms_epsilon,
                       _lib._TORCH_TO_CODE[dtype], int(tied), 0)


def block_param_shapes(o: TransformerBlockOptions) -> dict:
    """Shapes of the 11 parameter tensors of a block (include/core/transformer_block.h:36-47)."""
    d, i, q, kv, hd = o.hidden_size, o.intermediate_size, o.num_query_heads * o.head_dim, o.num_kv_heads * o.head_dim, o.head_dim
    return {"attention_norm": (d,), "q_projection": (q, d), "k_projection": (kv, d), "q_norm": (hd,), "k_norm": (hd,),
            "v_projection": (kv, d), "o_projection": (d, q), "ffn_norm": (d,), "gate_proj": (i, d), "up_proj": (i, d),
            "down_proj": (d, i)}


class TransformerBlockWorkspace:
    """Activations saved by the forward (include/core/transformer_block.h:65-93)."""

    def __init__(self, options: TransformerBlockOptions, batch: int, seq: int, dtype=torch.float16, device="cuda",
                 save_attention_norm: bool = True):
        o = options
        rows = batch * seq
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        self.norm = e(rows, o.hidden_size)
        self.query = e(batch, seq, o.num_query_heads, o.head_dim)
        self.key = e(batch, seq, o.num_kv_heads, o.head_dim)
        self.value = e(batch, seq, o.num_kv_heads, o.head_dim)
        self.query_pre_norm = e(batch, seq, o.num_query_heads, o.head_dim)
        self.key_pre_norm = e(batch, seq, o.num_kv_heads, o.head_dim)
        self.attention_output = e(batch, seq, o.num_query_heads, o.head_dim)
        self.attention_logsumexp = torch.empty(batch, seq, o.num_query_heads, dtype=torch.float32, device=device)
        self.gate = e(rows, o.intermediate_size)
        self.up = e(rows, o.intermediate_size)
        self.activated = e(rows, o.intermediate_size)
        # not in the reference's workspace (it recomputes the attention norm in the backward): rows*hidden elements
        # per layer buy one RMSNorm pass per layer; None restores the recomputation
        self.attention_norm_output = e(rows, o.hidden_size) if save_attention_norm else None
        self.batch, self.seq = batch, seq

    def c_struct(self) -> BlockSaved:
        return BlockSaved(*[(getattr(self, n).data_ptr() if getattr(self, n) is not None else None) for n in BLOCK_SAVED_FIELDS])


class TransformerBlockBackwardWorkspace:
    """Scratch of the block forward/backward; one buffer of cgpt_block_workspace_bytes() bytes serves every
    layer (the reference allocates 17 tensors per layer, include/core/transformer_block.h:126-171)."""

    def __init__(self, cfg: ModelConfig, batch: int, seq: int, device="cuda"):
        nbytes = int(lib.cgpt_block_workspace_bytes(C.byref(cfg), batch, seq))
        if nbytes == 0:
            raise _lib.CgptInvalidArgument("transformer block: invalid configuration")
        self.buffer = torch.empty(nbytes, dtype=torch.uint8, device=device)


def _params_struct(tensors: dict) -> BlockParams:
    return BlockParams(*[tensors[n].data_ptr() for n in BLOCK_PARAM_FIELDS])


def _check_block_tensors(tensors: dict, o: TransformerBlockOptions, dtype, what: str) -> None:
    for name, shape in block_param_shapes(o).items():
        t = tensors[name]
        if not (t.is_cuda and t.dtype == dtype and tuple(t.shape) == shape and t.is_contiguous()):
            raise _lib.CgptInvalidArgument(f"transformer block: {what}.{name} must be a contiguous CUDA {dtype} tensor of shape {shape}")


def transformer_block_forward(output, input, weights: dict, workspace: TransformerBlockWorkspace, cos_cache, sin_cache,
                              cublas_context, stream, options: TransformerBlockOptions, position_offset: int = 0,
                              scratch: TransformerBlockBackwardWorkspace | None = None):
    """transformer_block_forward (include/core/transformer_block.h:182-196), training path (no KV cache)."""
    _validate_block(options)
    if input.dim() != 2 or output.shape != input.shape or input.shape[1] != options.hidden_size:
        raise _lib.CgptInvalidArgument("transformer block input/output must be [batch * sequence, hidden]")
    if workspace.batch * workspace.seq != input.shape[0]:
        raise _lib.CgptInvalidArgument("workspace batch * sequence must be equal input rows")
    _check_block_tensors(weights, options, input.dtype, "weights")
    cfg = _config(TransformerModelOptions(1, 1, options), input.dtype, cos_cache.shape[0], False)
    scratch = scratch or TransformerBlockBackwardWorkspace(cfg, workspace.batch, workspace.seq)
    w, sv = _params_struct(weights), workspace.c_struct()
    check(lib.cgpt_block_forward(ptr(output), ptr(input), C.byref(w), C.byref(sv), scratch.buffer.data_ptr(),
                                 ptr(cos_cache), ptr(sin_cache), C.byref(cfg), workspace.batch, workspace.seq,
                                 position_offset, stream_ptr(stream)), "transformer_block_forward")


def transformer_block_backward(grad_input, grad_output, input, weights: dict, gradients: dict,
                               forward_workspace: TransformerBlockWorkspace,
                               backward_workspace: TransformerBlockBackwardWorkspace, cos_cache, sin_cache,
                               cublas_context, stream, options: TransformerBlockOptions, position_offset: int = 0):
    """transformer_block_backward (include/core/transformer_block.h:229-242)."""
    _validate_block(options)
    if (input.dim() != 2 or grad_output.shape != input.shape or grad_input.shape != input.shape
            or input.dtype != grad_output.dtype or input.dtype != grad_input.dtype or not input.is_cuda):
        raise _lib.CgptInvalidArgument("transformer block backward: invalid input or output gradient")
    if input.shape[1] != options.hidden_size or forward_workspace.batch * forward_workspace.seq != input.shape[0]:
        raise _lib.CgptInvalidArgument("transformer block backward: forward workspace does not match input")
    _check_block_tensors(weights, options, input.dtype, "weights")
    _check_block_tensors(gradients, options, input.dtype, "gradients")
    cfg = _config(TransformerModelOptions(1, 1, options), input.dtype, cos_cache.shape[0], False)
    w, g, sv = _params_struct(weights), _params_struct(gradients), forward_workspace.c_struct()
    check(lib.cgpt_block_backward(ptr(grad_input), ptr(grad_output), ptr(input), C.byref(w), C.byref(g), C.byref(sv),
                                  backward_workspace.buffer.data_ptr(), ptr(cos_cache), ptr(sin_cache), C.byref(cfg),
                                  forward_workspace.batch, forward_workspace.seq, position_offset, stream_ptr(stream)),
          "transformer_block_backward")


def cut_cross_entropy_forward_backward(loss, input_gradient, classifier_gradient, input, classifier, device_targets,
                                       target_count, stream=None, gradient_scale: float = 1.0,
                                       accumulate_classifier_gradient: bool = False, chunk_rows: int = 0, form: int = 0):
    """cut_cross_entropy_forward_backward (include/ops/cut_cross_entropy.h:25-33); F32, F16 or BF16.
    form: 0 = the library's default, 1 = row kernel over stored logits, 2 = tile statistics from the logits product's
    epilogue + one streaming gradient pass, 3 = logits never stored (recomputed; gradient written by the epilogue)."""
    ts = (input_gradient, classifier_gradient, input, classifier)
    if any((not t.is_cuda) or t.dtype != input.dtype or not t.is_contiguous() for t in ts) or input.dim() != 2 \
            or classifier.dim() != 2 or classifier.shape[1] != input.shape[1]:
        raise _lib.CgptInvalidArgument("cut_cross_entropy: input and classifier must be non-empty CUDA matrices of one dtype")
    if target_count != input.shape[0] or input_gradient.shape != input.shape or classifier_gradient.shape != classifier.shape:
        raise _lib.CgptInvalidArgument("cut_cross_entropy: incompatible gradient or target count")
    if not (loss.is_cuda and loss.dtype == torch.float32 and tuple(loss.shape) == (1,)):
        raise _lib.CgptInvalidArgument("cut_cross_entropy: loss must be a CUDA F32 tensor with shape [1]")
    check(lib.cgpt_cut_cross_entropy_form(int(form), ptr(loss), ptr(input_gradient), ptr(classifier_gradient), ptr(input),
                                          ptr(classifier), ptr(device_targets), input.shape[0], classifier.shape[0],
                                          input.shape[1], float(gradient_scale), int(accumulate_classifier_gradient),
                                          chunk_rows, dtype_code(input), stream_ptr(stream)),
          "cut_cross_entropy_forward_backward")


class ModelStorage:
    """Weights and gradients of the whole model, tied embedding / LM head by default (the trainer's
    ModelStorage, train/train.cpp:251-300). Weights are N(0, std) from a seeded torch generator, output
    projections (o, down) use std / sqrt(2 * layers), norms are 1 (src/core/weight_initialization.cu:158-179
    uses the same scheme with a host mt19937_64 stream)."""

    def __init__(self, options: TransformerModelOptions, dtype=torch.float16, seed: int = 0, std: float = 0.02,
                 tied: bool = True, device="cuda"):
        self.options, self.dtype, self.tied = options, dtype, tied
        b = options.block_options
        _validate_block(b)
        gen = torch.Generator(device="cpu").manual_seed(seed)

        def normal(shape, s):
            return (torch.randn(shape, generator=gen, dtype=torch.float32) * s).to(device=device, dtype=dtype)

        out_std = std / math.sqrt(2.0 * options.num_layers)
        self.token_embedding = normal((options.vocabulary_size, b.hidden_size), std)
        self.lm_head = self.token_embedding if tied else normal((options.vocabulary_size, b.hidden_size), std)
        self.final_norm = torch.ones(b.hidden_size, dtype=dtype, device=device)
        self.layers = []
        for _ in range(options.num_layers):
            layer = {}
            for name, shape in block_param_shapes(b).items():
                if name.endswith("norm"):
                    layer[name] = torch.ones(shape, dtype=dtype, device=device)
                else:
                    layer[name] = normal(shape, out_std if name in ("o_projection", "down_proj") else std)
            self.layers.append(layer)
        # Gradients live in ONE flat buffer, laid out in the order the backward finishes them (final norm,
        # last layer ... first layer, embedding last), so data-parallel all-reduce works on contiguous
        # buckets of it. Every tensor starts on a 256-byte boundary.
        order = [("final_norm", self.final_norm)]
        for li in reversed(range(options.num_layers)):
            for n in reversed(BLOCK_PARAM_FIELDS):
                order.append((f"layers.{li}.{n}", self.layers[li][n]))
        if not tied:
            order.append(("lm_head", self.lm_head))
        order.append(("token_embedding", self.token_embedding))
        align = 256 // self.token_embedding.element_size()
        offsets, total = {}, 0
        for name, t in order:
            offsets[name] = total
            total += (t.numel() + align - 1) // align * align
        self.flat_gradients = torch.zeros(total, dtype=dtype, device=device)
        self.gradient_offsets = offsets
        view = lambda name, t: self.flat_gradients[offsets[name]:offsets[name] + t.numel()].view(t.shape)
        self.g_token_embedding = view("token_embedding", self.token_embedding)
        self.g_lm_head = self.g_token_embedding if tied else view("lm_head", self.lm_head)
        self.g_final_norm = view("final_norm", self.final_norm)
        self.g_layers = [{n: view(f"layers.{li}.{n}", t) for n, t in layer.items()} for li, layer in enumerate(self.layers)]

    def final_gradient_elements(self, steps_done: int) -> int:
        """Elements at the start of ``flat_gradients`` that are final once the backward has run steps
        0 .. steps_done-1 (0 = final norm, 1..layers = blocks from the last to the first, layers+1 = embedding).
        The buffer is laid out in exactly that order; with tied embeddings the LM-head gradient shares the
        embedding's slot and only becomes final with the last step."""
        L = self.options.num_layers
        if steps_done <= 0:
            return 0
        if steps_done >= L + 2:
            return self.flat_gradients.numel()
        if steps_done == L + 1:
            # all blocks done; an untied LM-head gradient was already complete before the backward started
            return self.gradient_offsets["token_embedding"]
        # steps 0 .. steps_done-1 finished the final norm and blocks L-1 .. L-steps_done+1: the next block's first
        # tensor (the layout lists a block's tensors in reverse field order) is where the final prefix ends
        return self.gradient_offsets[f"layers.{L - steps_done}.{BLOCK_PARAM_FIELDS[-1]}"]

    def parameters_and_gradients(self):
        """(parameter, gradient) pairs in the trainer's order (train/train.cpp:302-320)."""
        pairs = [(self.token_embedding, self.g_token_embedding)]
        if not self.tied:
            pairs.append((self.lm_head, self.g_lm_head))
        pairs.append((self.final_norm, self.g_final_norm))
        for layer, grads in zip(self.layers, self.g_layers):
            pairs += [(layer[n], grads[n]) for n in BLOCK_PARAM_FIELDS]
        return pairs

    def num_parameters(self) -> int:
        return sum(p.numel() for p, _ in self.parameters_and_gradients())


class TransformerModelWorkspace:
    """Saved activations of the forward for every layer (include/core/transformer_model.h:44-62)."""

    def __init__(self, options: TransformerModelOptions, batch: int, seq: int, dtype=torch.float16, device="cuda"):
        b = options.block_options
        rows = batch * seq
        self.batch, self.seq = batch, seq
        self.layers = [TransformerBlockWorkspace(b, batch, seq, dtype, device) for _ in range(options.num_layers)]
        self.layer_inputs = [torch.empty(rows, b.hidden_size, dtype=dtype, device=device) for _ in range(options.num_layers)]
        self.hidden = torch.empty(rows, b.hidden_size, dtype=dtype, device=device)
        self.normalized = torch.empty(rows, b.hidden_size, dtype=dtype, device=device)
        self._saved_arr = (BlockSaved * options.num_layers)(*[l.c_struct() for l in self.layers])
        self._inputs_arr = (C.c_void_p * options.num_layers)(*[t.data_ptr() for t in self.layer_inputs])
        self.c = ModelSaved(self._saved_arr, self._inputs_arr, self.hidden.data_ptr(), self.normalized.data_ptr())


class TransformerModelBackwardWorkspace:
    """Scratch of the model backward: the block scratch (shared by all layers), two ping-pong hidden-gradient
    buffers inside it, and grad_normalized (include/core/transformer_model.h:84-109)."""

    def __init__(self, options: TransformerModelOptions, batch: int, seq: int, dtype=torch.float16, device="cuda",
                 max_seq: int | None = None):
        self.cfg = _config(options, dtype, max_seq or seq, True)
        self.block = TransformerBlockBackwardWorkspace(self.cfg, batch, seq, device)
        self.grad_normalized = torch.empty(batch * seq, options.block_options.hidden_size, dtype=dtype, device=device)


def _model_structs(storage: ModelStorage):
    w_arr = (BlockParams * len(storage.layers))(*[_params_struct(l) for l in storage.layers])
    g_arr = (BlockParams * len(storage.layers))(*[_params_struct(l) for l in storage.g_layers])
    w = ModelTensors(storage.token_embedding.data_ptr(), w_arr, storage.final_norm.data_ptr(), storage.lm_head.data_ptr())
    g = ModelTensors(storage.g_token_embedding.data_ptr(), g_arr, storage.g_final_norm.data_ptr(), storage.g_lm_head.data_ptr())
    return w, g, (w_arr, g_arr)


def transformer_model_forward(logits, device_token_ids, batch_size, sequence_length, storage: ModelStorage,
                              workspace: TransformerModelWorkspace, cos_cache, sin_cache, cublas_context, stream,
                              options: TransformerModelOptions, scratch: TransformerModelBackwardWorkspace | None = None):
    """transformer_model_forward (include/core/transformer_model.h:111-131). ``logits=None`` stops after the
    final RMSNorm (``workspace.normalized``), for the cut-cross-entropy loss."""
    if device_token_ids is None or batch_size == 0 or sequence_length == 0:
        raise _lib.CgptInvalidArgument("transformer model requires token IDs and positive batch/sequence dimensions")
    if len(storage.layers) != options.num_layers or len(workspace.layers) != options.num_layers:
        raise _lib.CgptInvalidArgument("transformer model weights/workspace layer count mismatch")
    rows = batch_size * sequence_length
    if logits is not None and (tuple(logits.shape) != (rows, options.vocabulary_size) or logits.dtype != storage.dtype):
        raise _lib.CgptInvalidArgument("transformer model: logits must be [rows, vocabulary]")
    scratch = scratch or TransformerModelBackwardWorkspace(options, batch_size, sequence_length, storage.dtype, max_seq=cos_cache.shape[0])
    cfg = _config(options, storage.dtype, cos_cache.shape[0], storage.tied)
    w, _, keep = _model_structs(storage)
    check(lib.cgpt_model_forward(ptr(logits), ptr(device_token_ids), C.byref(w), C.byref(workspace.c),
                                 scratch.block.buffer.data_ptr(), ptr(cos_cache), ptr(sin_cache), C.byref(cfg), batch_size,
                                 sequence_length, stream_ptr(stream)), "transformer_model_forward")
    return keep


def transformer_model_backward(grad_logits, device_token_ids, batch_size, sequence_length, storage: ModelStorage,
                               forward_workspace: TransformerModelWorkspace,
                               backward_workspace: TransformerModelBackwardWorkspace, cos_cache, sin_cache,
                               cublas_context, stream, options: TransformerModelOptions,
                               steps: tuple[int, int] | None = None):
    """transformer_model_backward (include/core/transformer_model.h:176-190). ``grad_logits=None`` starts from
    ``backward_workspace.grad_normalized`` (already written by the cut-cross-entropy loss together with the
    LM-head gradient). ``steps=(begin, end)`` runs only that range of the backward's steps (0 = final norm,
    1..layers = blocks from last to first, layers+1 = embedding), for drivers that start reducing finished
    gradients in between; the default runs all of them."""
    if device_token_ids is None or batch_size == 0 or sequence_length == 0 or len(storage.g_layers) != options.num_layers:
        raise _lib.CgptInvalidArgument("transformer model backward: invalid model state or token IDs")
    rows = batch_size * sequence_length
    if grad_logits is not None and (tuple(grad_logits.shape) != (rows, options.vocabulary_size) or grad_logits.dtype != storage.dtype):
        raise _lib.CgptInvalidArgument("transformer model backward: invalid logits gradient or workspace shape")
    cfg = _config(options, storage.dtype, cos_cache.shape[0], storage.tied)
    w, g, keep = _model_structs(storage)
    begin, end = steps if steps is not None else (0, options.num_layers + 2)
    check(lib.cgpt_model_backward_steps(ptr(grad_logits), ptr(backward_workspace.grad_normalized), ptr(device_token_ids),
                                        C.byref(w), C.byref(g), C.byref(forward_workspace.c),
                                        backward_workspace.block.buffer.data_ptr(), ptr(cos_cache), ptr(sin_cache),
                                        C.byref(cfg), batch_size, sequence_length, begin, end, stream_ptr(stream)),
          "transformer_model_backward")
    return keep


def rotary_cache(sequence_length: int, rotary_dim: int, dtype=torch.float16, device="cuda"):
    """cos/sin tables [sequence_length, rotary_dim/2] as the trainer builds them (train/train.cpp:322-333):
    theta = pos / 10000^(2i/rotary_dim) in fp32, then stored in `dtype`."""
    pos = torch.arange(sequence_length, dtype=torch.float32)[:, None]
    i = torch.arange(rotary_dim // 2, dtype=torch.float32)[None, :]
    theta = pos / torch.pow(torch.tensor(10000.0), 2.0 * i / float(rotary_dim))
    return torch.cos(theta).to(device=device, dtype=dtype), torch.sin(theta).to(device=device, dtype=dtype)
