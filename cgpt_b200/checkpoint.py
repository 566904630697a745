"""Checkpoints: model weights in the reference's safetensors layout plus the optimizer state the reference drops.

`model.safetensors` uses the tensor names and dtypes of the reference's exporter
(src/core/huggingface_export.cpp:361-380: model.embed_tokens.weight, model.norm.weight, lm_head.weight,
model.layers.N.{input_layernorm, self_attn.{q,k,v,o}_proj, self_attn.{q,k}_norm, post_attention_layernorm,
mlp.{gate,up,down}_proj}.weight), so a directory written here loads with the reference's `--load-dir`
(train/train.cpp:428-432) and vice versa. The reference resumes AdamW from zero moments and step 0;
`optimizer.safetensors` (fp32 master weights, first and second moments under the same names, and the step count)
closes that gap.
"""
from __future__ import annotations

import json
import os

import torch
from safetensors.torch import load_file, save_file

# our block field -> name below "model.layers.N."
_BLOCK_NAMES = {
    "attention_norm": "input_layernorm.weight",
    "q_projection": "self_attn.q_proj.weight",
    "k_projection": "self_attn.k_proj.weight",
    "q_norm": "self_attn.q_norm.weight",
    "k_norm": "self_attn.k_norm.weight",
    "v_projection": "self_attn.v_proj.weight",
    "o_projection": "self_attn.o_proj.weight",
    "ffn_norm": "post_attention_layernorm.weight",
    "gate_proj": "mlp.gate_proj.weight",
    "up_proj": "mlp.up_proj.weight",
    "down_proj": "mlp.down_proj.weight",
}


def named_parameters(storage) -> list[tuple[str, torch.Tensor]]:
    """(reference tensor name, parameter) in the trainer's parameter order (train/train.cpp:302-320)."""
    out = [("model.embed_tokens.weight", storage.token_embedding)]
    if not storage.tied:
        out.append(("lm_head.weight", storage.lm_head))
    out.append(("model.norm.weight", storage.final_norm))
    for i, layer in enumerate(storage.layers):
        for field, tensor in layer.items():
            out.append((f"model.layers.{i}.{_BLOCK_NAMES[field]}", tensor))
    return out


def save_model(directory: str, storage) -> str:
    """Writes model.safetensors. A tied LM head is written as its own tensor, as the reference does."""
    os.makedirs(directory, exist_ok=True)
    tensors = {name: t.detach().cpu().contiguous() for name, t in named_parameters(storage)}
    if storage.tied:
        tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    path = os.path.join(directory, "model.safetensors")
    save_file(tensors, path)
    return path


def load_model(directory: str, storage) -> None:
    """Copies model.safetensors into the allocated parameters; names, shapes and dtypes must match."""
    tensors = load_file(os.path.join(directory, "model.safetensors"))
    for name, dst in named_parameters(storage):
        if name not in tensors:
            raise KeyError(f"Tensor missing from safetensors: {name}")
        src = tensors[name]
        if tuple(src.shape) != tuple(dst.shape) or src.dtype != dst.dtype:
            raise ValueError(f"{name}: checkpoint has {tuple(src.shape)} {src.dtype}, model has {tuple(dst.shape)} {dst.dtype}")
        dst.copy_(src)


def save_optimizer(directory: str, storage, states, extra: dict | None = None) -> str:
    """Writes optimizer.safetensors: `<name>.master`, `<name>.m`, `<name>.v` (fp32) and the step counts."""
    os.makedirs(directory, exist_ok=True)
    names = [n for n, _ in named_parameters(storage)]
    if len(names) != len(states):
        raise ValueError("one optimizer state per parameter expected")
    tensors, steps = {}, {}
    for name, st in zip(names, states):
        tensors[name + ".master"] = st.master_parameter.detach().cpu().contiguous()
        tensors[name + ".m"] = st.first_moment.detach().cpu().contiguous()
        tensors[name + ".v"] = st.second_moment.detach().cpu().contiguous()
        steps[name] = int(st.step)
    meta = {"steps": json.dumps(steps), "extra": json.dumps(extra or {})}
    path = os.path.join(directory, "optimizer.safetensors")
    save_file(tensors, path, metadata=meta)
    return path


def load_optimizer(directory: str, storage, states) -> dict:
    """Restores master weights, moments and step counts in place; returns the `extra` dictionary saved with them."""
    from safetensors import safe_open
    path = os.path.join(directory, "optimizer.safetensors")
    names = [n for n, _ in named_parameters(storage)]
    with safe_open(path, framework="pt") as f:
        meta = f.metadata() or {}
        steps = json.loads(meta.get("steps", "{}"))
        for name, st in zip(names, states):
            for suffix, dst in ((".master", st.master_parameter), (".m", st.first_moment), (".v", st.second_moment)):
                src = f.get_tensor(name + suffix)
                if tuple(src.shape) != tuple(dst.shape):
                    raise ValueError(f"{name}{suffix}: shape {tuple(src.shape)} != {tuple(dst.shape)}")
                dst.copy_(src)
            st.step = int(steps.get(name, 0))
    return json.loads(meta.get("extra", "{}"))


def has_optimizer(directory: str) -> bool:
    return os.path.exists(os.path.join(directory, "optimizer.safetensors"))
