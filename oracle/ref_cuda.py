"""ctypes access to oracle/_ref/libcgpt_ref_cuda.so: the reference's own CUDA operators rebuilt for sm_100a
(TEST INFRASTRUCTURE; built by oracle/build_ref.py from the sources under the reference checkout, wrapper
oracle/ref_wrap_cuda.cpp). Every function takes torch CUDA tensors and runs one reference entry point on torch's
current stream."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libcgpt_ref_cuda.so"
_DT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
_lib = None


def available() -> bool:
    return LIB_PATH.exists()


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(LIB_PATH))
        _lib.ref_cuda_last_error.restype = C.c_char_p
    return _lib


def _p(t):
    return C.c_void_p(t.data_ptr())


def _s():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _z(*v):
    return [C.c_size_t(int(x)) for x in v]


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: {lib().ref_cuda_last_error().decode()}")


def rmsnorm_forward(y, x, w, eps):
    _check(lib().ref_cuda_rmsnorm_forward(_p(y), _p(x), _p(w), *_z(*x.shape), C.c_float(eps), _DT[x.dtype], _s()), "rmsnorm_forward")


def rmsnorm_backward(dx, dw, dy, x, w, eps):
    _check(lib().ref_cuda_rmsnorm_backward(_p(dx), _p(dw), _p(dy), _p(x), _p(w), *_z(*x.shape), C.c_float(eps), _DT[x.dtype], _s()),
           "rmsnorm_backward")


def rope_forward(q, k, cos, sin, rotary=0, offset=0):
    b, s, hq, d = q.shape
    _check(lib().ref_cuda_rope_forward(_p(q), _p(k), _p(cos), _p(sin), *_z(b, s, hq, k.shape[2], d, rotary, offset, cos.shape[0]),
                                       _DT[q.dtype], _s()), "rope_forward")


def rope_backward(dq, dk, dq_rot, dk_rot, cos, sin, rotary=0, offset=0):
    b, s, hq, d = dq.shape
    _check(lib().ref_cuda_rope_backward(_p(dq), _p(dk), _p(dq_rot), _p(dk_rot), _p(cos), _p(sin),
                                        *_z(b, s, hq, dk.shape[2], d, rotary, offset, cos.shape[0]), _DT[dq.dtype], _s()), "rope_backward")


def swiglu_forward(y, gate, up):
    _check(lib().ref_cuda_swiglu_forward(_p(y), _p(gate), _p(up), *_z(*gate.shape), _DT[gate.dtype], _s()), "swiglu_forward")


def swiglu_backward(dgate, dup, dy, gate, up):
    _check(lib().ref_cuda_swiglu_backward(_p(dgate), _p(dup), _p(dy), _p(gate), _p(up), *_z(*gate.shape), _DT[gate.dtype], _s()),
           "swiglu_backward")


def embedding_backward(gw, dy, ids, accumulate):
    _check(lib().ref_cuda_embedding_backward(_p(gw), _p(dy), _p(ids), *_z(ids.numel(), gw.shape[0], gw.shape[1]), int(accumulate),
                                             _DT[gw.dtype], _s()), "embedding_backward")


def cross_entropy(loss, grad, logits, targets, gradient_scale):
    _check(lib().ref_cuda_cross_entropy(_p(loss), _p(grad), _p(logits), _p(targets), *_z(*logits.shape), C.c_float(gradient_scale),
                                        _DT[logits.dtype], _s()), "cross_entropy")


def cut_cross_entropy(loss, gx, gc, x, c, targets):
    _check(lib().ref_cuda_cut_cross_entropy(_p(loss), _p(gx), _p(gc), _p(x), _p(c), _p(targets), *_z(x.shape[0], c.shape[0], x.shape[1]),
                                            _DT[x.dtype], _s()), "cut_cross_entropy")


def attention_forward(out, lse, q, k, v, causal=True, offset=0, scale=0.0):
    b, sq, hq, d = q.shape
    _check(lib().ref_cuda_attention_forward(_p(out), _p(lse), _p(q), _p(k), _p(v), *_z(b, sq, k.shape[1], hq, k.shape[2], d), int(causal),
                                            C.c_size_t(offset), C.c_float(scale), _DT[q.dtype], _s()), "attention_forward")


def attention_backward(dq, dk, dv, dout, out, lse, q, k, v, causal=True, offset=0, scale=0.0):
    b, sq, hq, d = q.shape
    _check(lib().ref_cuda_attention_backward(_p(dq), _p(dk), _p(dv), _p(dout), _p(out), _p(lse), _p(q), _p(k), _p(v),
                                             *_z(b, sq, k.shape[1], hq, k.shape[2], d), int(causal), C.c_size_t(offset), C.c_float(scale),
                                             _DT[q.dtype], _s()), "attention_backward")


# ------------------------------------------------------------------------------------------------------------------
# The reference's block / model / optimizer (oracle/ref_wrap_model.cpp): its trainer's tensors and its trainer's step.
BLOCK_FIELDS = ("attention_norm", "q_projection", "k_projection", "q_norm", "k_norm", "v_projection", "o_projection",
                "ffn_norm", "gate_proj", "up_proj", "down_proj")


def _mcheck(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: {lib().ref_model_last_error().decode()}")


def _view(ptr: int, numel: int, dtype) -> torch.Tensor:
    """A torch tensor over device memory owned by the reference library (no copy, no ownership)."""
    esize = torch.empty(0, dtype=dtype).element_size()

    class _Mem:
        __cuda_array_interface__ = {"shape": (numel,), "typestr": {2: "<f2", 4: "<f4"}[esize], "data": (ptr, False), "version": 2}

    t = torch.as_tensor(_Mem(), device="cuda")
    return t.view(dtype) if t.dtype != dtype else t


class RefModel:
    """The reference's fp16 model with tied embedding, its workspaces, logits and AdamW state for one (batch, seq), and
    its trainer's step (train/train.cpp:536-556). `params[name]` / `grads[name]` are torch views of the reference's own
    device tensors, named token_embedding, final_norm, layers.<i>.<field>."""

    def __init__(self, vocab, layers, hidden, intermediate, q_heads, kv_heads, head_dim, rotary, eps, batch, seq, cos, sin):
        L = lib()
        L.ref_model_last_error.restype = C.c_char_p
        L.ref_model_create.restype = C.c_void_p
        self.h = L.ref_model_create(*_z(vocab, layers, hidden, intermediate, q_heads, kv_heads, head_dim, rotary), C.c_float(eps),
                                    *_z(batch, seq), _p(cos), _p(sin))
        if not self.h:
            raise RuntimeError("ref_model_create: " + L.ref_model_last_error().decode())
        self.h = C.c_void_p(self.h)
        self.params, self.grads, self.order = {}, {}, []
        self._refresh_views()

    def _refresh_views(self):
        L = lib()
        name = C.create_string_buffer(96)
        for i in range(L.ref_model_num_params(self.h)):
            n, p, g = C.c_size_t(), C.c_void_p(), C.c_void_p()
            _mcheck(L.ref_model_param(self.h, i, name, C.c_size_t(96), C.byref(n), C.byref(p), C.byref(g)), "ref_model_param")
            key = name.value.decode()
            if key not in self.params:
                self.order.append(key)
            self.params[key] = _view(p.value, n.value, torch.float16)
            self.grads[key] = _view(g.value, n.value, torch.float16)

    def init(self, seed: int):
        """The reference's own seeded initialisation (src/core/weight_initialization.cu:122-181)."""
        _mcheck(lib().ref_model_init(self.h, C.c_uint64(seed)), "ref_model_init")

    def reset_optimizer(self):
        _mcheck(lib().ref_model_reset_optimizer(self.h), "ref_model_reset_optimizer")

    def state(self, i: int):
        """(master, first moment, second moment) fp32 views of parameter i in `order`."""
        a, b, c = C.c_void_p(), C.c_void_p(), C.c_void_p()
        _mcheck(lib().ref_model_state(self.h, i, C.byref(a), C.byref(b), C.byref(c)), "ref_model_state")
        n = self.params[self.order[i]].numel()
        return tuple(_view(x.value, n, torch.float32) for x in (a, b, c))

    def step(self, ids, targets, loss_scale, graph=False):
        fn = lib().ref_model_step_graph if graph else lib().ref_model_step
        _mcheck(fn(self.h, _p(ids), _p(targets), C.c_float(loss_scale), _s()), "ref_model_step")

    def adamw(self, lr, beta1, beta2, eps, weight_decay, loss_scale, max_grad_norm):
        _mcheck(lib().ref_model_adamw(self.h, *(C.c_float(v) for v in (lr, beta1, beta2, eps, weight_decay, loss_scale, max_grad_norm)),
                                      _s()), "ref_model_adamw")

    def check(self):
        ok, step = C.c_int(), C.c_uint64()
        _mcheck(lib().ref_model_check(self.h, C.byref(ok), C.byref(step), _s()), "ref_model_check")
        return bool(ok.value), int(step.value)

    def loss(self) -> float:
        out = C.c_float()
        _mcheck(lib().ref_model_loss(self.h, C.byref(out), _s()), "ref_model_loss")
        return float(out.value)

    def close(self):
        if self.h:
            self.params.clear(); self.grads.clear()
            lib().ref_model_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()


def block_forward_backward(out, grad_input, grad_output, input, weights: dict, grads: dict, cos, sin, batch, seq, hidden,
                           intermediate, q_heads, kv_heads, head_dim, rotary, eps):
    """transformer_block_forward then transformer_block_backward of the reference on fp16 device tensors."""
    lib().ref_model_last_error.restype = C.c_char_p
    w = (C.c_void_p * 11)(*[weights[n].data_ptr() for n in BLOCK_FIELDS])
    g = (C.c_void_p * 11)(*[grads[n].data_ptr() for n in BLOCK_FIELDS])
    _mcheck(lib().ref_block_forward_backward(_p(out), _p(grad_input), _p(grad_output), _p(input), w, g, _p(cos), _p(sin),
                                             *_z(batch, seq, hidden, intermediate, q_heads, kv_heads, head_dim, rotary), C.c_float(eps),
                                             _s()), "ref_block_forward_backward")


def linear_backward(dx, dw, db, dy, x, w, accumulate=(False, False, False)):
    lib().ref_model_last_error.restype = C.c_char_p
    rows, out_f = dy.shape
    _mcheck(lib().ref_cuda_linear_backward(_p(dx), _p(dw), _p(db), _p(dy), _p(x), _p(w), *_z(rows, x.shape[1], out_f),
                                           *(int(a) for a in accumulate), _DT[x.dtype], _s()), "linear_backward")
