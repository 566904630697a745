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
