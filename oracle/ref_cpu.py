"""ctypes access to ``oracle/_ref/libcgpt_ref_cpu.so`` -- the reference's own CPU operators compiled from
its sources by ``oracle/build_ref.py`` (TEST INFRASTRUCTURE; used by tests, by the fixture generator in
``tests/golden`` and by the CPU-baseline leg of ``bench.py``).

All functions take and return fp32 numpy arrays; ``dtype`` ("f16", "bf16", "f32") selects the storage type
of the reference's CPU tensors, i.e. inputs are rounded to it on entry and outputs carry its rounding.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libcgpt_ref_cpu.so"
CODES = {"f16": 0, "bf16": 1, "f32": 2}
_lib = None


def available() -> bool:
    return LIB_PATH.exists()


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise FileNotFoundError(f"{LIB_PATH} missing: run `python oracle/build_ref.py` where the reference is checked out")
        _lib = C.CDLL(str(LIB_PATH))
        _lib.ref_last_error.restype = C.c_char_p
        _lib.ref_cpu_forward_loss.restype = C.c_double
    return _lib


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _ok(rc, what):
    if rc < 0:
        raise RuntimeError(f"{what}: {lib().ref_last_error().decode()}")
    return rc


def _sz(*v):
    return [C.c_size_t(int(x)) for x in v]


def rmsnorm_forward(x, w, eps, dtype="f32"):
    x, w = _f(x), _f(w)
    y = np.empty_like(x)
    _ok(lib().ref_rmsnorm_forward(_p(y), _p(x), _p(w), *_sz(x.shape[0], x.shape[1]), C.c_float(eps), CODES[dtype]), "rmsnorm_forward")
    return y


def rmsnorm_backward(dy, x, w, eps, dtype="f32"):
    dy, x, w = _f(dy), _f(x), _f(w)
    dx, dw = np.empty_like(x), np.empty_like(w)
    _ok(lib().ref_rmsnorm_backward(_p(dx), _p(dw), _p(dy), _p(x), _p(w), *_sz(x.shape[0], x.shape[1]), C.c_float(eps),
                                   CODES[dtype]), "rmsnorm_backward")
    return dx, dw


def rope_forward(q, k, cos, sin, rotary_dim=0, offset=0, dtype="f32"):
    q, k, cos, sin = _f(q).copy(), _f(k).copy(), _f(cos), _f(sin)
    b, s, hq, d = q.shape
    _ok(lib().ref_rope_forward(_p(q), _p(k), _p(cos), _p(sin), *_sz(b, s, hq, k.shape[2], d, rotary_dim, offset, cos.shape[0]),
                               CODES[dtype]), "rope_forward")
    return q, k


def rope_backward(dq_rot, dk_rot, cos, sin, rotary_dim=0, offset=0, dtype="f32"):
    dq_rot, dk_rot, cos, sin = _f(dq_rot), _f(dk_rot), _f(cos), _f(sin)
    b, s, hq, d = dq_rot.shape
    dq, dk = np.empty_like(dq_rot), np.empty_like(dk_rot)
    _ok(lib().ref_rope_backward(_p(dq), _p(dk), _p(dq_rot), _p(dk_rot), _p(cos), _p(sin),
                                *_sz(b, s, hq, dk_rot.shape[2], d, rotary_dim, offset, cos.shape[0]), CODES[dtype]), "rope_backward")
    return dq, dk


def swiglu_forward(gate, up, dtype="f32"):
    gate, up = _f(gate), _f(up)
    g2 = gate.reshape(-1, gate.shape[-1])
    y = np.empty_like(g2)
    _ok(lib().ref_swiglu_forward(_p(y), _p(g2), _p(up), *_sz(g2.shape[0], g2.shape[1]), CODES[dtype]), "swiglu_forward")
    return y.reshape(gate.shape)


def swiglu_backward(dy, gate, up, dtype="f32"):
    dy, gate, up = _f(dy), _f(gate), _f(up)
    g2 = gate.reshape(-1, gate.shape[-1])
    dg, du = np.empty_like(g2), np.empty_like(g2)
    _ok(lib().ref_swiglu_backward(_p(dg), _p(du), _p(dy), _p(g2), _p(up), *_sz(g2.shape[0], g2.shape[1]), CODES[dtype]), "swiglu_backward")
    return dg.reshape(gate.shape), du.reshape(gate.shape)


def embedding_forward(ids, weight, dtype="f32"):
    ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
    weight = _f(weight)
    out = np.empty((ids.size, weight.shape[1]), np.float32)
    _ok(lib().ref_embedding_forward(_p(out), _p(ids), _p(weight), *_sz(ids.size, weight.shape[0], weight.shape[1]), CODES[dtype]), "embedding_forward")
    return out


def embedding_backward(dy, ids, vocab, accumulate_into=None, dtype="f32"):
    ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
    dy = _f(dy).reshape(ids.size, -1)
    gw = np.zeros((vocab, dy.shape[1]), np.float32) if accumulate_into is None else _f(accumulate_into).copy()
    _ok(lib().ref_embedding_backward(_p(gw), _p(dy), _p(ids), *_sz(ids.size, vocab, dy.shape[1]),
                                     int(accumulate_into is not None), CODES[dtype]), "embedding_backward")
    return gw


def linear_forward(x, w, dtype="f32"):
    x, w = _f(x), _f(w)
    y = np.empty((x.shape[0], w.shape[0]), np.float32)
    _ok(lib().ref_linear_forward(_p(y), _p(x), _p(w), *_sz(x.shape[0], w.shape[1], w.shape[0]), CODES[dtype]), "linear_forward")
    return y


def linear_backward(dy, x, w, dtype="f32", acc=(None, None, None)):
    dy, x, w = _f(dy), _f(x), _f(w)
    dx = np.zeros_like(x) if acc[0] is None else _f(acc[0]).copy()
    dw = np.zeros_like(w) if acc[1] is None else _f(acc[1]).copy()
    db = np.zeros(w.shape[0], np.float32) if acc[2] is None else _f(acc[2]).copy()
    _ok(lib().ref_linear_backward(_p(dx), _p(dw), _p(db), _p(dy), _p(x), _p(w), *_sz(x.shape[0], w.shape[1], w.shape[0]),
                                  int(acc[0] is not None), int(acc[1] is not None), int(acc[2] is not None), CODES[dtype]), "linear_backward")
    return dx, dw, db


def attention_forward(q, k, v, causal=True, offset=0, scale=0.0, dtype="f32"):
    q, k, v = _f(q), _f(k), _f(v)
    b, sq, hq, d = q.shape
    out = np.empty_like(q)
    lse = np.empty((b, sq, hq), np.float32)
    _ok(lib().ref_attention_forward_lse(_p(out), _p(lse), _p(q), _p(k), _p(v), *_sz(b, sq, k.shape[1], hq, k.shape[2], d),
                                        int(causal), C.c_size_t(offset), C.c_float(scale), CODES[dtype]), "attention_forward")
    return out, lse


def attention_backward(do, q, k, v, out=None, lse=None, causal=True, offset=0, scale=0.0, dtype="f32"):
    do, q, k, v = _f(do), _f(q), _f(k), _f(v)
    b, sq, hq, d = q.shape
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    dims = _sz(b, sq, k.shape[1], hq, k.shape[2], d)
    if out is None:
        _ok(lib().ref_attention_backward(_p(dq), _p(dk), _p(dv), _p(do), _p(q), _p(k), _p(v), *dims, int(causal),
                                         C.c_size_t(offset), C.c_float(scale), CODES[dtype]), "attention_backward")
    else:
        out, lse = _f(out), _f(lse)
        _ok(lib().ref_attention_backward_lse(_p(dq), _p(dk), _p(dv), _p(do), _p(out), _p(lse), _p(q), _p(k), _p(v), *dims,
                                             int(causal), C.c_size_t(offset), C.c_float(scale), CODES[dtype]), "attention_backward_lse")
    return dq, dk, dv


def cross_entropy(logits, targets, gradient_scale=1.0, dtype="f32", with_grad=True):
    logits = _f(logits)
    targets = np.ascontiguousarray(targets, dtype=np.uint32)
    loss = np.zeros(1, np.float32)
    grad = np.empty_like(logits) if with_grad else None
    _ok(lib().ref_cross_entropy(_p(loss), _p(grad) if with_grad else None, _p(logits), _p(targets),
                                *_sz(logits.shape[0], logits.shape[1]), C.c_float(gradient_scale), CODES[dtype]), "cross_entropy")
    return float(loss[0]), grad


def adamw_step(param, grad, master, m, v, step, lr, beta1, beta2, eps, wd, loss_scale=1.0, max_grad_norm=np.inf, dtype="f32"):
    param, grad, master, m, v = (_f(a).copy() for a in (param, grad, master, m, v))
    st = C.c_ulonglong(step)
    applied = _ok(lib().ref_adamw_step_cpu(_p(param), _p(grad), _p(master), _p(m), _p(v), C.c_size_t(param.size), C.byref(st),
                                           *(C.c_float(x) for x in (lr, beta1, beta2, eps, wd, loss_scale, max_grad_norm)),
                                           CODES[dtype]), "adamw_step")
    return param, master, m, v, int(st.value), bool(applied)


def cpu_forward_loss(flat_weights, ids, targets, batch, seq, layers, d, hq, hkv, hd, inter, vocab, eps=1e-5, repeats=1):
    """Times the reference's CPU forward + loss (seconds, median of `repeats`) and returns (seconds, loss)."""
    w = _f(flat_weights)
    ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
    targets = np.ascontiguousarray(targets, dtype=np.uint32).reshape(-1)
    loss = C.c_float(0)
    secs = lib().ref_cpu_forward_loss(C.byref(loss), _p(w), _p(ids), _p(targets), *_sz(batch, seq, layers, d, hq, hkv, hd, inter, vocab),
                                      C.c_float(eps), int(repeats))
    if secs < 0:
        raise RuntimeError(f"cpu_forward_loss: {lib().ref_last_error().decode()}")
    return float(secs), float(loss.value)
