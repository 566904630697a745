"""GPU parity of the fused per-head QK-RMSNorm + RoPE kernels (through the C ABI) against the oracle's composition
rmsnorm -> (round to storage dtype) -> rope, forward and backward, and against the library's own separate ops."""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import TOL, assert_close, dev, host, rounded
from oracle import cgpt_oracle as O

pytestmark = pytest.mark.gpu


def _call(name, lib, ptrs, dims, eps, t):
    fn = getattr(lib.lib, name)
    return fn(*[None if p is None else p.data_ptr() for p in ptrs], *dims, C.c_float(eps), lib.dtype_code(t), lib.stream_ptr())


@pytest.mark.parametrize("b,s,hq,hkv,d,rot,off,dt", [(2, 128, 4, 2, 64, 0, 0, "f16"), (4, 256, 8, 2, 128, 0, 0, "f16"),
                                                     (1, 77, 12, 4, 64, 32, 5, "f16"), (2, 33, 2, 1, 32, 0, 0, "bf16"),
                                                     (1, 50, 3, 3, 256, 128, 2, "f16")])
def test_fused_matches_oracle_and_separate_ops(b, s, hq, hkv, d, rot, off, dt):
    from cgpt_b200 import _lib, ops
    r = np.random.default_rng(b * 7 + s + d)
    rd = rot or d
    cos, sin = O.rotary_cache(s + off + 1, rd)
    cos_d, sin_d = dev(cos, dt), dev(sin, dt)
    q_pre, k_pre = dev(r.standard_normal((b, s, hq, d)), dt), dev(r.standard_normal((b, s, hkv, d)), dt)
    wq, wk = dev(1 + 0.1 * r.standard_normal(d), dt), dev(1 + 0.1 * r.standard_normal(d), dt)
    dims = (b, s, hq, hkv, d, rot, off, cos_d.shape[0])
    q, k = torch.full_like(q_pre, float("nan")), torch.full_like(k_pre, float("nan"))
    _lib.check(_call("cgpt_qknorm_rope_forward", _lib, (q, k, q_pre, k_pre, wq, wk, cos_d, sin_d), dims, 1e-5, q_pre), "fwd")
    # oracle: rmsnorm -> storage rounding -> rope
    def fwd(x, w):
        n = O.rnd(O.rmsnorm_forward(rounded(x).reshape(-1, d), rounded(w), 1e-5), dt).reshape(x.shape)
        return O.rope_forward(n, rounded(cos_d), rounded(sin_d), rot, off)
    assert_close(host(q), fwd(q_pre, wq), TOL[dt], "q"); assert_close(host(k), fwd(k_pre, wk), TOL[dt], "k")
    # the separate ops of the library agree to the last bit or two (their fp32 sums run in a different order)
    q2, k2 = torch.empty_like(q), torch.empty_like(k)
    ops.rmsnorm_forward(q2.view(-1, d), q_pre.view(-1, d), wq, 1e-5); ops.rmsnorm_forward(k2.view(-1, d), k_pre.view(-1, d), wk, 1e-5)
    ops.rope_forward(q2, k2, cos_d, sin_d, None, ops.RopeOptions(rot, off))
    assert_close(host(q), host(q2), TOL[dt], "fused vs separate q"); assert_close(host(k), host(k2), TOL[dt], "fused vs separate k")

    dq_rot, dk_rot = dev(r.standard_normal((b, s, hq, d)), dt), dev(r.standard_normal((b, s, hkv, d)), dt)
    dq, dk = torch.full_like(q_pre, float("nan")), torch.full_like(k_pre, float("nan"))
    gwq, gwk = torch.full_like(wq, float("nan")), torch.full_like(wk, float("nan"))
    _lib.check(_call("cgpt_qknorm_rope_backward", _lib, (dq, dk, gwq, gwk, dq_rot, dk_rot, q_pre, k_pre, wq, wk, cos_d, sin_d), dims,
                     1e-5, q_pre), "bwd")
    def bwd(g, x, w):
        un = O.rnd(O.rope_backward(rounded(g), rounded(cos_d), rounded(sin_d), rot, off), dt)
        dx, dw = O.rmsnorm_backward(un.reshape(-1, d), rounded(x).reshape(-1, d), rounded(w), 1e-5)
        return dx.reshape(x.shape), dw
    edq, egwq = bwd(dq_rot, q_pre, wq); edk, egwk = bwd(dk_rot, k_pre, wk)
    assert_close(host(dq), edq, TOL[dt], "dq"); assert_close(host(dk), edk, TOL[dt], "dk")
    assert_close(host(gwq), egwq, TOL[dt] * 2, "dw_q"); assert_close(host(gwk), egwk, TOL[dt] * 2, "dw_k")
    dq3, dk3, g3, g4 = torch.empty_like(dq), torch.empty_like(dk), torch.empty_like(gwq), torch.empty_like(gwk)
    _lib.check(_call("cgpt_qknorm_rope_backward", _lib, (dq3, dk3, g3, g4, dq_rot, dk_rot, q_pre, k_pre, wq, wk, cos_d, sin_d), dims,
                     1e-5, q_pre), "bwd")
    assert torch.equal(dq, dq3) and torch.equal(gwq, g3) and torch.equal(gwk, g4), "must be bit-reproducible"


def test_unsupported_shapes_are_reported():
    from cgpt_b200 import _lib
    x = dev(np.ones((1, 4, 2, 48)), "f16"); w = dev(np.ones(48), "f16"); c = dev(np.ones((4, 24)), "f16")
    rc = _call("cgpt_qknorm_rope_forward", _lib, (x, x, x, x, w, w, c, c), (1, 4, 2, 2, 48, 0, 0, 4), 1e-5, x)
    assert rc == 6   # CGPT_ERR_UNSUPPORTED: head_dim 48 is not a power of two; callers fall back to the separate ops
