"""GPU parity of attention forward/backward (through the C ABI) against the numpy oracle, the committed
outputs of the reference's CPU attention, and the shapes of the reference's own tests
(tests/flash_attention_test.cu:306-388: Sq != Sk, non-zero offset, explicit scale, D = 32/64/128).
Both the generic path and (where it applies) the tensor-core path are exercised.
Tolerance: norm-scaled max error 1e-2 for fp16 gradients (the parity bar), 3e-2 absolute on the reference
test shapes (the reference test's own tolerance).
"""
from pathlib import Path

import numpy as np
import pytest
import torch

import known_answers as KA
from gpu_util import assert_close, dev, host, rounded
from oracle import cgpt_oracle as O

pytestmark = pytest.mark.gpu
GOLD = np.load(Path(__file__).parent / "golden" / "ref_cpu_ops.npz")


@pytest.fixture(scope="module")
def ops():
    from cgpt_b200 import ops as m
    return m


def run_case(ops, b, sq, sk, hq, hkv, d, off, scale, dt, causal=True, force_generic=False, seed=0, tol=1e-2, with_lse=True):
    r = np.random.default_rng(seed + sq + d)
    q, k, v, do = (dev(r.standard_normal(s), dt) for s in ((b, sq, hq, d), (b, sk, hkv, d), (b, sk, hkv, d), (b, sq, hq, d)))
    opts = ops.FlashAttentionOptions(hq, hkv, d, scale, causal, off)
    out = torch.full_like(q, float("nan")); lse = torch.full((b, sq, hq), float("nan"), device="cuda")
    ops.flash_gqa_attention_forward_with_lse(out, lse, q, k, v, None, opts, force_generic=force_generic)
    eo, el = O.attention_forward(rounded(q), rounded(k), rounded(v), causal, off, scale)
    assert_close(host(out), eo, tol, "out")
    np.testing.assert_allclose(host(lse), el, atol=2e-3, rtol=1e-3)
    dq, dk, dv = torch.full_like(q, float("nan")), torch.full_like(k, float("nan")), torch.full_like(v, float("nan"))
    if with_lse:
        ops.flash_gqa_attention_backward_with_lse(dq, dk, dv, do, out, lse, q, k, v, None, opts, force_generic=force_generic)
    else:
        ops.flash_gqa_attention_backward(dq, dk, dv, do, q, k, v, None, opts)
    # ground truth: fp32 oracle on the same (rounded) inputs with the saved O / LSE the kernel was given
    edq, edk, edv = O.attention_backward(rounded(do), rounded(q), rounded(k), rounded(v), host(out), host(lse), causal, off, scale)
    assert_close(host(dq), edq, tol, "dq"); assert_close(host(dk), edk, tol, "dk"); assert_close(host(dv), edv, tol, "dv")
    return (q, k, v, do, out, lse, dq, dk, dv, opts)


@pytest.mark.parametrize("case", KA.ATTENTION_CASES)
@pytest.mark.parametrize("with_lse", [True, False])
def test_reference_test_shapes(ops, case, with_lse):
    c = case
    got = run_case(ops, c["batch"], c["sq"], c["sk"], c["hq"], c["hkv"], c["d"], c["offset"], c["scale"], "f16", with_lse=with_lse)
    q, k, v, do, out, lse, dq, dk, dv, _ = got
    edq, edk, edv = O.attention_backward(rounded(do), rounded(q), rounded(k), rounded(v), None, None, True, c["offset"], c["scale"])
    for a, e in ((dq, edq), (dk, edk), (dv, edv)):
        np.testing.assert_allclose(host(a), e, atol=3e-2)


@pytest.mark.parametrize("dt,tol", [("f32", 1e-4), ("bf16", 4e-2)])
def test_other_dtypes_and_non_causal(ops, dt, tol):
    run_case(ops, 2, 17, 17, 4, 2, 32, 0, 0.0, dt, tol=tol)
    run_case(ops, 1, 9, 21, 6, 2, 40, 0, 0.3, dt, causal=False, tol=tol)


@pytest.mark.parametrize("force_generic", [True, False])
@pytest.mark.parametrize("b,s,hq,hkv,d", [(2, 128, 4, 2, 64), (1, 256, 8, 2, 128), (2, 200, 12, 4, 64), (1, 384, 4, 4, 128), (1, 130, 2, 1, 64)])
def test_model_shapes_f16(ops, b, s, hq, hkv, d, force_generic):
    run_case(ops, b, s, s, hq, hkv, d, 0, 0.0, "f16", force_generic=force_generic)


def test_accumulate_and_determinism(ops):
    q, k, v, do, out, lse, dq, dk, dv, opts = run_case(ops, 1, 192, 192, 4, 2, 64, 0, 0.0, "f16")
    dq2, dk2, dv2 = dq.clone(), dk.clone(), dv.clone()
    ops.flash_gqa_attention_backward_with_lse(dq2, dk2, dv2, do, out, lse, q, k, v, None, opts, accumulate_grads=True)
    assert_close(host(dq2), 2 * host(dq), 4e-3, "acc dq"); assert_close(host(dk2), 2 * host(dk), 4e-3, "acc dk")
    assert_close(host(dv2), 2 * host(dv), 4e-3, "acc dv")
    dq3, dk3, dv3 = torch.empty_like(dq), torch.empty_like(dk), torch.empty_like(dv)
    ops.flash_gqa_attention_backward_with_lse(dq3, dk3, dv3, do, out, lse, q, k, v, None, opts)
    assert torch.equal(dq, dq3) and torch.equal(dk, dk3) and torch.equal(dv, dv3), "attention backward must be bit-reproducible"


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_golden_reference_cpu_attention(ops, dt):
    tol = 1e-4 if dt == "f32" else 6e-3
    for name in "abc":
        kk = f"attn_{dt}_{name}"
        b, sq, sk, hq, hkv, d, off = (int(x) for x in GOLD[kk + "_cfg"])
        sc = float(GOLD[kk + "_scale"])
        q, k, v, do = (dev(GOLD[kk + s], dt) for s in ("_q", "_k", "_v", "_do"))
        opts = ops.FlashAttentionOptions(hq, hkv, d, sc, True, off)
        out = torch.empty_like(q); lse = torch.empty((b, sq, hq), device="cuda")
        ops.flash_gqa_attention_forward_with_lse(out, lse, q, k, v, None, opts)
        assert_close(host(out), GOLD[kk + "_o"], tol, "o"); np.testing.assert_allclose(host(lse), GOLD[kk + "_lse"], atol=2e-3)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ops.flash_gqa_attention_backward_with_lse(dq, dk, dv, do, dev(GOLD[kk + "_o"], dt), dev(GOLD[kk + "_lse"]), q, k, v, None, opts)
        for a, s in ((dq, "_dq"), (dk, "_dk"), (dv, "_dv")):
            assert_close(host(a), GOLD[kk + s], tol, s)


def test_validation(ops):
    q = dev(np.zeros((1, 4, 4, 32)), "f16"); k = dev(np.zeros((1, 4, 2, 32)), "f16")
    o = ops.FlashAttentionOptions(4, 2, 32)
    with pytest.raises(ValueError):   # causal range: offset + sq > sk
        ops.flash_gqa_attention_backward(torch.empty_like(q), torch.empty_like(k), torch.empty_like(k), q, q, k, k, None,
                                         ops.FlashAttentionOptions(4, 2, 32, 0.0, True, 3))
    with pytest.raises(ValueError):   # heads not divisible
        ops.flash_gqa_attention_backward(torch.empty_like(q), torch.empty_like(k), torch.empty_like(k), q, q, k, k, None,
                                         ops.FlashAttentionOptions(4, 3, 32))
    with pytest.raises(ValueError):   # dtype mismatch
        ops.flash_gqa_attention_backward(torch.empty_like(q), torch.empty_like(k), torch.empty_like(k), q.float(), q, k, k, None, o)
