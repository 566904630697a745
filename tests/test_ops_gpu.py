"""GPU parity of the memory-bound kernels (through the C ABI) against the numpy oracle, the committed
outputs of the reference's CPU operators, and the reference tests' known answers.

Tolerances (gpu_util.TOL) are norm-scaled max errors: 2e-5 fp32, 2e-3 fp16, 1.6e-2 bf16 - i.e. one rounding
of the storage dtype; the parity bar for fp16-path gradients is 1e-2.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

import known_answers as KA
from gpu_util import TOL, assert_close, dev, host, ids_dev, rounded
from oracle import cgpt_oracle as O

pytestmark = pytest.mark.gpu
GOLD = np.load(Path(__file__).parent / "golden" / "ref_cpu_ops.npz")


@pytest.fixture(scope="module")
def ops():
    from cgpt_b200 import ops as m
    return m


def rng(seed):
    return np.random.default_rng(seed)


# ------------------------------------------------------------------------------------------ RMSNorm
RMS_SHAPES = [(3, 7, "f32"), (2, 4096, "f16"), (129, 513, "bf16"), (512, 4096, "f16"), (40, 64, "f16"), (1000, 128, "f16"),
              (300, 1024, "f16"), (77, 768, "f16"), (33, 2048, "bf16"), (5, 1024, "f32"), (64, 688, "f16"), (9, 100, "f32")]


@pytest.mark.parametrize("rows,hidden,dt", RMS_SHAPES)
def test_rmsnorm_forward_backward(ops, rows, hidden, dt):
    r = rng(rows * 7 + hidden)
    x, dy, w = dev(r.standard_normal((rows, hidden)), dt), dev(r.standard_normal((rows, hidden)), dt), dev(1 + 0.02 * r.standard_normal(hidden), dt)
    y, dx, dw = torch.full_like(x, float("nan")), torch.full_like(x, float("nan")), torch.full_like(w, float("nan"))
    ops.rmsnorm_forward(y, x, w, 1e-5)
    ops.rmsnorm_backward(dx, dw, dy, x, w, 1e-5)
    ey = O.rmsnorm_forward(rounded(x), rounded(w), 1e-5)
    edx, edw = O.rmsnorm_backward(rounded(dy), rounded(x), rounded(w), 1e-5)
    assert_close(host(y), ey, TOL[dt], "y"); assert_close(host(dx), edx, TOL[dt], "dx")
    assert_close(host(dw), edw, TOL[dt] * 2, "dw")
    # determinism: same bits on a second run
    dx2, dw2 = torch.empty_like(dx), torch.empty_like(dw)
    ops.rmsnorm_backward(dx2, dw2, dy, x, w, 1e-5)
    assert torch.equal(dx, dx2) and torch.equal(dw, dw2)


@pytest.mark.parametrize("rows,hidden,dt", [(300, 1024, "f16"), (77, 768, "f16"), (1000, 256, "bf16"), (257, 520, "f16"),
                                            (33, 2048, "bf16"), (5, 1024, "f32"), (64, 100, "f16")])
@pytest.mark.parametrize("with_residual", [True, False])
def test_rmsnorm_dual(ops, rows, hidden, dt, with_residual):
    """Both norms of one input in one pass against the oracle and against the single-norm operators: the forward is
    bit-identical to two single calls; the backward sums residual + both input gradients in fp32 with one rounding, so
    it agrees with the oracle's fp32 sum (and with the chained single calls to a rounding of the storage dtype).
    Shapes of the one-pass kernels (16-bit, 256..1024 columns) and shapes that fall back to the single operators."""
    r = rng(rows + hidden)
    x, da, db, res = (dev(r.standard_normal((rows, hidden)), dt) for _ in range(4))
    wa, wb = dev(1 + 0.05 * r.standard_normal(hidden), dt), dev(1 + 0.05 * r.standard_normal(hidden), dt)
    ya, yb, ya1, yb1 = (torch.full_like(x, float("nan")) for _ in range(4))
    ops.rmsnorm_forward_dual(ya, yb, x, wa, wb, 1e-5)
    ops.rmsnorm_forward(ya1, x, wa, 1e-5); ops.rmsnorm_forward(yb1, x, wb, 1e-5)
    assert torch.equal(ya, ya1) and torch.equal(yb, yb1)
    dx, dwa, dwb = torch.full_like(x, float("nan")), torch.full_like(wa, float("nan")), torch.full_like(wb, float("nan"))
    ops.rmsnorm_backward_dual(dx, dwa, dwb, da, db, x, wa, wb, 1e-5, residual=res if with_residual else None)
    ea, ewa = O.rmsnorm_backward(rounded(da), rounded(x), rounded(wa), 1e-5)
    eb, ewb = O.rmsnorm_backward(rounded(db), rounded(x), rounded(wb), 1e-5)
    want = ea + eb + (rounded(res) if with_residual else 0.0)
    assert_close(host(dx), want, TOL[dt], "dual dx")
    assert_close(host(dwa), ewa, TOL[dt] * 2, "dual dw a"); assert_close(host(dwb), ewb, TOL[dt] * 2, "dual dw b")
    dw1 = torch.empty_like(wa)
    ops.rmsnorm_backward(torch.empty_like(x), dw1, da, x, wa, 1e-5)
    assert torch.equal(dw1, dwa)       # same partial sums, same order
    if with_residual:                  # in place over the residual
        dx2 = res.clone()
        ops.rmsnorm_backward_dual(dx2, dwa, dwb, da, db, x, wa, wb, 1e-5, residual=dx2)
        assert torch.equal(dx2, dx)


def test_rmsnorm_backward_residuals(ops):
    r = rng(3)
    x, dy, a, b = (dev(r.standard_normal((257, 1024)), "f16") for _ in range(4))
    w = dev(1 + 0.02 * r.standard_normal(1024), "f16")
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    ops.rmsnorm_backward(dx, dw, dy, x, w, 1e-5, residual_a=a, residual_b=b)
    edx, _ = O.rmsnorm_backward(rounded(dy), rounded(x), rounded(w), 1e-5)
    assert_close(host(dx), edx + rounded(a) + rounded(b), TOL["f16"], "dx+res")


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_rmsnorm_golden(ops, dt):
    for rows, hidden in ((3, 7), (40, 64), (17, 256)):
        k = f"rms_{dt}_{rows}x{hidden}"
        x, dy, w = dev(GOLD[k + "_x"], dt), dev(GOLD[k + "_dy"], dt), dev(GOLD[k + "_w"], dt)
        y, dx, dw = torch.empty_like(x), torch.empty_like(x), torch.empty_like(w)
        ops.rmsnorm_forward(y, x, w, 1e-5); ops.rmsnorm_backward(dx, dw, dy, x, w, 1e-5)
        assert_close(host(y), GOLD[k + "_y"], TOL[dt], "y"); assert_close(host(dx), GOLD[k + "_dx"], TOL[dt], "dx")
        assert_close(host(dw), GOLD[k + "_dw"], TOL[dt] * 2, "dw")


def test_rmsnorm_rejects_bad_arguments(ops):
    x = dev(np.ones((2, 8)), "f16"); w = dev(np.ones(8), "f16")
    with pytest.raises(ValueError):
        ops.rmsnorm_backward(torch.empty_like(x), torch.empty_like(w), x, x, dev(np.ones(4), "f16"), 1e-5)
    with pytest.raises(ValueError):
        ops.rmsnorm_backward(torch.empty_like(x), torch.empty_like(w), x, x.float(), w, 1e-5)
    with pytest.raises(ValueError):
        ops.rmsnorm_forward(torch.empty_like(x), x, w, 0.0)


# --------------------------------------------------------------------------------------------- RoPE
@pytest.mark.parametrize("dt,tol", [("f32", 1e-5), ("f16", 3e-3), ("bf16", 2e-2)])
def test_rope_backward_known_answer(ops, dt, tol):
    c = KA.ROPE_BWD
    gq, gk = dev(c["grad_rotated_query"], dt), dev(c["grad_rotated_key"], dt)
    oq, ok = torch.full_like(gq, float("nan")), torch.full_like(gk, float("nan"))
    ops.rope_backward(oq, ok, gq, gk, dev(c["cos"], dt), dev(c["sin"], dt), None, ops.RopeOptions(rotary_dim=2))
    np.testing.assert_allclose(host(oq), c["grad_query"], atol=tol); np.testing.assert_allclose(host(ok), c["grad_key"], atol=tol)


@pytest.mark.parametrize("b,s,hq,hkv,d,rot,off,dt", [(1, 512, 32, 8, 128, 0, 0, "f16"), (1, 512, 32, 8, 128, 0, 0, "bf16"),
                                                     (2, 128, 4, 2, 64, 0, 0, "f16"), (2, 37, 12, 4, 64, 32, 5, "f16"),
                                                     (3, 16, 8, 2, 128, 0, 3, "f32"), (2, 9, 3, 1, 6, 4, 1, "f16"), (4, 64, 8, 2, 128, 0, 0, "f16")])
def test_rope_forward_backward(ops, b, s, hq, hkv, d, rot, off, dt):
    r = rng(b + s + d)
    rd = rot or d
    cos, sin = O.rotary_cache(s + off + 3, rd)
    cos_d, sin_d = dev(cos, dt), dev(sin, dt)
    q, k = dev(r.standard_normal((b, s, hq, d)), dt), dev(r.standard_normal((b, s, hkv, d)), dt)
    opts = ops.RopeOptions(rotary_dim=rot, position_offset=off)
    eq = O.rope_backward(rounded(q), rounded(cos_d), rounded(sin_d), rot, off); ek = O.rope_backward(rounded(k), rounded(cos_d), rounded(sin_d), rot, off)
    oq, ok = torch.full_like(q, float("nan")), torch.full_like(k, float("nan"))
    ops.rope_backward(oq, ok, q, k, cos_d, sin_d, None, opts)
    assert_close(host(oq), eq, TOL[dt], "dq"); assert_close(host(ok), ek, TOL[dt], "dk")
    fq = O.rope_forward(rounded(q), rounded(cos_d), rounded(sin_d), rot, off); fk = O.rope_forward(rounded(k), rounded(cos_d), rounded(sin_d), rot, off)
    q2, k2 = q.clone(), k.clone()
    ops.rope_forward(q2, k2, cos_d, sin_d, None, opts)
    assert_close(host(q2), fq, TOL[dt], "q"); assert_close(host(k2), fk, TOL[dt], "k")
    # in-place backward of the rotated tensors returns the originals (rotation is orthogonal)
    ops.rope_backward(q2, k2, q2, k2, cos_d, sin_d, None, opts)
    assert_close(host(q2), rounded(q), TOL[dt] * 3, "roundtrip q")


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_rope_golden(ops, dt):
    for rotary, off in ((0, 0), (8, 3)):
        k = f"rope_{dt}_r{rotary}_o{off}"
        q, kk, cos, sin = (dev(GOLD[k + s], dt) for s in ("_q", "_k", "_cos", "_sin"))
        oq, ok = torch.empty_like(q), torch.empty_like(kk)
        ops.rope_backward(oq, ok, q, kk, cos, sin, None, ops.RopeOptions(rotary, off))
        assert_close(host(oq), GOLD[k + "_bq"], TOL[dt], "bq"); assert_close(host(ok), GOLD[k + "_bk"], TOL[dt], "bk")


# ------------------------------------------------------------------------------------------- SwiGLU
@pytest.mark.parametrize("n,dt", [((64, 688), "f16"), ((1000, 2048), "f16"), ((7, 33), "f32"), ((129, 513), "bf16"), ((4096, 2048), "f16")])
def test_swiglu(ops, n, dt):
    r = rng(n[0])
    g, u, dy = dev(3 * r.standard_normal(n), dt), dev(r.standard_normal(n), dt), dev(r.standard_normal(n), dt)
    y, dg, du = (torch.full_like(g, float("nan")) for _ in range(3))
    ops.swiglu_forward(y, g, u); ops.swiglu_backward(dg, du, dy, g, u)
    assert_close(host(y), O.swiglu_forward(rounded(g), rounded(u)), TOL[dt], "y")
    eg, eu = O.swiglu_backward(rounded(dy), rounded(g), rounded(u))
    assert_close(host(dg), eg, TOL[dt], "dgate"); assert_close(host(du), eu, TOL[dt], "dup")
    # accumulate flags add to what is already there
    dg2, du2 = dg.clone(), du.clone()
    ops.swiglu_backward(dg2, du2, dy, g, u, None, ops.SwiGLUBackwardOptions(accumulate_gate=True))
    assert_close(host(dg2), 2 * rounded(dg), TOL[dt] * 2, "acc gate"); assert torch.equal(du2, du)


def test_swiglu_extreme_inputs_stay_finite(ops):
    g = dev(np.array([[-64.0, 64.0, -30.0, 30.0, 0.0, 1e-4, -1e-4, 11.0]] * 4), "f16")
    u = dev(np.full((4, 8), 64.0), "f16")
    y, dg, du = (torch.empty_like(g) for _ in range(3))
    ops.swiglu_forward(y, g, u); ops.swiglu_backward(dg, du, u, g, u)
    torch.cuda.synchronize()
    assert torch.isfinite(y).all() and torch.isfinite(du).all()


# ---------------------------------------------------------------------------------------- Embedding
@pytest.mark.parametrize("dt,tol", [("f16", 1e-2), ("bf16", 5e-2)])
def test_embedding_backward_known_answer(ops, dt, tol):
    c = KA.EMBEDDING_BWD
    gw = torch.full((3, 4), float("nan"), device="cuda", dtype=dev(c["grad_output"], dt).dtype)
    ops.embedding_backward(gw, dev(c["grad_output"], dt), ids_dev(c["ids"]), 3)
    np.testing.assert_allclose(host(gw), c["grad_weight"], atol=tol)


@pytest.mark.parametrize("tokens,vocab,hidden,dt", [(512, 32000, 4096, "f16"), (256, 32000, 256, "f16"), (1000, 50, 24, "f32"), (333, 17, 7, "bf16")])
def test_embedding_forward_backward(ops, tokens, vocab, hidden, dt):
    r = rng(tokens)
    ids = r.integers(0, vocab, tokens)
    ids[::17] = vocab + 5          # out-of-table ids are skipped
    ids[1::5] = ids[0]             # heavy repetition of one id
    w, dy = dev(r.standard_normal((vocab, hidden)), dt), dev(r.standard_normal((tokens, hidden)), dt)
    idd = ids_dev(ids)
    out = torch.full((tokens, hidden), float("nan"), device="cuda", dtype=w.dtype)
    ops.embedding_forward(out, idd, tokens, w)
    valid = ids < vocab
    assert torch.equal(out[torch.from_numpy(valid).cuda()], w[torch.from_numpy(ids[valid]).cuda()])
    gw = torch.full_like(w, float("nan"))
    ops.embedding_backward(gw, dy, idd, tokens)
    assert_close(host(gw), O.embedding_backward(rounded(dy), ids, vocab), TOL[dt], "gw")
    gw2 = w.clone()
    ops.embedding_backward(gw2, dy, idd, tokens, None, ops.EmbeddingBackwardOptions(accumulate_weight=True))
    assert_close(host(gw2), O.embedding_backward(rounded(dy), ids, vocab, accumulate_into=rounded(w)), TOL[dt], "gw acc")
    gw3 = torch.empty_like(w)
    ops.embedding_backward(gw3, dy, idd, tokens)
    assert torch.equal(gw, gw3), "embedding backward must be bit-reproducible"


# ------------------------------------------------------------------------------------ Cross entropy
def test_cross_entropy_known_answers(ops):
    c = KA.CE
    loss = torch.zeros(1, device="cuda"); grad = torch.empty(2, 3, device="cuda")
    ops.cross_entropy_forward_backward(loss, grad, dev(c["logits"]), ids_dev(c["targets"]), 2)
    np.testing.assert_allclose(host(loss), [c["loss"]], atol=1e-5); np.testing.assert_allclose(host(grad), c["grad"], atol=1e-5)
    c = KA.CE_SCALED
    loss = torch.zeros(1, device="cuda"); grad = torch.empty(1, 2, device="cuda")
    ops.cross_entropy_forward_backward(loss, grad, dev(c["logits"]), ids_dev(c["targets"]), 1, None, 1024.0)
    np.testing.assert_allclose(host(loss), [c["loss"]], atol=1e-5); np.testing.assert_allclose(host(grad), c["grad"], atol=1e-3)
    with pytest.raises(ValueError):   # tests/cross_entropy_test.cu:58-63: target count must equal rows
        ops.cross_entropy_forward_backward(loss, torch.empty(2, 3, device="cuda"), dev(KA.CE["logits"]), ids_dev([0, 1]), 1)


@pytest.mark.parametrize("rows,vocab,dt", [(512, 50257, "f32"), (256, 32000, "f16"), (33, 1000, "bf16"), (16, 120000, "f16")])
def test_cross_entropy(ops, rows, vocab, dt):
    r = rng(rows)
    z = dev(3 * r.standard_normal((rows, vocab)), dt)
    t = r.integers(0, vocab, rows); t[3] = vocab + 1
    loss = torch.zeros(1, device="cuda"); grad = torch.full_like(z, float("nan"))
    ops.cross_entropy_forward_backward(loss, grad, z, ids_dev(t), rows, None, 1024.0)
    el, eg = O.cross_entropy(rounded(z), t, 1024.0)
    assert abs(float(loss.item()) - float(el)) <= 2e-5 * max(1.0, abs(float(el)))
    assert_close(host(grad), eg, TOL[dt] * 2, "grad")
    loss2 = torch.zeros(1, device="cuda")
    ops.cross_entropy_forward(loss2, z, ids_dev(t), rows)
    assert torch.equal(loss, loss2)


# --------------------------------------------------------------------------------------------- adds
def test_add_tensors(ops):
    r = rng(0)
    a, b, c = (dev(r.standard_normal((100, 1024)), "f16") for _ in range(3))
    out = torch.empty_like(a)
    ops.add_tensors(out, a, b, None, c)
    assert_close(host(out), rounded(a) + rounded(b) + rounded(c), TOL["f16"], "a+b+c")
    want = rounded(a) + rounded(b)
    ops.add_tensors(a, a, b)   # in place, as add_inplace
    assert_close(host(a), want, TOL["f16"], "inplace")
