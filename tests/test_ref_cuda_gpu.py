"""Parity against the reference's OWN CUDA kernels, rebuilt for sm_100a (oracle/_ref/libcgpt_ref_cuda.so, built by
oracle/build_ref.py from the reference's sources): both implementations run on the same device tensors.

Tolerances (norm-scaled error of tests/gpu_util.py unless stated): both sides round fp32 results to fp16 once, so
element-wise ops agree to an fp16 ulp (2e-3); RoPE has a single fp32 expression per element and must be bit-equal;
gradients that the reference accumulates with fp16 atomics (embedding rows, dK/dV of its scalar attention path) carry
the reference's own rounding noise and are held to the 1e-2 parity bar of fp16-path gradients.
"""
import numpy as np
import pytest
import torch

from gpu_util import assert_close, host
from oracle import ref_cuda as R

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not R.available(), reason="oracle/_ref/libcgpt_ref_cuda.so not built")]


@pytest.fixture(scope="module")
def ops():
    from cgpt_b200 import ops as m
    return m


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g, device="cuda") * scale).half()


@pytest.mark.parametrize("rows,hidden", [(512, 1024), (300, 768), (2048, 128), (64, 2048)])
def test_rmsnorm(ops, rows, hidden):
    x, dy, w = rnd(rows, hidden), rnd(rows, hidden, seed=1), (1 + rnd(hidden, scale=0.02, seed=2))
    y0, y1 = torch.empty_like(x), torch.empty_like(x)
    R.rmsnorm_forward(y0, x, w, 1e-5)
    ops.rmsnorm_forward(y1, x, w, 1e-5)
    assert_close(host(y1), host(y0), 2e-3, "rmsnorm forward")
    dx0, dx1, dw0, dw1 = torch.empty_like(x), torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)
    R.rmsnorm_backward(dx0, dw0, dy, x, w, 1e-5)
    ops.rmsnorm_backward(dx1, dw1, dy, x, w, 1e-5)
    assert_close(host(dx1), host(dx0), 2e-3, "rmsnorm dx")
    assert_close(host(dw1), host(dw0), 2e-3, "rmsnorm dw")


@pytest.mark.parametrize("hq,hkv,d", [(12, 4, 64), (8, 2, 128)])
def test_rope_bit_equal(ops, hq, hkv, d):
    from cgpt_b200.model import rotary_cache
    b, s = 2, 96
    cos, sin = rotary_cache(s, d)
    q, k = rnd(b, s, hq, d), rnd(b, s, hkv, d, seed=3)
    q0, k0, q1, k1 = q.clone(), k.clone(), q.clone(), k.clone()
    R.rope_forward(q0, k0, cos, sin)
    ops.rope_forward(q1, k1, cos, sin)
    assert torch.equal(q0, q1) and torch.equal(k0, k1)
    dq0, dk0, dq1, dk1 = (torch.empty_like(t) for t in (q, k, q, k))
    R.rope_backward(dq0, dk0, q, k, cos, sin)
    ops.rope_backward(dq1, dk1, q, k, cos, sin)
    assert torch.equal(dq0, dq1) and torch.equal(dk0, dk1)


def test_swiglu(ops):
    g, u, dy = rnd(777, 688), rnd(777, 688, seed=1), rnd(777, 688, seed=2)
    y0, y1 = torch.empty_like(g), torch.empty_like(g)
    R.swiglu_forward(y0, g, u)
    ops.swiglu_forward(y1, g, u)
    assert_close(host(y1), host(y0), 2e-3, "swiglu forward")
    a0, b0, a1, b1 = (torch.empty_like(g) for _ in range(4))
    R.swiglu_backward(a0, b0, dy, g, u)
    ops.swiglu_backward(a1, b1, dy, g, u)
    assert_close(host(a1), host(a0), 2e-3, "swiglu dgate")
    assert_close(host(b1), host(b0), 2e-3, "swiglu dup")


def test_embedding_backward(ops):
    vocab, hidden, tokens = 500, 256, 4096          # every row is hit ~8 times: the reference sums them with fp16 atomics
    ids = torch.randint(0, vocab, (tokens,), device="cuda", dtype=torch.int32)
    dy = rnd(tokens, hidden, scale=0.1)
    g0 = torch.zeros(vocab, hidden, device="cuda", dtype=torch.float16)
    g1 = torch.zeros_like(g0)
    R.embedding_backward(g0, dy, ids, True)
    ops.embedding_backward(g1, dy, ids, tokens, None, ops.EmbeddingBackwardOptions(accumulate_weight=True))
    assert_close(host(g1), host(g0), 1e-2, "embedding backward")


@pytest.mark.parametrize("rows,vocab", [(64, 32000), (300, 1000)])
def test_cross_entropy(ops, rows, vocab):
    z = rnd(rows, vocab, scale=2.0)
    t = torch.randint(0, vocab, (rows,), device="cuda", dtype=torch.int32)
    l0, l1 = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    g0, g1 = torch.empty_like(z), torch.empty_like(z)
    R.cross_entropy(l0, g0, z, t, 1024.0)
    ops.cross_entropy_forward_backward(l1, g1, z, t, rows, None, 1024.0)
    assert abs(float(l0) - float(l1)) < 1e-4 * max(1.0, abs(float(l0)))
    assert_close(host(g1), host(g0), 2e-3, "cross-entropy gradient", metric="max")


def test_cut_cross_entropy_f32(ops):
    from cgpt_b200 import model as M
    rows, hidden, vocab = 96, 64, 512
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(rows, hidden, generator=g, device="cuda")
    c = torch.randn(vocab, hidden, generator=g, device="cuda") * 0.1
    t = torch.randint(0, vocab, (rows,), device="cuda", dtype=torch.int32)
    l0, l1 = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    gx0, gx1, gc0, gc1 = torch.empty_like(x), torch.empty_like(x), torch.zeros_like(c), torch.zeros_like(c)
    R.cut_cross_entropy(l0, gx0, gc0, x, c, t)
    M.cut_cross_entropy_forward_backward(l1, gx1, gc1, x, c, t, rows, None, 1.0)
    assert abs(float(l0) - float(l1)) < 1e-5 * max(1.0, abs(float(l0)))
    assert_close(host(gx1), host(gx0), 1e-4, "cce grad input")
    assert_close(host(gc1), host(gc0), 1e-4, "cce grad classifier", metric="max")


@pytest.mark.parametrize("b,s,hq,hkv,d", [(2, 256, 12, 4, 64), (1, 256, 8, 2, 128), (2, 192, 4, 2, 64)])
def test_attention(ops, b, s, hq, hkv, d):
    q, k, v, do = rnd(b, s, hq, d), rnd(b, s, hkv, d, seed=1), rnd(b, s, hkv, d, seed=2), rnd(b, s, hq, d, seed=3)
    opts = ops.FlashAttentionOptions(hq, hkv, d)
    o0, o1 = torch.empty_like(q), torch.empty_like(q)
    l0, l1 = torch.empty(b, s, hq, device="cuda"), torch.empty(b, s, hq, device="cuda")
    R.attention_forward(o0, l0, q, k, v)
    ops.flash_gqa_attention_forward_with_lse(o1, l1, q, k, v, None, opts)
    assert_close(host(o1), host(o0), 4e-3, "attention output")
    assert float((l0 - l1).abs().max()) < 2e-3
    grads = []
    for fn, o, l in ((R.attention_backward, o0, l0), (None, o0, l0)):
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        if fn is not None:
            fn(dq, dk, dv, do, o, l, q, k, v)
        else:
            ops.flash_gqa_attention_backward_with_lse(dq, dk, dv, do, o, l, q, k, v, None, opts)
        grads.append((dq, dk, dv))
    if d == 128:        # the reference's tensor-core path: fp32 accumulation on both sides
        for name, a, r in zip(("dq", "dk", "dv"), grads[1], grads[0]):
            assert_close(host(a), host(r), 1e-2, "attention " + name)
        return
    # head_dim 64 takes the reference's scalar path, which sums dK/dV with fp16 atomicAdd of fp16-rounded partials
    # (src/ops/backward/attention_backward.cu:76-80,491-492): its own rounding noise grows with the number of query
    # rows per key and differs from run to run (observed 1.5e-2 .. 3.7e-2 on identical inputs). Both are therefore
    # measured against the fp32 restatement: ours must meet the 1e-2 bar and must not be further from it than the
    # reference's kernels are; the direct comparison only guards against a gross mismatch (1e-1).
    from gpu_util import scaled_err
    from oracle import cgpt_oracle as O
    want = O.attention_backward(host(do), host(q), host(k), host(v), host(o0), host(l0), True, 0, 0.0)
    for name, a, r, w in zip(("dq", "dk", "dv"), grads[1], grads[0], want):
        ours, theirs = scaled_err(host(a), w), scaled_err(host(r), w)
        assert ours <= 1e-2, f"attention {name}: {ours:.3e} against the fp32 restatement"
        assert ours <= theirs + 2e-3, f"attention {name}: ours {ours:.3e}, reference kernels {theirs:.3e}"
        assert_close(host(a), host(r), 1e-1, "attention " + name + " (reference scalar path)")
