"""GPU parity of the tcgen05 GEMM / linear forward / linear backward (through the C ABI).

The contraction is a floating-point kernel, so it is compared with a plain fp32 matmul of the same
16-bit inputs (torch on the GPU, numpy oracle for the reference's known answers). Tolerance: the output
is rounded once to the storage dtype, so the norm-scaled max error must stay below 4e-3 (fp16) /
3e-2 (bf16); the parity bar for fp16-path gradients is 1e-2.
"""
import numpy as np
import pytest
import torch

import known_answers as KA
from gpu_util import assert_close, dev, host
from oracle import cgpt_oracle as O

pytestmark = pytest.mark.gpu
TOL = {torch.float16: 4e-3, torch.bfloat16: 3e-2, torch.float32: 1e-5}


@pytest.fixture(scope="module")
def ops():
    from cgpt_b200 import ops as m
    return m


def _operands(m, n, k, a_layout, b_layout, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn((k, m) if a_layout else (m, k), generator=g, device="cuda").to(dtype)
    b = torch.randn((k, n) if b_layout else (n, k), generator=g, device="cuda").to(dtype)
    a32 = a.float().t() if a_layout else a.float()
    b32 = b.float() if b_layout else b.float().t()
    return a, b, a32 @ b32


SHAPES = [(128, 128, 64), (128, 128, 16), (128, 256, 128), (256, 128, 192), (128, 128, 1024), (384, 640, 1000),
          (200, 136, 72), (4096, 1024, 1024), (1024, 1024, 8192), (256, 1024, 8192), (2048, 1024, 4096), (512, 32000, 256)]


@pytest.mark.parametrize("a_layout,b_layout", [(0, 0), (0, 1), (1, 1), (1, 0)])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_f16_layouts(ops, m, n, k, a_layout, b_layout):
    a, b, want = _operands(m, n, k, a_layout, b_layout, torch.float16, m + n + k)
    c = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float16)
    ops.gemm(c, a, b, m, n, k, a_layout, b_layout)
    torch.cuda.synchronize()
    assert_close(host(c), host(want) / 1.0, TOL[torch.float16], f"gemm {m}x{n}x{k} layouts {a_layout}{b_layout}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gemm_other_dtypes(ops, dtype):
    for a_layout, b_layout in [(0, 0), (0, 1), (1, 1)]:
        a, b, want = _operands(256, 384, 512, a_layout, b_layout, dtype, 9)
        c = torch.empty((256, 384), device="cuda", dtype=dtype)
        ops.gemm(c, a, b, 256, 384, 512, a_layout, b_layout)
        assert_close(host(c), host(want), TOL[dtype], f"{dtype} {a_layout}{b_layout}")


def test_gemm_accumulate_and_simt_agree(ops):
    a, b, want = _operands(256, 256, 512, 0, 1, torch.float16, 4)
    c0 = torch.randn((256, 256), device="cuda").half()
    c = c0.clone()
    ops.gemm(c, a, b, 256, 256, 512, 0, 1, accumulate=True)
    assert_close(host(c), host(want + c0.float()), TOL[torch.float16], "accumulate")
    c2 = c0.clone()
    ops.gemm(c2, a, b, 256, 256, 512, 0, 1, accumulate=True, force_simt=True)
    assert_close(host(c2), host(c), 4e-3, "simt vs tensor core")   # each is rounded to fp16 independently


def test_linear_backward_known_answers(ops):
    c = KA.LINEAR_BWD
    x, w, dy = dev(c["input"]), dev(c["weight"]), dev(c["grad_output"])
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty(2, device="cuda")
    ops.linear_backward(dx, dw, db, dy, x, w)
    np.testing.assert_allclose(host(dx), c["grad_input"], atol=1e-5); np.testing.assert_allclose(host(dw), c["grad_weight"], atol=1e-5)
    np.testing.assert_allclose(host(db), c["grad_bias"], atol=1e-5)
    ops.linear_backward(dx, dw, db, dy, x, w, None, None, ops.LinearBackwardOptions(accumulate_input=True, accumulate_weight=True, accumulate_bias=True))
    np.testing.assert_allclose(host(dx), 2 * c["grad_input"], atol=1e-5); np.testing.assert_allclose(host(dw), 2 * c["grad_weight"], atol=1e-5)
    np.testing.assert_allclose(host(db), 2 * c["grad_bias"], atol=1e-5)
    c = KA.LINEAR_BWD_F16
    x, w, dy = dev(c["input"], "f16"), dev(c["weight"], "f16"), dev(c["grad_output"], "f16")
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty(3, device="cuda", dtype=torch.float16)
    ops.linear_backward(dx, dw, db, dy, x, w)
    np.testing.assert_allclose(host(dx), c["grad_input"], atol=0.1); np.testing.assert_allclose(host(dw), c["grad_weight"], atol=0.2)
    np.testing.assert_allclose(host(db), c["grad_bias"], atol=0.1)


@pytest.mark.parametrize("rows,inf,outf", [(256, 256, 256), (256, 256, 688), (256, 688, 256), (4096, 1024, 2048), (512, 768, 32000), (1000, 64, 128)])
def test_linear_forward_backward_model_shapes(ops, rows, inf, outf):
    g = torch.Generator(device="cuda").manual_seed(rows + inf)
    x = torch.randn((rows, inf), generator=g, device="cuda").half()
    w = (0.05 * torch.randn((outf, inf), generator=g, device="cuda")).half()
    dy = torch.randn((rows, outf), generator=g, device="cuda").half()
    y, dx, dw = torch.empty((rows, outf), device="cuda", dtype=torch.float16), torch.empty_like(x), torch.empty_like(w)
    db = torch.empty(outf, device="cuda", dtype=torch.float16)
    ops.linear_forward(y, x, w)
    ops.linear_backward(dx, dw, db, dy, x, w)
    assert_close(host(y), host(x.float() @ w.float().t()), 4e-3, "y")
    assert_close(host(dx), host(dy.float() @ w.float()), 4e-3, "dx")
    assert_close(host(dw), host(dy.float().t() @ x.float()), 4e-3, "dw")
    assert_close(host(db), host(dy.float().sum(0)), 4e-3, "db")
    dx2 = dx.clone()
    ops.linear_backward(dx2, None, None, dy, x, w, None, None, ops.LinearBackwardOptions(accumulate_input=True))
    assert_close(host(dx2), 2 * host(dy.float() @ w.float()), 5e-3, "dx accumulate")


def test_device_status_clean(ops):
    from cgpt_b200 import _lib
    assert _lib.device_status(clear=False) == 0, "a tensor-core kernel gave up on a bounded wait"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,in_f,outs", [(512, 256, (256, 64, 64)), (4096, 1024, (1024, 256, 256)), (1000, 136, (200, 72)),
                                            (2048, 1024, (2048, 2048)), (256, 128, (64,))])
def test_linear_backward_input_fused(ops, dtype, rows, in_f, outs):
    """dX = sum_i dY_i W_i in one launch against the fp32 sum of matmuls; also with accumulation into dX."""
    g = torch.Generator(device="cuda").manual_seed(rows + in_f + len(outs))
    dys = [torch.randn(rows, o, generator=g, device="cuda").to(dtype) for o in outs]
    ws = [(torch.randn(o, in_f, generator=g, device="cuda") * 0.05).to(dtype) for o in outs]
    want = sum(dy.float() @ w.float() for dy, w in zip(dys, ws))
    dx = torch.full((rows, in_f), float("nan"), device="cuda", dtype=dtype)
    ops.linear_backward_input_fused(dx, dys, ws)
    torch.cuda.synchronize()
    assert_close(host(dx), host(want), TOL[dtype], f"fused dX {dtype} {rows}x{in_f} {outs}")
    base = torch.randn(rows, in_f, generator=g, device="cuda").to(dtype)
    dx2 = base.clone()
    ops.linear_backward_input_fused(dx2, dys, ws, accumulate_input=True)
    assert_close(host(dx2), host(want + base.float()), TOL[dtype], f"fused dX accumulate {dtype}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,out_f,ins", [(512, 256, (256, 512)), (4096, 1024, (1024, 2048)), (1000, 136, (200, 72)),
                                            (300, 320, (64,)), (256, 64, (128, 128, 32)), (2048, 1000, (256, 64))])
def test_linear_forward_sum(ops, dtype, rows, out_f, ins):
    """Y = R + sum_i X_i W_i^T in one launch against the fp32 sum of matmuls: shapes the CTA-pair epilogue takes (also with
    a ragged last row tile, 300 rows), shapes that fall back to product + elementwise add (out % 64 != 0, fp32), no
    residual, and Y aliasing R."""
    g = torch.Generator(device="cuda").manual_seed(rows + out_f + len(ins))
    xs = [torch.randn(rows, i, generator=g, device="cuda").to(dtype) for i in ins]
    ws = [(torch.randn(out_f, i, generator=g, device="cuda") * 0.05).to(dtype) for i in ins]
    r = torch.randn(rows, out_f, generator=g, device="cuda").to(dtype)
    prod = sum(x.float() @ w.float().T for x, w in zip(xs, ws))
    y = torch.full((rows, out_f), float("nan"), device="cuda", dtype=dtype)
    ops.linear_forward_sum(y, xs, ws, r)
    torch.cuda.synchronize()
    assert_close(host(y), host(prod + r.float()), TOL[dtype], f"sum of projections + residual {dtype} {rows}x{out_f} {ins}")
    y2 = torch.full_like(y, float("nan"))
    ops.linear_forward_sum(y2, xs, ws)
    assert_close(host(y2), host(prod), TOL[dtype], "sum of projections")
    pair_epilogue = dtype != torch.float32 and out_f % 64 == 0 and out_f >= 256 and rows >= 256
    y3 = r.clone()
    if pair_epilogue:      # in place over the residual: every element is read by the thread that later stores its tile row
        ops.linear_forward_sum(y3, xs, ws, y3)
        assert torch.equal(y3, y)
    else:
        with pytest.raises(Exception):
            ops.linear_forward_sum(y3, xs, ws, y3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,in_f,inter", [(256, 128, 128), (4096, 1024, 2048), (1000, 136, 200), (384, 256, 688)])
def test_linear_swiglu_forward(ops, dtype, rows, in_f, inter):
    """Fused gate/up/activation against the three separate operators (same rounding points) and the fp32 matmul."""
    g = torch.Generator(device="cuda").manual_seed(rows + inter)
    x = torch.randn(rows, in_f, generator=g, device="cuda").to(dtype)
    wg = (torch.randn(inter, in_f, generator=g, device="cuda") * 0.1).to(dtype)
    wu = (torch.randn(inter, in_f, generator=g, device="cuda") * 0.1).to(dtype)
    gate, up, act = (torch.full((rows, inter), float("nan"), device="cuda", dtype=dtype) for _ in range(3))
    ops.linear_swiglu_forward(gate, up, act, x, wg, wu)
    g_ref, u_ref, a_ref = torch.empty_like(gate), torch.empty_like(up), torch.empty_like(act)
    ops.linear_forward(g_ref, x, wg)
    ops.linear_forward(u_ref, x, wu)
    ops.swiglu_forward(a_ref, g_ref, u_ref)
    torch.cuda.synchronize()
    assert_close(host(gate), host(x.float() @ wg.float().t()), TOL[dtype], "gate vs fp32")
    assert_close(host(up), host(x.float() @ wu.float().t()), TOL[dtype], "up vs fp32")
    assert torch.equal(gate, g_ref) and torch.equal(up, u_ref), "projections differ from linear_forward"
    assert torch.equal(act, a_ref), "activation differs from swiglu_forward on the stored projections"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,in_f,outs", [(32768, 1024, (1024, 256, 256)), (4096, 256, (256, 128, 128)), (1000, 136, (200, 72)),
                                            (256, 128, (64,)), (20000, 512, (512, 512, 1024))])
def test_linear_forward_fused(ops, dtype, rows, in_f, outs):
    """Several projections of one input in one launch: bit-identical to the separate linear_forward calls."""
    g = torch.Generator(device="cuda").manual_seed(rows + in_f + len(outs))
    x = torch.randn(rows, in_f, generator=g, device="cuda").to(dtype)
    ws = [(torch.randn(o, in_f, generator=g, device="cuda") * 0.05).to(dtype) for o in outs]
    ys = [torch.full((rows, o), float("nan"), device="cuda", dtype=dtype) for o in outs]
    ops.linear_forward_fused(ys, x, ws)
    for y, w in zip(ys, ws):
        ref = torch.empty_like(y)
        ops.linear_forward(ref, x, w)
        torch.cuda.synchronize()
        assert torch.equal(y, ref), f"fused projection {tuple(w.shape)} differs from linear_forward"
        assert_close(host(y[:512]), host(x[:512].float() @ w.float().t()), TOL[dtype], "fused projection vs fp32")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,in_f,outs", [(32768, 1024, (1024, 256, 256)), (8192, 1024, (2048, 2048)), (4096, 256, (256, 128, 128)),
                                            (1000, 264, (200, 72)), (512, 512, (64,)), (20000, 512, (512, 384, 1024))])
def test_linear_backward_weight_fused(ops, dtype, rows, in_f, outs):
    """dW_i = dY_i^T X for several projections of one input in one launch, against the fp32 products, with and without
    accumulation into dW."""
    g = torch.Generator(device="cuda").manual_seed(rows + in_f + len(outs))
    x = torch.randn(rows, in_f, generator=g, device="cuda").to(dtype)
    dys = [(torch.randn(rows, o, generator=g, device="cuda") * 0.05).to(dtype) for o in outs]
    want = [dy.float().t() @ x.float() for dy in dys]
    gws = [torch.full((o, in_f), float("nan"), device="cuda", dtype=dtype) for o in outs]
    ops.linear_backward_weight_fused(gws, dys, x)
    torch.cuda.synchronize()
    tol = 2 * TOL[dtype] if dtype != torch.float32 else 1e-4       # K = rows: long fp32 sums, one rounding
    for gw, w in zip(gws, want):
        assert_close(host(gw), host(w), tol, f"fused dW {dtype} {tuple(gw.shape)}")
    base = [torch.randn(o, in_f, generator=g, device="cuda").to(dtype) for o in outs]
    acc = [b.clone() for b in base]
    ops.linear_backward_weight_fused(acc, dys, x, accumulate_weight=True)
    for a, b, w in zip(acc, base, want):
        assert_close(host(a), host(w + b.float()), tol, f"fused dW accumulate {dtype}")
