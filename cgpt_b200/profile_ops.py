"""`python -m cgpt_b200.profile_ops <op> [--iters N]`: launches one operator a few times on inputs larger
than L2 but a few hundred MB at most, so that `ncu -k regex:<kernel>` captures of it end by themselves.
Ops: gemm_fwd, gemm_dx, gemm_dw, linear_sum (output + down projection + residual as one product), attention_fwd,
attention_bwd, rmsnorm_bwd, rmsnorm_dual_fwd, rmsnorm_dual_bwd (both norms of one input in one pass), swiglu_bwd, rope_bwd, embedding_bwd, adamw,
cross_entropy, cce (one 8192-row chunk of the cut cross-entropy at hidden 1024, vocabulary 32000; --cce-form 1|2|3),
qknorm_fwd, qknorm_bwd.
Prints the CUDA-event time per launch (taken without a profiler attached it is the number to quote)."""
from __future__ import annotations

import argparse

import torch

from . import ops, optim


def _run(fn, iters):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("op")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--attention-shape", choices=["104m", "d64"], default="104m",
                    help="attention ops: 8/2 heads of 128 (the 104m layer) or 12/4 heads of 64")
    ap.add_argument("--cce-form", type=int, default=0, help="cce: 0 default, 1 row kernel, 2 tile statistics, 3 recompute")
    ap.add_argument("--rows", type=int, default=8192, help="cce: rows (8192 is one chunk)")
    ap.add_argument("--cce-chunk", type=int, default=0, help="cce: rows per chunk (0 = the library's choice)")
    a = ap.parse_args()
    h = lambda *s: torch.randn(*s, device="cuda").half()
    T, d, I = 32768, 1024, 2048
    if a.op in ("gemm_fwd", "gemm_dx", "gemm_dw"):
        x, w, dy = h(T, d), h(I, d) * 0.02, h(T, I)
        y, dx, dw = torch.empty(T, I, device="cuda", dtype=torch.float16), torch.empty_like(x), torch.empty_like(w)
        fn = {"gemm_fwd": lambda: ops.linear_forward(y, x, w),
              "gemm_dx": lambda: ops.linear_backward(dx, None, None, dy, x, w),
              "gemm_dw": lambda: ops.linear_backward(None, dw, None, dy, x, w)}[a.op]
        ms = _run(fn, a.iters)
        print(f"{a.op} {T}x{I}x{d}: {ms * 1e3:.1f} us, {2.0 * T * d * I / ms / 1e9:.1f} TFLOP/s")
    elif a.op in ("attention_fwd", "attention_bwd"):
        B, S, Hq, Hkv, D = (32, 1024, 8, 2, 128) if a.attention_shape == "104m" else (32, 1024, 12, 4, 64)
        q, k, v, do = h(B, S, Hq, D), h(B, S, Hkv, D), h(B, S, Hkv, D), h(B, S, Hq, D)
        o, lse = torch.empty_like(q), torch.empty(B, S, Hq, device="cuda")
        opts = ops.FlashAttentionOptions(Hq, Hkv, D)
        ops.flash_gqa_attention_forward_with_lse(o, lse, q, k, v, None, opts)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        fwd = 4.0 * S * S * D * Hq * B / 2
        if a.op == "attention_fwd":
            ms = _run(lambda: ops.flash_gqa_attention_forward_with_lse(o, lse, q, k, v, None, opts), a.iters)
            print(f"attention_fwd B{B} S{S} {Hq}/{Hkv} D{D}: {ms * 1e3:.1f} us, {fwd / ms / 1e9:.1f} TFLOP/s")
        else:
            ms = _run(lambda: ops.flash_gqa_attention_backward_with_lse(dq, dk, dv, do, o, lse, q, k, v, None, opts), a.iters)
            print(f"attention_bwd B{B} S{S} {Hq}/{Hkv} D{D}: {ms * 1e3:.1f} us, {2.5 * fwd / ms / 1e9:.1f} TFLOP/s (5 GEMMs, causal half)")
    elif a.op == "rmsnorm_bwd":
        x, dy, w = h(T, d), h(T, d), torch.ones(d, device="cuda", dtype=torch.float16)
        dx, dw = torch.empty_like(x), torch.empty_like(w)
        ms = _run(lambda: ops.rmsnorm_backward(dx, dw, dy, x, w, 1e-5), a.iters)
        print(f"rmsnorm_bwd {T}x{d}: {ms * 1e3:.1f} us, {3.0 * T * d * 2 / ms / 1e6:.0f} GB/s algorithmic")
    elif a.op == "rmsnorm_dual_bwd":
        x, da, db, res = h(T, d), h(T, d), h(T, d), h(T, d)
        wa, wb = torch.ones(d, device="cuda", dtype=torch.float16), torch.ones(d, device="cuda", dtype=torch.float16)
        dx, dwa, dwb = torch.empty_like(x), torch.empty_like(wa), torch.empty_like(wb)
        ms = _run(lambda: ops.rmsnorm_backward_dual(dx, dwa, dwb, da, db, x, wa, wb, 1e-5, residual=res), a.iters)
        print(f"rmsnorm_dual_bwd {T}x{d} (+ residual): {ms * 1e3:.1f} us, {5.0 * T * d * 2 / ms / 1e6:.0f} GB/s algorithmic")
    elif a.op == "rmsnorm_dual_fwd":
        x = h(T, d)
        wa, wb = torch.ones(d, device="cuda", dtype=torch.float16), torch.ones(d, device="cuda", dtype=torch.float16)
        ya, yb = torch.empty_like(x), torch.empty_like(x)
        ms = _run(lambda: ops.rmsnorm_forward_dual(ya, yb, x, wa, wb, 1e-5), a.iters)
        print(f"rmsnorm_dual_fwd {T}x{d}: {ms * 1e3:.1f} us, {3.0 * T * d * 2 / ms / 1e6:.0f} GB/s algorithmic")
    elif a.op == "linear_sum":
        xa, xb, res = h(T, d), h(T, I), h(T, d)
        wo, wd = h(d, d) * 0.02, h(d, I) * 0.02
        y = torch.empty_like(res)
        ms = _run(lambda: ops.linear_forward_sum(y, [xa, xb], [wo, wd], res), a.iters)
        print(f"linear_sum {T}x{d}x({d}+{I}) + residual: {ms * 1e3:.1f} us, {2.0 * T * d * (d + I) / ms / 1e9:.1f} TFLOP/s")
    elif a.op == "swiglu_bwd":
        g, u, dy = h(T, I), h(T, I), h(T, I)
        dg, du = torch.empty_like(g), torch.empty_like(g)
        ms = _run(lambda: ops.swiglu_backward(dg, du, dy, g, u), a.iters)
        print(f"swiglu_bwd {T}x{I}: {ms * 1e3:.1f} us, {5.0 * T * I * 2 / ms / 1e6:.0f} GB/s algorithmic")
    elif a.op == "rope_bwd":
        from . import model
        B, S, Hq, Hkv, D = (32, 1024, 8, 2, 128) if a.attention_shape == "104m" else (32, 1024, 12, 4, 64)
        gq, gk = h(B, S, Hq, D), h(B, S, Hkv, D)
        dq, dk = torch.empty_like(gq), torch.empty_like(gk)
        cos, sin = model.rotary_cache(S, D)
        ms = _run(lambda: ops.rope_backward(dq, dk, gq, gk, cos, sin), a.iters)
        print(f"rope_bwd B{B} S{S} {Hq}/{Hkv} D{D}: {ms * 1e3:.1f} us, {2.0 * (gq.numel() + gk.numel()) * 2 / ms / 1e6:.0f} GB/s algorithmic")
    elif a.op == "embedding_bwd":
        V = 32000
        dy, ids = h(T, d), torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
        gw = torch.empty(V, d, device="cuda", dtype=torch.float16)
        ms = _run(lambda: ops.embedding_backward(gw, dy, ids, T), a.iters)
        print(f"embedding_bwd {T} tokens x {d} into {V} rows: {ms * 1e3:.1f} us (sort + owner-row kernel), "
              f"{(T * d * 2 + V * d * 2 + 4 * T) / ms / 1e6:.0f} GB/s algorithmic")
    elif a.op == "cross_entropy":
        rows, V = 8192, 32000
        z, t = h(rows, V), torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
        loss = torch.zeros(1, device="cuda")
        ms = _run(lambda: ops.cross_entropy_forward_backward(loss, z, z, t, rows, None, 1024.0), a.iters)
        print(f"cross_entropy {rows}x{V} in place: {ms * 1e3:.1f} us, {2.0 * rows * V * 2 / ms / 1e6:.0f} GB/s algorithmic")
    elif a.op == "cce":
        from . import model as M
        rows, V = a.rows, 32000
        x, c = h(rows, d), h(V, d) * 0.02
        t = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
        loss, dx, dc = torch.zeros(1, device="cuda"), torch.empty_like(x), torch.empty_like(c)
        ms = _run(lambda: M.cut_cross_entropy_forward_backward(loss, dx, dc, x, c, t, rows, None, 1024.0, form=a.cce_form,
                                                               chunk_rows=a.cce_chunk), a.iters)
        print(f"cce form {a.cce_form} chunk {a.cce_chunk} {rows}x{d}x{V}: {ms * 1e3:.1f} us, {3 * 2.0 * rows * d * V / ms / 1e9:.1f} TFLOP/s on 3 products, "
              f"loss {float(loss.item()):.6f}")
    elif a.op == "adamw":
        sizes = [32000 * 1024] + [1024 * 1024, 2048 * 1024, 2048 * 1024, 1024 * 2048] * 8
        ps = [h(n) * 0.02 for n in sizes]
        gs = [h(n) for n in sizes]
        sts = [optim.AdamWState.for_parameter(p) for p in ps]
        ws = optim.AdamWWorkspace()
        ent = [optim.AdamWBatchEntry(p, g, s) for p, g, s in zip(ps, gs, sts)]
        o = optim.AdamWOptions(3e-4, 0.9, 0.95, 1e-8, 0.1, 1024.0, 1.0)
        ms = _run(lambda: optim.adamw_step_many_async(ent, o, ws), a.iters)
        n = sum(sizes)
        print(f"adamw {n / 1e6:.1f}M params: {ms * 1e3:.1f} us, {30.0 * n / ms / 1e6:.0f} GB/s algorithmic (2+28 B/param)")
    elif a.op in ("qknorm_fwd", "qknorm_bwd"):
        from . import _lib, model
        B, S, Hq, Hkv, D = (32, 1024, 8, 2, 128) if a.attention_shape == "104m" else (32, 1024, 12, 4, 64)
        q, k, gq, gk = h(B, S, Hq, D), h(B, S, Hkv, D), h(B, S, Hq, D), h(B, S, Hkv, D)
        oq, ok = torch.empty_like(q), torch.empty_like(k)
        wq, wk = torch.ones(D, device="cuda").half(), torch.ones(D, device="cuda").half()
        dwq, dwk = torch.empty_like(wq), torch.empty_like(wk)
        cos, sin = model.rotary_cache(S, D)
        p = lambda t: t.data_ptr()
        st = torch.cuda.current_stream().cuda_stream
        if a.op == "qknorm_fwd":
            fn = lambda: _lib.check(_lib.lib.cgpt_qknorm_rope_forward(p(oq), p(ok), p(q), p(k), p(wq), p(wk), p(cos), p(sin), B, S, Hq,
                                                                      Hkv, D, D, 0, S, 1e-5, 0, st), "qknorm_rope_forward")
            nbytes = 2 * (q.numel() + k.numel()) * 2
        else:
            fn = lambda: _lib.check(_lib.lib.cgpt_qknorm_rope_backward(p(oq), p(ok), p(dwq), p(dwk), p(gq), p(gk), p(q), p(k), p(wq),
                                                                       p(wk), p(cos), p(sin), B, S, Hq, Hkv, D, D, 0, S, 1e-5, 0, st),
                                    "qknorm_rope_backward")
            nbytes = 3 * (q.numel() + k.numel()) * 2
        ms = _run(fn, a.iters)
        print(f"{a.op} B{B} S{S} {Hq}/{Hkv} D{D}: {ms * 1e3:.1f} us, {nbytes / ms / 1e6:.0f} GB/s algorithmic")
    else:
        raise SystemExit(f"unknown op {a.op}")


if __name__ == "__main__":
    main()
