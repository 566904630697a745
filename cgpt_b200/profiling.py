"""Live measurement helpers used by bench.py (CUDA events recorded by the library around its own launches)."""
from __future__ import annotations

import ctypes as C

import os

import torch

from ._lib import check, lib


def model_flops_per_token(options) -> float:
    """Model FLOPs per token of one training step: 6 x matmul weights (forward + two backward products, LM head
    counted once per use, embedding lookup 0) + causal attention forward (4*S*d/2) and backward (2.5x forward)."""
    b = options.block_options
    qd, kvd = b.num_query_heads * b.head_dim, b.num_kv_heads * b.head_dim
    per_layer = b.hidden_size * (qd + 2 * kvd) + qd * b.hidden_size + 3 * b.hidden_size * b.intermediate_size
    n_mm = options.num_layers * per_layer + options.vocabulary_size * b.hidden_size
    return 6.0 * n_mm


def attention_flops_per_token(options, seq: int) -> float:
    b = options.block_options
    fwd = 4.0 * seq * b.num_query_heads * b.head_dim / 2.0          # QK^T and PV, causal half
    return options.num_layers * (fwd + 2.5 * fwd)


def time_gemms(train_step, steps: int = 2) -> dict:
    """Runs `steps` eager (non-graph) model steps with event pairs around every tensor-core GEMM launch and returns
    the per-step totals: ms inside the kernel, algorithmic TFLOP/s, launches, and the model FLOPs of a step."""
    ts = train_step
    # one stream for this pass: with the block's two branches on two streams a GEMM's event pair would also span the
    # time it waits for SMs held by the other branch's kernels
    check(lib.cgpt_b200_set_branch_streams(0), "set_branch_streams")
    check(lib.cgpt_b200_gemm_timing(1), "gemm_timing")
    reducer, ts._reducer = getattr(ts, "_reducer", None), None    # this pass runs on one rank only: no collectives
    try:
        with torch.cuda.stream(ts.stream):
            # Head start for the host: the event pairs bracket GPU time, and a launch the host has not submitted yet when
            # the GPU reaches its first event would put the GPU's wait for the host inside the bracket. 40 ms of spinning
            # on the stream lets the host enqueue the whole pass before the GPU starts it.
            torch.cuda._sleep(int(0.040 * 1.9e9))
            for _ in range(steps):
                ts.enqueue_model_step()
        ts.stream.synchronize()
        ms, fl, n = C.c_double(0), C.c_double(0), C.c_uint64(0)
        check(lib.cgpt_b200_gemm_timing_read(C.byref(ms), C.byref(fl), C.byref(n)), "gemm_timing_read")
    finally:
        ts._reducer = reducer
        check(lib.cgpt_b200_gemm_timing(0), "gemm_timing")
        check(lib.cgpt_b200_set_branch_streams(int(os.environ.get("CGPT_B200_BRANCH_STREAMS", "0") == "1")), "set_branch_streams")
    tokens = ts.batch * ts.seq
    model = (model_flops_per_token(ts.options) + attention_flops_per_token(ts.options, ts.seq)) * tokens
    return {"ms": ms.value / steps, "tflops": fl.value / ms.value / 1e9 if ms.value > 0 else 0.0,
            "launches": int(n.value) // steps, "gemm_flops": fl.value / steps, "model_flops": model}


def time_cut_cross_entropy(rows: int, hidden: int, vocab: int, iters: int = 5, form: int = 0) -> dict:
    """The loss layer alone: cut cross-entropy forward + backward (loss, dX, dC) on fp16 N(0,1) activations, an N(0,0.02)
    classifier and uniform targets, gradient scale 1024. Credited work: three products of 2*rows*vocab*hidden FLOPs (logits,
    dX, dC); algorithmic bytes: X, C, dX, dC and the targets. Time: CUDA events around `iters` calls after 2 warm-up calls."""
    from . import model as M
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(rows, hidden, generator=g, device="cuda").half()
    c = (torch.randn(vocab, hidden, generator=g, device="cuda") * 0.02).half()
    t = torch.randint(0, vocab, (rows,), generator=g, device="cuda", dtype=torch.int32)
    loss = torch.zeros(1, device="cuda")
    dx, dc = torch.empty_like(x), torch.empty_like(c)
    fn = lambda: M.cut_cross_entropy_forward_backward(loss, dx, dc, x, c, t, rows, None, 1024.0, form=form)
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    flops = 3.0 * 2.0 * rows * vocab * hidden
    return {"shape": f"{rows} x {hidden} x {vocab}", "form": form, "us": ms * 1e3, "tflops": flops / ms / 1e9, "credited_flops": flops,
            "algorithmic_bytes": 2.0 * 2 * (rows * hidden + vocab * hidden) + 4 * rows, "loss": float(loss.item())}


def time_cut_cross_entropy_forms(rows: int, hidden: int, vocab: int, rounds: int = 3, iters: int = 3) -> dict:
    """The three forms of the loss layer side by side on the same inputs (see time_cut_cross_entropy). The forms are timed
    in turn, `rounds` times over, and the median per form is reported, so that a drifting power-capped clock does not
    favour whichever form runs first."""
    from . import model as M
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(rows, hidden, generator=g, device="cuda").half()
    c = (torch.randn(vocab, hidden, generator=g, device="cuda") * 0.02).half()
    t = torch.randint(0, vocab, (rows,), generator=g, device="cuda", dtype=torch.int32)
    loss = torch.zeros(1, device="cuda")
    dx, dc = torch.empty_like(x), torch.empty_like(c)
    names = {1: "rows", 2: "tiles", 3: "recompute"}
    times = {f: [] for f in names}
    for f in names:     # warm-up: scratch arena, kernel attributes
        M.cut_cross_entropy_forward_backward(loss, dx, dc, x, c, t, rows, None, 1024.0, form=f)
    torch.cuda.synchronize()
    for _ in range(rounds):
        for f in names:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                M.cut_cross_entropy_forward_backward(loss, dx, dc, x, c, t, rows, None, 1024.0, form=f)
            e1.record()
            torch.cuda.synchronize()
            times[f].append(e0.elapsed_time(e1) / iters)
    flops = 3.0 * 2.0 * rows * vocab * hidden
    out = {}
    for f, name in names.items():
        ms = sorted(times[f])[len(times[f]) // 2]
        out[name] = {"us": ms * 1e3, "tflops": flops / ms / 1e9}
    return out


def time_attention_backward(batch: int, seq: int, q_heads: int, kv_heads: int, head_dim: int, iters: int = 10) -> dict:
    """Standalone causal GQA attention backward (flash_gqa_attention_backward_with_lse) on seeded N(0,1) fp16 inputs, O and
    the logsumexp taken from the forward on the same inputs. Time: CUDA events around `iters` back-to-back calls after 3
    warm-up calls; a call's inputs and outputs exceed L2. FLOPs: 5 products of 2*S*S*D per (batch, query head), causal
    half; the recomputation the kernels do beyond those 5 is not credited."""
    from . import ops
    g = torch.Generator(device="cuda").manual_seed(2)
    n = lambda *s: torch.randn(*s, generator=g, device="cuda").half()
    q, k, v = n(batch, seq, q_heads, head_dim), n(batch, seq, kv_heads, head_dim), n(batch, seq, kv_heads, head_dim)
    do = n(batch, seq, q_heads, head_dim)
    o, lse = torch.empty_like(q), torch.empty(batch, seq, q_heads, device="cuda")
    opts = ops.FlashAttentionOptions(q_heads, kv_heads, head_dim)
    ops.flash_gqa_attention_forward_with_lse(o, lse, q, k, v, None, opts)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    run = lambda: ops.flash_gqa_attention_backward_with_lse(dq, dk, dv, do, o, lse, q, k, v, None, opts)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    flops = 5.0 * 2.0 * seq * seq * head_dim * batch * q_heads / 2.0
    return {"shape": f"B{batch} S{seq} Hq{q_heads}/Hkv{kv_heads} D{head_dim} fp16 causal", "us": ms * 1e3,
            "tflops": flops / ms / 1e9, "flops": flops}


def main() -> None:
    """`python -m cgpt_b200.profiling [--steps K] [--warmup W] [--preset 104m] [--batch 32] [--seq 1024]`:
    runs eager (no CUDA graph) training steps so that a profiler sees every kernel launch of a step; prints the
    mean step time. Used for launch lists and profiler captures of the step."""
    import argparse

    from . import model as M
    from .train import TrainStep

    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--preset", default="104m")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=1024)
    args = ap.parse_args()
    opts = M.preset(args.preset)
    ts = TrainStep(opts, args.batch, args.seq, seed=0, use_graph=False)
    ts.token_ids.copy_(torch.randint(0, opts.vocabulary_size, (args.batch * args.seq,), dtype=torch.int32))
    ts.targets.copy_(torch.randint(0, opts.vocabulary_size, (args.batch * args.seq,), dtype=torch.int32))
    for _ in range(args.warmup):
        ts.step()
    ts.stream.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(ts.stream):
        e0.record()
    for _ in range(args.steps):
        ts.step()
    with torch.cuda.stream(ts.stream):
        e1.record()
    ts.stream.synchronize()
    print(f"eager step: {e0.elapsed_time(e1) / args.steps:.3f} ms, loss {ts.read_loss():.4f}")


if __name__ == "__main__":
    main()
