"""`python -m cgpt_b200.profile_step --model 1.3b --batch 8 --seq 4096 [--steps 5]`: times the training step (forward,
cut-cross-entropy loss, backward, AdamW) of any preset at any batch shape on one GPU, with CUDA events on the step's stream
after 3 warm-up steps, and prints one JSON line: ms per step, tokens/s, model TFLOP/s (6 x matmul weights + causal
attention, per token), peak device memory. Synthetic uniform token ids, seeded N(0, 0.02) weights."""
from __future__ import annotations

import argparse
import json
import math

import torch

from . import _lib, model as M, profiling
from .train import TrainStep


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="104m")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--eager", action="store_true", help="issue every step eagerly instead of replaying the captured graph")
    a = ap.parse_args()
    opts = M.preset(a.model)
    ts = TrainStep(opts, a.batch, a.seq, seed=0, use_graph=not a.eager)
    ids = torch.randint(0, opts.vocabulary_size, (a.batch, a.seq + 1), dtype=torch.int32, generator=torch.Generator().manual_seed(1))
    ts.upload_batch(ids[:, :-1].contiguous().pin_memory(), ids[:, 1:].contiguous().pin_memory())
    ts.step()
    first_loss = ts.read_loss()
    for _ in range(2):
        ts.step()
    ts.stream.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(ts.stream):
        e0.record()
    for _ in range(a.steps):
        ts.step()
    with torch.cuda.stream(ts.stream):
        e1.record()
    ts.stream.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    rows = a.batch * a.seq
    flops = rows * (profiling.model_flops_per_token(opts) + profiling.attention_flops_per_token(opts, a.seq))
    print(json.dumps({"model": a.model, "parameters": ts.storage.num_parameters(), "batch": a.batch, "seq_len": a.seq,
                      "ms_per_step": ms, "tokens_per_s": rows / ms * 1e3, "model_tflops": flops / ms / 1e9,
                      "first_loss": first_loss, "ln_vocab": math.log(opts.vocabulary_size), "last_loss": ts.read_loss(),
                      "optimizer_ok": bool(ts.check()), "device_status": _lib.device_status(clear=False),
                      "peak_memory_gb": torch.cuda.max_memory_allocated() / 1e9}))


if __name__ == "__main__":
    main()
