"""Benchmark of the training hot path: one step = forward + cut-cross-entropy loss + backward + AdamW of the
reference's `104m` preset (8 layers, d 1024, 8 Q / 2 KV heads, head_dim 128, SwiGLU 2048, vocab 32000, tied
embedding) at batch 32 x seq 1024 per GPU, fp16 activations/weights, fp32 master weights, loss scale 1024.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 is launched with torch.distributed.run (one rank per GPU, NCCL): pure data parallelism, gradients
averaged with bucketed all-reduces, per-GPU work fixed (weak scaling). Rank 0 prints one JSON line.

`value` is whole-job tokens/s with the batch already in HBM, timed on the device (CUDA events, max over
ranks); `e2e` includes the pinned-host -> device copy of every step's token ids / targets and the
device -> host read of the loss. `roofline` describes the dominant kernel (the tcgen05 GEMM): algorithmic
FLOPs of the GEMM launches of one step / their summed CUDA-event durations, against the measured cuBLAS
bf16 peak in MEASURED_PEAKS.json. `cpu_baseline` times the reference's own CPU forward + loss (its only CPU
path for this model) on a bounded sample on the host cores.

`--impl reference` times only that CPU path (all host threads) and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "104m_train_tokens_per_s"
UNIT = "tokens/s"
PRESET = "104m"
BATCH, SEQ = 32, 1024
PUBLISHED_TOKENS_PER_S = 151400.0   # reference README.md:168 (4.62 steps/s at 32 x 1024, hardware not stated)


# DRAM bytes of one launch of the dominant kernel, from an ncu capture of its most frequent large shape in the step
# (python -m cgpt_b200.profile_ops gemm_fwd under ncu, CTA-pair kernel): dram__bytes_read.sum 71.4 MB + dram__bytes_write.sum 85.2 MB.
GEMM_TRAFFIC_BYTES = 156.6e6
GEMM_TRAFFIC_NOTE = ("ncu, one launch of the 32768x2048x1024 forward GEMM (algorithmic A+B+C = 205.5 MB; part of C is still "
                     "in L2 when the kernel ends); the step's 108 launches have other shapes, none re-reads its operands from DRAM")


def workload_config(n_gpus: int) -> dict:
    return {"workload": "cgpt 104m preset training step (L8 d1024 Hq8/Hkv2 D128 I2048 V32000 tied), fp16 + fp32 master, "
                        "loss scale 1024, AdamW lr 3e-4 b(.9,.95) wd .1 clip 1.0, cut-cross-entropy loss",
            "batch_per_gpu": BATCH, "seq_len": SEQ, "global_batch": BATCH * n_gpus, "parallelism": f"dp{n_gpus}",
            "l2": "working set per step (activations + weights, several GB) is far larger than the 126 MB L2; no flush needed"}


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons every 200 ms while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.samples, self.proc, self.thread, self.index = [], None, None, device_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self) -> dict:
        sm, mx, reasons = [], 0, set()
        for p in self.samples:
            try:
                sm.append(float(p[1])); mx = max(mx, float(p[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


# -------------------------------------------------------------------------------------------- CPU baseline
def cpu_baseline(threads: int | None, batch: int = 2, seq: int = 256, repeats: int = 3) -> dict:
    """Times the reference's CPU forward + cross-entropy loss of the 104m model (oracle/_ref, built from the
    reference's own src/ops/cpu sources) on a bounded sample of batch x seq tokens."""
    import numpy as np
    from oracle import ref_cpu
    if threads:
        os.environ["OMP_NUM_THREADS"] = str(threads)
    if not ref_cpu.available():
        return {"value": None, "unit": UNIT, "cores": 0, "kind": "reference", "sample": "oracle/_ref/libcgpt_ref_cpu.so is missing"}
    layers, d, hq, hkv, hd, inter, vocab = 8, 1024, 8, 2, 128, 2048, 32000
    rng = np.random.default_rng(0)
    per_layer = d + hq * hd * d + hkv * hd * d + hd + hd + hkv * hd * d + d * hq * hd + d + inter * d + inter * d + d * inter
    flat = (0.02 * rng.standard_normal(vocab * d + layers * per_layer + d)).astype(np.float32)
    # norm weights = 1 (positions inside the flat layout)
    off = vocab * d
    for _ in range(layers):
        flat[off:off + d] = 1; o2 = off + d + hq * hd * d + hkv * hd * d
        flat[o2:o2 + 2 * hd] = 1; o3 = o2 + 2 * hd + hkv * hd * d + d * hq * hd
        flat[o3:o3 + d] = 1
        off += per_layer
    flat[off:off + d] = 1
    tokens = rng.integers(0, vocab, (batch, seq + 1))
    secs, loss = ref_cpu.cpu_forward_loss(flat, tokens[:, :-1], tokens[:, 1:], batch, seq, layers, d, hq, hkv, hd, inter, vocab, 1e-5, repeats)
    cores = int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))
    return {"value": batch * seq / secs, "unit": UNIT, "cores": cores, "kind": "reference",
            "sample": f"reference CPU ops (src/ops/cpu, -O3 -mavx2 -mfma -mf16c, OpenMP) forward + cross-entropy loss only "
                      f"(the reference has no CPU training step), 104m model, batch {batch} x seq {seq}, median of {repeats}; "
                      f"linear_forward_cpu is single-threaded for rows > 1; {secs:.2f} s per pass, loss {loss:.4f}",
            "seconds_per_pass": secs}


def run_reference(args) -> None:
    """The reference arm: the reference's own CPU implementation of the path. It has no CPU training step, so what runs is
    its CPU forward + cross-entropy loss of the same 104m model on a bounded sample (2 x 256 tokens per pass); the line says
    so in `config.workload`, and a whole 32 x 1024 step is NOT timed: `ms_per_step` is null and the extrapolated figure is
    labelled as such."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1 to its ranks; the arm is meant to use every host core it can
    threads = os.cpu_count() or 1
    steps = max(1, min(args.steps, 3))
    sample_batch, sample_seq = 2, 256
    base = cpu_baseline(threads, batch=sample_batch, seq=sample_seq, repeats=steps)
    config = workload_config(args.gpus)
    config["workload"] = (f"reference CPU path of the same 104m model: forward + cross-entropy loss only, {sample_batch} x {sample_seq} tokens "
                          f"per pass, {steps} passes (the reference has no CPU backward/optimizer step; GPU arm: " + config["workload"] + ")")
    config["sample_tokens_per_pass"] = sample_batch * sample_seq
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": 0, "ms_per_step": None,
            "ms_per_32x1024_step_extrapolated": None if base["value"] is None else 1000.0 * BATCH * SEQ / base["value"],
            "ms_per_pass": None if base.get("seconds_per_pass") is None else 1000.0 * base["seconds_per_pass"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config, "cpu_baseline": {k: v for k, v in base.items() if k != "seconds_per_pass"},
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def reference_gpu_step(args) -> dict:
    """Informational: the reference's own training step on this GPU -- its trainer's tensors and calls
    (transformer_model_forward -> cross_entropy_forward_backward -> transformer_model_backward replayed from its CudaGraph,
    then adamw_step_many_async; train/train.cpp:536-556), its kernels rebuilt for sm_100a and cuBLASLt for the linears --
    on the same 104m shape and batch, timed with CUDA events; and its attention backward alone. Runs in a child process so
    that its 20 GB of buffers and its own failure modes stay out of the measured process."""
    code = (
        "import json, sys, torch\n"
        "sys.path.insert(0, %r)\n"
        "from oracle import ref_cuda as R\n"
        "from cgpt_b200 import model as M\n"
        "B, S, steps = %d, %d, %d\n"
        "o = M.preset('104m'); b = o.block_options\n"
        "cos, sin = M.rotary_cache(S, b.rotary_dim)\n"
        "ref = R.RefModel(o.vocabulary_size, o.num_layers, b.hidden_size, b.intermediate_size, b.num_query_heads, b.num_kv_heads,\n"
        "                 b.head_dim, b.rotary_dim, b.rms_epsilon, B, S, cos, sin)\n"
        "ref.init(0)\n"
        "g = torch.Generator(device='cuda').manual_seed(1)\n"
        "ids = torch.randint(0, o.vocabulary_size, (B * S,), generator=g, device='cuda', dtype=torch.int32)\n"
        "tg = torch.randint(0, o.vocabulary_size, (B * S,), generator=g, device='cuda', dtype=torch.int32)\n"
        "st = torch.cuda.Stream()\n"
        "def step():\n"
        "    ref.step(ids, tg, 1024.0, graph=True); ref.adamw(3e-4, 0.9, 0.95, 1e-8, 0.1, 1024.0, 1.0)\n"
        "with torch.cuda.stream(st):\n"
        "    for _ in range(3): step()\n"
        "    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)\n"
        "    e0.record(st)\n"
        "    for _ in range(steps): step()\n"
        "    e1.record(st)\n"
        "    st.synchronize()\n"
        "    ms = e0.elapsed_time(e1) / steps\n"
        "    loss = ref.loss(); ok, n = ref.check()\n"
        "out = {'ms_per_step': ms, 'tokens_per_s': B * S / ms * 1e3, 'steps': steps, 'loss': loss, 'optimizer_ok': ok}\n"
        "ref.close()\n"
        "def attn(Hq, Hkv, D, iters):\n"
        "    h = lambda *s: torch.randn(*s, device='cuda').half()\n"
        "    q, k, v, do = h(B, S, Hq, D), h(B, S, Hkv, D), h(B, S, Hkv, D), h(B, S, Hq, D)\n"
        "    o_, lse = torch.empty_like(q), torch.empty(B, S, Hq, device='cuda')\n"
        "    R.attention_forward(o_, lse, q, k, v)\n"
        "    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)\n"
        "    R.attention_backward(dq, dk, dv, do, o_, lse, q, k, v); torch.cuda.synchronize()\n"
        "    a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)\n"
        "    a.record()\n"
        "    for _ in range(iters): R.attention_backward(dq, dk, dv, do, o_, lse, q, k, v)\n"
        "    b_.record(); torch.cuda.synchronize()\n"
        "    us = a.elapsed_time(b_) / iters * 1e3\n"
        "    return {'shape': f'B{B} S{S} {Hq}/{Hkv} D{D}', 'us': us, 'tflops': 2.5 * 4.0 * S * S * D * Hq * B / 2 / us / 1e6}\n"
        "out['attention_backward'] = [attn(8, 2, 128, 5), attn(12, 4, 64, 2)]\n"
        "print('REFERENCE_GPU ' + json.dumps(out))\n"
    ) % (str(ROOT), BATCH, SEQ, max(3, min(args.steps, 10)))
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=900)
    for ln in proc.stdout.splitlines():
        if ln.startswith("REFERENCE_GPU "):
            out = json.loads(ln[len("REFERENCE_GPU "):])
            out["what"] = ("the reference's trainer step (CUDA graph of forward + cross-entropy on materialised fp16 logits + backward, then its "
                           "181-launch AdamW) with its own kernels rebuilt for sm_100a and cuBLASLt, same model, batch and GPU; informational")
            return out
    return {"error": (proc.stderr or proc.stdout)[-400:], "rc": proc.returncode}


# ------------------------------------------------------------------------------------------------ our arm
def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text())
        except json.JSONDecodeError:
            pass
    return {}


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    pg = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        pg = dist.group.WORLD
    from cgpt_b200 import _lib, model as M
    from cgpt_b200.train import TrainStep

    opts = M.preset(PRESET)
    # N > 1: the bucketed all-reduce overlaps the backward inside the captured graph; CGPT_B200_OVERLAP_ALLREDUCE=0 issues all
    # buckets after the backward instead (still inside the graph)
    overlap = os.environ.get("CGPT_B200_OVERLAP_ALLREDUCE", "1") == "1"
    ts = TrainStep(opts, BATCH, SEQ, seed=0, process_group=pg, overlap_allreduce=overlap)
    rows = BATCH * SEQ
    gen = torch.Generator().manual_seed(1234 + rank)
    pool = 4
    host_tokens = [torch.randint(0, opts.vocabulary_size, (BATCH, SEQ + 1), generator=gen, dtype=torch.int32) for _ in range(pool)]
    host_ids = [t[:, :-1].contiguous().pin_memory() for t in host_tokens]
    host_tgt = [t[:, 1:].contiguous().pin_memory() for t in host_tokens]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # launches of one model step (forward + loss + backward), counted on the eager warm-up inside step()
    ts.upload_batch(host_ids[0], host_tgt[0])
    c0 = _lib.launch_count()
    ts.step()
    ts.stream.synchronize()
    launches_first = _lib.launch_count() - c0       # eager pass + capture pass + 3 optimizer launches
    model_launches = (launches_first - 3) // 2
    for _ in range(max(0, args.warmup - 1)):
        ts.step()
    barrier()

    # ---- device-resident timing: K steps, CUDA events on the step's stream, max over ranks
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # The clock sampler runs from here to the end of the end-to-end loop: both loops are the same load, and with many
    # GPUs on the box one nvidia-smi query can take longer than the device-resident loop alone.
    clocks = ClockSampler(local)
    clocks.__enter__()
    barrier()
    with torch.cuda.stream(ts.stream):
        e0.record()
    for _ in range(args.steps):
        ts.step()
    with torch.cuda.stream(ts.stream):
        e1.record()
    barrier()
    ms_total = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms_total, op=dist.ReduceOp.MAX)
    ms_step = float(ms_total.item()) / args.steps
    value = world * rows / (ms_step / 1000.0)
    final_loss = ts.read_loss()
    ok = ts.check()

    # ---- end to end: pinned host -> device ids/targets every step, loss read back every step
    barrier()
    t0 = time.perf_counter()
    # The loss of every step is copied to pinned host memory and read by the host, one step late: the host waits for
    # step i's loss after it has enqueued step i + 1, as a training loop that logs the loss does, so the GPU never idles.
    pending, e2e_losses = None, []
    for i in range(args.steps):
        ts.upload_batch(host_ids[i % pool], host_tgt[i % pool])
        ts.step()
        handle = ts.read_loss_async()
        if pending is not None:
            e2e_losses.append(pending.value())
        pending = handle
    e2e_losses.append(pending.value())
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], device="cuda")
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_value = world * rows * args.steps / float(e2e_s.item())
    # still no sample (a short run on a box whose nvidia-smi is slow): keep the same load running until one arrives
    # (rank 0 decides and every rank follows: a step holds collectives)
    deadline = time.perf_counter() + 5.0
    while True:
        more = torch.tensor([1 if (not clocks.samples and time.perf_counter() < deadline) else 0], device="cuda", dtype=torch.int32)
        if world > 1:
            dist.broadcast(more, 0)
        if int(more.item()) == 0:
            break
        ts.step()
        ts.stream.synchronize()
    clocks.__exit__(None, None, None)

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / world) / PUBLISHED_TOKENS_PER_S, "dtype": "f16", "data": "synthetic",
            "config": workload_config(world),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 2 * rows * 4, "d2h_bytes_per_step": 4,
                    "loss_reads": len(e2e_losses), "loss_read": "every step, asynchronous pinned copy, consumed one step late"},
            "gpu_launches": args.steps * (model_launches + 3), "clocks": clocks.summary(),
            "final_loss": final_loss, "optimizer_ok": bool(ok), "device_status": _lib.device_status(clear=False)}

    if rank == 0:
        # ---- roofline of the dominant kernel (tcgen05 GEMM): eager re-run with CUDA events around every GEMM launch
        try:
            from cgpt_b200 import profiling
            gemm = profiling.time_gemms(ts)
            peaks = measured_peaks()
            peak = peaks.get("bf16_tflops_sustained")
            which = "measured (MEASURED_PEAKS.json bf16_tflops_sustained; B200 fp16 and bf16 dense rates are equal)"
            if peak is None:
                peak, which = 1400.0, "fallback (1.4 PFLOP/s sustained)"
            line["roofline"] = {"bound": "tensor", "achieved": gemm["tflops"], "peak": peak, "unit": "TFLOP/s",
                                "frac": gemm["tflops"] / peak, "traffic": GEMM_TRAFFIC_BYTES,
                                "traffic_note": GEMM_TRAFFIC_NOTE,
                                "kernel": "gemm_tcgen05_pair_kernel (forward, dX) + gemm_pair_softmax_kernel (LM-head logits with the softmax "
                                          "statistics epilogue) + gemm_tcgen05_persistent_kernel (dW)",
                                "launches_per_step": gemm["launches"], "ms_per_step_in_kernel": gemm["ms"],
                                "share_of_step": gemm["ms"] / ms_step, "peak_source": which,
                                "model_flops_per_step": gemm["model_flops"], "model_tflops": gemm["model_flops"] / ms_step / 1e9}
        except Exception as exc:  # the bench line must still be printed
            line["roofline"] = {"bound": "tensor", "achieved": None, "peak": None, "unit": "TFLOP/s", "frac": None,
                                "traffic": None, "error": repr(exc)}
        try:   # the metric's second half: standalone attention backward, configuration 2 and the 104m layer shape
            ab = [profiling.time_attention_backward(32, 1024, 12, 4, 64), profiling.time_attention_backward(32, 1024, 8, 2, 128)]
            burst = measured_peaks().get("bf16_tflops")
            line["attention_backward"] = [dict(a, frac_of_measured_burst_peak=(a["tflops"] / burst if burst else None)) for a in ab]
        except Exception as exc:
            line["attention_backward"] = {"error": repr(exc)}
        try:   # the loss layer on its own at 32768 tokens x d 768 x vocab 32000 (three products credited)
            line["cce"] = profiling.time_cut_cross_entropy(32768, 768, 32000)
            burst = measured_peaks().get("bf16_tflops")
            line["cce"]["frac_of_measured_burst_peak"] = line["cce"]["tflops"] / burst if burst else None
            # the three forms of a chunk side by side: row kernel over stored logits, tile statistics from the logits
            # product's epilogue, logits never stored (recomputed; four products for the three credited)
            line["cce"]["forms"] = profiling.time_cut_cross_entropy_forms(32768, 768, 32000)
        except Exception as exc:
            line["cce"] = {"error": repr(exc)}
        if world == 1:
            try:   # informational: the reference's own CUDA step (its kernels rebuilt for sm_100a + cuBLASLt) on this GPU
                line["reference_gpu"] = reference_gpu_step(args)
            except Exception as exc:
                line["reference_gpu"] = {"error": repr(exc)}
        try:
            line["cpu_baseline"] = {k: v for k, v in cpu_baseline(os.cpu_count()).items() if k != "seconds_per_pass"} if world == 1 else None
        except Exception as exc:
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "reference", "sample": repr(exc)}
        print(json.dumps(line), flush=True)
    ts.close()      # the captured graph holds the collectives: release it before the process group goes
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        # The line is printed and every rank is past its last collective. Should the process group's shutdown stall (its
        # watchdog waiting on work it can no longer observe), leave after 30 s instead of holding the launcher for minutes.
        guard = threading.Timer(30.0, lambda: os._exit(0))
        guard.daemon = True
        guard.start()
        dist.destroy_process_group()
        guard.cancel()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
