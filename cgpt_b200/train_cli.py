"""Data-parallel training driver: `python -m cgpt_b200.train_cli` (1 GPU) or under torchrun (one rank per GPU).

Mirrors the reference trainer's loop and flags (train/train.cpp:40-64 defaults, :88-112 flags, :388-426 sample split and
schedule, :532-599 step loop) for the part that is on the training hot path: pre-tokenised input, train/validation
split by shuffled samples (seed 42), cosine schedule with 2 % automatic warm-up, static loss scale, validation every N
steps, `loss.csv`, weights written in the reference's safetensors layout. Tokeniser training, text generation and the
progress bar are not rebuilt: `--input` takes token ids (`.npy`, or raw little-endian uint32 `.bin`), or `--synthetic N`
draws N uniform ids. Beyond the reference: ranks (global batch = ranks x `--batch-size`; rank r takes rows
[r*B, (r+1)*B) of it), and `optimizer.safetensors`, so `--load-dir` resumes master weights, moments and step count.
"""
from __future__ import annotations

import argparse
import math
import os
import time
from dataclasses import dataclass

import numpy as np


@dataclass
class Split:
    train: np.ndarray        # [n_train, sequence_length + 1] int32
    validation: np.ndarray   # [n_val, sequence_length + 1]


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="cgpt_b200.train_cli", description=__doc__.split("\n")[0])
    p.add_argument("--input", default=None, help="token ids: .npy (any integer dtype) or raw uint32 .bin")
    p.add_argument("--synthetic", type=int, default=0, help="draw this many uniform token ids instead of --input")
    p.add_argument("--output-dir", default="train/huggingface")
    p.add_argument("--load-dir", default=None)
    p.add_argument("--vocab-size", type=int, default=32000)
    p.add_argument("--batch-size", type=int, default=None, help="sequences per rank (default 8; 1 for --model 104m)")
    p.add_argument("--sequence-length", type=int, default=1024)
    p.add_argument("--epochs", type=int, default=10)
    p.add_argument("--max-steps", type=int, default=0, help="0 = all batches of every epoch")
    p.add_argument("--validation-interval", type=int, default=500)
    p.add_argument("--validation-batches", type=int, default=64)
    p.add_argument("--learning-rate", type=float, default=3.0e-4)
    p.add_argument("--min-learning-rate", type=float, default=3.0e-5)
    p.add_argument("--warmup-steps", type=int, default=0, help="0 = 2%% of the run")
    p.add_argument("--loss-scale", type=float, default=1024.0)
    p.add_argument("--model", default="small", help="preset: 104m, small, tiny, 1.3b")
    p.add_argument("--validation-fraction", type=float, default=0.1)
    p.add_argument("--save-avg-loss", action="store_true")
    p.add_argument("--checkpoint-interval", type=int, default=0, help="also write a checkpoint to <output-dir>/step-N every N steps (0 = only at the end)")
    p.add_argument("--overlap-allreduce", action=argparse.BooleanOptionalAction, default=True,
                   help="ranks > 1: start each gradient bucket's all-reduce during the backward, inside the captured graph "
                        "(--no-overlap-allreduce: all buckets after the backward)")
    p.add_argument("--seed", type=int, default=0)
    return p


def resolve_arguments(args: argparse.Namespace) -> argparse.Namespace:
    """Defaults that depend on other flags and the reference's validation (train/train.cpp:94-97,126-137,339)."""
    if args.batch_size is None:
        args.batch_size = 1 if args.model == "104m" else 8
    if args.batch_size <= 0 or args.sequence_length <= 0 or args.epochs <= 0:
        raise ValueError("batch size, sequence length and epochs must be positive")
    if not (math.isfinite(args.validation_fraction) and 0.0 < args.validation_fraction < 1.0):
        raise ValueError("--validation-fraction must be in (0, 1)")
    if not (args.learning_rate > 0 and 0 <= args.min_learning_rate <= args.learning_rate):
        raise ValueError("learning rates must satisfy 0 <= min <= initial, initial > 0")
    if not args.loss_scale > 0:
        raise ValueError("--loss-scale must be positive")
    if args.validation_interval <= 0 or args.validation_batches <= 0:
        raise ValueError("validation interval and batches must be positive")
    if (args.input is None) == (args.synthetic <= 0):
        raise ValueError("give exactly one of --input and --synthetic N")
    return args


def load_tokens(args: argparse.Namespace) -> np.ndarray:
    if args.synthetic > 0:
        return np.random.default_rng(args.seed).integers(0, args.vocab_size, size=args.synthetic, dtype=np.int64).astype(np.int32)
    if not os.path.exists(args.input):
        raise FileNotFoundError(f"Missing input: {args.input}")
    tokens = np.load(args.input) if args.input.endswith(".npy") else np.fromfile(args.input, dtype="<u4")
    tokens = np.asarray(tokens).reshape(-1)
    if tokens.size and (int(tokens.max()) >= args.vocab_size or int(tokens.min()) < 0):
        raise ValueError("token id outside the vocabulary")
    return tokens.astype(np.int32)


def split_samples(tokens: np.ndarray, batch: int, seq: int, validation_fraction: float) -> Split:
    """Samples of seq + 1 tokens starting every seq tokens, shuffled with seed 42; the last
    clamp(fraction * n, batch, n - batch) of the shuffled order are the validation set (train/train.cpp:388-411)."""
    if batch * seq + 1 > tokens.size // 2:
        raise RuntimeError("Not enough tokens for one training and validation batch")
    n = (tokens.size - 1) // seq
    n_val = min(max(int(n * validation_fraction), batch), n - batch)
    order = np.random.default_rng(42).permutation(n)
    starts = order * seq
    windows = np.lib.stride_tricks.sliding_window_view(tokens, seq + 1)
    train = np.ascontiguousarray(windows[starts[: n - n_val]])
    val = np.ascontiguousarray(windows[starts[n - n_val:]])
    return Split(train, val)


def schedule_lengths(args: argparse.Namespace, batches_per_epoch: int) -> tuple[int, int]:
    """(total steps, warm-up steps) as train/train.cpp:422-425."""
    total = batches_per_epoch * args.epochs
    if args.max_steps:
        total = min(args.max_steps, total)
    warmup = args.warmup_steps if args.warmup_steps else (max(1, total // 50) if total > 1 else 0)
    return total, warmup


def rank_slice(global_batch: np.ndarray, rank: int, per_rank: int) -> np.ndarray:
    """Rows [rank * per_rank, (rank + 1) * per_rank) of a [world * per_rank, seq + 1] batch."""
    return global_batch[rank * per_rank:(rank + 1) * per_rank]


def main(argv=None) -> int:
    args = resolve_arguments(build_parser().parse_args(argv))
    import torch
    import torch.distributed as dist

    from . import checkpoint, model as M, optim as O
    from .train import TrainStep

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    pg = None
    if world > 1:
        dist.init_process_group("nccl")
        pg = dist.group.WORLD
    log = print if rank == 0 else (lambda *a, **k: None)

    tokens = load_tokens(args)
    B, S = args.batch_size, args.sequence_length
    split = split_samples(tokens, B * world, S, args.validation_fraction)
    batches_per_epoch = split.train.shape[0] // (B * world)
    val_batches = min(args.validation_batches, split.validation.shape[0] // (B * world))
    if batches_per_epoch == 0 or val_batches == 0:
        raise RuntimeError("Not enough tokens for one training and validation batch")
    total_steps, warmup = schedule_lengths(args, batches_per_epoch)
    scheduler = O.LearningRateScheduler(O.LearningRateSchedulerOptions(args.learning_rate, args.min_learning_rate, warmup, total_steps))

    options = M.preset(args.model, vocabulary_size=args.vocab_size)
    adamw = O.AdamWOptions(args.learning_rate, 0.9, 0.95, 1e-8, 0.1, args.loss_scale, 1.0)   # train/train.cpp:434-441
    ts = TrainStep(options, B, S, dtype=torch.float16, seed=args.seed, loss_scale=args.loss_scale, adamw=adamw, process_group=pg,
                   overlap_allreduce=args.overlap_allreduce)
    log(f"model {args.model}: {ts.storage.num_parameters() / 1e6:.1f}M parameters, ranks {world}, "
        f"global batch {B * world} x {S}, {total_steps} steps ({warmup} warm-up)")
    first_step = 0
    if args.load_dir:
        checkpoint.load_model(args.load_dir, ts.storage)
        if checkpoint.has_optimizer(args.load_dir):
            first_step = int(checkpoint.load_optimizer(args.load_dir, ts.storage, ts.states).get("step", 0))
        else:   # the reference's resume: fresh optimizer state from the loaded weights
            for (p, _), st in zip(ts.storage.parameters_and_gradients(), ts.states):
                st.master_parameter.copy_(p.float())
        ts.adopt_default_stream_work()      # the loads above ran on torch's current stream
        log(f"loaded {args.load_dir}, resuming at step {first_step}")

    # The step is asynchronous: the host runs several steps ahead of the GPU, so a pinned staging buffer may only be
    # rewritten once the copy that reads it has executed. A small ring of buffers, each guarded by an event.
    ring = [(torch.empty(B, S, dtype=torch.int32).pin_memory(), torch.empty(B, S, dtype=torch.int32).pin_memory(),
             torch.cuda.Event()) for _ in range(4)]
    staged = 0

    def stage(sample_rows: np.ndarray) -> None:
        nonlocal staged
        host_ids, host_targets, copied = ring[staged % len(ring)]
        if staged >= len(ring):
            copied.synchronize()
        staged += 1
        rows = torch.from_numpy(rank_slice(sample_rows, rank, B))
        host_ids.copy_(rows[:, :-1])
        host_targets.copy_(rows[:, 1:])
        ts.upload_batch(host_ids, host_targets)
        copied.record(ts.stream)

    def validate() -> float:
        total = 0.0
        for i in range(val_batches):
            stage(split.validation[i * B * world:(i + 1) * B * world])
            total += ts.validation_loss()
        mean = torch.tensor([total / val_batches], device="cuda")
        if world > 1:
            dist.all_reduce(mean)
            mean /= world
        return float(mean.item())

    def save(step: int, directory: str | None = None) -> None:
        # The step just enqueued (graph replay, all-reduce, AdamW) runs on ts.stream while the copies below run on torch's
        # current stream: drain the step first, on every rank, and let check() refresh the optimizer's host-side step
        # counters, which the checkpoint stores (they are otherwise only refreshed at the logging points).
        ts.stream.synchronize()
        ts.check()
        if rank == 0:
            directory = directory or args.output_dir
            checkpoint.save_model(directory, ts.storage)
            checkpoint.save_optimizer(directory, ts.storage, ts.states, {"step": step})

    loss_log = None
    if args.save_avg_loss and rank == 0:
        os.makedirs(args.output_dir, exist_ok=True)
        loss_log = open(os.path.join(args.output_dir, "loss.csv"), "w")
        loss_log.write("step,loss\n")

    step, t0, tokens_seen, window_loss, window_n = first_step, time.time(), 0, 0.0, 0
    epoch_rng = np.random.default_rng(42)
    # A resumed run continues where the saved one stopped: the permutations of the completed epochs are drawn and
    # dropped, and the batches of the current epoch that were already consumed are skipped.
    for _ in range(first_step // batches_per_epoch):
        epoch_rng.permutation(split.train.shape[0])
    skip = first_step % batches_per_epoch
    while step < total_steps:
        order = epoch_rng.permutation(split.train.shape[0])
        for b in range(skip, batches_per_epoch):
            if step >= total_steps:
                break
            stage(split.train[order[b * B * world:(b + 1) * B * world]])
            ts.step(scheduler.learning_rate(step))
            step += 1
            tokens_seen += B * S * world
            if step % 10 == 0 or step == total_steps:
                loss = ts.read_loss()
                ok = ts.check()
                window_loss, window_n = window_loss + loss, window_n + 1
                dt = time.time() - t0
                log(f"step {step}/{total_steps} loss {loss:.4f} lr {scheduler.learning_rate(step - 1):.3e} "
                    f"{tokens_seen / dt:,.0f} tokens/s{'' if ok else ' (non-finite gradients: step skipped)'}")
                if loss_log is not None:
                    loss_log.write(f"{step},{window_loss / window_n}\n")
                    loss_log.flush()
                    window_loss, window_n = 0.0, 0
            if step % args.validation_interval == 0 or step == total_steps:
                log(f"step {step}: validation loss {validate():.4f}")
            if args.checkpoint_interval and step % args.checkpoint_interval == 0 and step < total_steps:
                save(step, os.path.join(args.output_dir, f"step-{step}"))   # train/train.cpp:493-526 exports to <output>/step-N
    save(step)
    if loss_log is not None:
        loss_log.close()
    ts.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
