"""Data-parallel plumbing of the training step: bucketing of the flat gradient buffer and the all-reduce.

The reference has no multi-GPU path; this is new code. One process per GPU, identical weights and optimizer
state on every rank, per-rank batches. The loss layer already multiplies gradients by loss_scale / world, so a
SUM all-reduce yields the loss-scaled average gradient on every rank, and every rank then takes the same AdamW
skip / clip decision on identical data. This module has no CUDA dependency (it is tested with gloo on CPU).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def make_buckets(flat: torch.Tensor, bucket_bytes: int) -> list[torch.Tensor]:
    """Contiguous views of `flat` of about bucket_bytes each, in storage order (= the order in which the backward
    finishes the gradients). The views alias `flat`: reducing them reduces the gradients in place."""
    if flat.dim() != 1 or not flat.is_contiguous():
        raise ValueError("make_buckets: flat gradient buffer must be 1-D and contiguous")
    per = max(1, int(bucket_bytes) // flat.element_size())
    return [flat[i:i + per] for i in range(0, flat.numel(), per)]


def gradient_scale(loss_scale: float, world_size: int) -> float:
    """Multiplier the loss layer applies to its gradients: loss scale for fp16 range, 1/world for the average."""
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    return float(loss_scale) / float(world_size)


def allreduce_buckets(buckets, group=None, async_op: bool = False):
    """SUM all-reduce of every bucket. With async_op the work handles are returned (wait on them before AdamW)."""
    if group is None and not dist.is_initialized():
        return []
    works = []
    for b in buckets:
        w = dist.all_reduce(b, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
        if async_op:
            works.append(w)
    return works
