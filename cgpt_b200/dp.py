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


class BucketReducer:
    """Starts the all-reduce of each bucket as soon as the backward has finished every gradient in it.

    ``buckets`` are consecutive views of one flat buffer whose storage order is the order in which the backward
    finishes gradients. ``advance(final_elements)`` is called after a piece of the backward with the number of
    leading elements that are now final; every bucket that lies entirely below that mark and has not been started is
    reduced asynchronously (the collective runs on the communication stream and overlaps the rest of the backward).
    ``finish()`` starts whatever is left and waits for all of them."""

    def __init__(self, buckets, group=None):
        self.buckets = list(buckets)
        self.group = group
        self.ends = []
        total = 0
        for b in self.buckets:
            total += b.numel()
            self.ends.append(total)
        self.started = 0
        self.works = []

    def advance(self, final_elements: int) -> int:
        """Returns how many buckets were started by this call."""
        n = 0
        while self.started < len(self.buckets) and self.ends[self.started] <= final_elements:
            self.works.append(dist.all_reduce(self.buckets[self.started], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            self.started += 1
            n += 1
        return n

    def finish(self) -> None:
        self.advance(self.ends[-1] if self.ends else 0)
        for w in self.works:
            w.wait()
        self.works = []
        self.started = 0
