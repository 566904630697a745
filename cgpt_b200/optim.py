"""Host-side mirror of CGPT's AdamW API (reference ``include/optim/adamw.h``, ``src/optim/adamw.cu``)
and of its learning-rate schedule (``include/optim/lr_scheduler.h``).

``AdamWState``, ``AdamWBatchEntry``, ``AdamWWorkspace``, ``adamw_step_many_async``, ``adamw_check`` and
``adamw_step`` keep the reference's names and semantics; the arithmetic runs in ``libcgpt_b200.so``.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field

import torch

from . import _lib
from ._lib import AdamWOptions as _COptions
from ._lib import AdamWTensor as _CTensor
from ._lib import check, dtype_code, lib, stream_ptr


@dataclass
class AdamWOptions:
    """include/optim/adamw.h:12-27 (same defaults)."""
    learning_rate: float = 1.0e-3
    beta1: float = 0.9
    beta2: float = 0.999
    epsilon: float = 1.0e-8
    weight_decay: float = 1.0e-2
    loss_scale: float = 1.0
    max_grad_norm: float = math.inf

    def validate(self) -> None:
        """Same conditions as validate_options in src/optim/adamw.cu:28-45."""
        ok = (self.learning_rate >= 0 and 0 <= self.beta1 < 1 and 0 <= self.beta2 < 1 and self.epsilon > 0
              and self.weight_decay >= 0 and self.loss_scale > 0 and self.max_grad_norm > 0)
        if not ok or any(math.isnan(v) for v in (self.learning_rate, self.beta1, self.beta2, self.epsilon,
                                                  self.weight_decay, self.loss_scale, self.max_grad_norm)):
            raise _lib.CgptInvalidArgument("adamw: invalid options")

    def _c(self) -> _COptions:
        return _COptions(self.learning_rate, self.beta1, self.beta2, self.epsilon, self.weight_decay,
                         self.loss_scale, self.max_grad_norm)


@dataclass
class AdamWState:
    """fp32 master copy and moments of one parameter (include/optim/adamw.h:33-47)."""
    master_parameter: torch.Tensor
    first_moment: torch.Tensor
    second_moment: torch.Tensor
    step: int = 0

    @staticmethod
    def for_parameter(parameter: torch.Tensor, stream=None) -> "AdamWState":
        """master = float(parameter), moments = 0 (src/optim/adamw.cu:362-395)."""
        if not parameter.is_cuda:
            raise _lib.CgptInvalidArgument("AdamWState.for_parameter: CUDA tensor required")
        with torch.cuda.stream(stream) if stream is not None else _null():
            return AdamWState(parameter.detach().to(torch.float32).clone(),
                              torch.zeros_like(parameter, dtype=torch.float32),
                              torch.zeros_like(parameter, dtype=torch.float32), 0)


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


@dataclass
class AdamWBatchEntry:
    """include/optim/adamw.h:52-56."""
    parameter: torch.Tensor
    gradient: torch.Tensor
    state: AdamWState


@dataclass
class AdamWWorkspace:
    """Device-side step counter, flags and work table; binds to one entry list on first use
    (src/optim/adamw.cu:283-305)."""
    _handle: C.c_void_p | None = None
    _states: list = field(default_factory=list)
    _keys: tuple = ()

    def __del__(self):
        # at interpreter shutdown the module globals may already be gone; the process is about to release everything
        handle, self._handle = getattr(self, "_handle", None), None
        if handle is not None and lib is not None:
            try:
                lib.cgpt_adamw_destroy(handle)
            except Exception:
                pass


def _validate_entry(e: AdamWBatchEntry) -> None:
    p, g, s = e.parameter, e.gradient, e.state
    if p is None or g is None or s is None:
        raise _lib.CgptInvalidArgument("adamw_step_many_async: null entry")
    if not (p.is_cuda and g.is_cuda):
        raise _lib.CgptInvalidArgument("adamw_step_many_async: CUDA tensors required")
    if p.dtype != g.dtype or p.shape != g.shape:
        raise _lib.CgptInvalidArgument("adamw_step: parameter and gradient must match")
    for t in (s.master_parameter, s.first_moment, s.second_moment):
        if t.dtype != torch.float32 or t.shape != p.shape:
            raise _lib.CgptInvalidArgument("adamw_step: master parameter and moment buffers must be F32")
    for t in (p, g, s.master_parameter, s.first_moment, s.second_moment):
        if not t.is_contiguous():
            raise _lib.CgptInvalidArgument("adamw_step: tensors must be contiguous")


def adamw_bind(entries, workspace: AdamWWorkspace, stream=None) -> list:
    """Binds the workspace to the entry list (device tables, step counter seeded from the states) without taking a step;
    adamw_step_many_async does it on first use (src/optim/adamw.cu:283-305). Allocates: call it outside stream capture.
    Returns the validated entry list; raises if the workspace is already bound to a different list."""
    entries = list(entries)
    if not entries:
        raise _lib.CgptInvalidArgument("adamw_step_many_async: empty parameter list")
    keys = tuple((e.parameter.data_ptr(), e.gradient.data_ptr(), e.state.master_parameter.data_ptr())
                 for e in entries)
    if workspace._handle is None:
        initial = entries[0].state.step
        for e in entries:
            _validate_entry(e)
            if e.state.step != initial:
                raise _lib.CgptInvalidArgument("adamw_step_many_async: states must share one initial step")
        arr = (_CTensor * len(entries))()
        for i, e in enumerate(entries):
            arr[i] = _CTensor(e.parameter.data_ptr(), e.gradient.data_ptr(), e.state.master_parameter.data_ptr(),
                              e.state.first_moment.data_ptr(), e.state.second_moment.data_ptr(),
                              e.parameter.numel(), dtype_code(e.parameter), 0)
        handle = C.c_void_p()
        check(lib.cgpt_adamw_create(C.byref(handle), arr, len(entries), initial, stream_ptr(stream)),
              "adamw_step_many_async")
        workspace._handle = handle
        workspace._states = [e.state for e in entries]
        workspace._keys = keys
    elif len(workspace._states) != len(entries):
        raise _lib.CgptInvalidArgument("adamw_step_many_async: workspace entries changed")
    elif any(a is not b.state for a, b in zip(workspace._states, entries)) or keys != workspace._keys:
        raise _lib.CgptInvalidArgument("adamw_step_many_async: workspace states changed")
    return entries


def adamw_step_many_async(entries, options: AdamWOptions, workspace: AdamWWorkspace, stream=None,
                          learning_rate_device: torch.Tensor | None = None) -> None:
    """One fused optimizer step over all entries (include/optim/adamw.h:101-105). With `learning_rate_device` (an fp32
    CUDA tensor of one element) the update reads the learning rate from it when it runs instead of taking
    options.learning_rate at launch: the form that can be captured into a CUDA graph and replayed under a schedule."""
    options.validate()
    adamw_bind(entries, workspace, stream)
    copts = options._c()
    if learning_rate_device is not None:
        if not (learning_rate_device.is_cuda and learning_rate_device.dtype == torch.float32 and learning_rate_device.numel() == 1):
            raise _lib.CgptInvalidArgument("adamw_step_many_async: learning_rate_device must be one fp32 CUDA element")
        check(lib.cgpt_adamw_step_device_lr(workspace._handle, C.byref(copts), learning_rate_device.data_ptr(), stream_ptr(stream)),
              "adamw_step_many_async")
        return
    check(lib.cgpt_adamw_step(workspace._handle, C.byref(copts), stream_ptr(stream)), "adamw_step_many_async")


def adamw_check(workspace: AdamWWorkspace, stream=None) -> bool:
    """Synchronises, refreshes ``state.step`` on the host and returns False if any step since the last
    check was skipped for non-finite gradients (src/optim/adamw.cu:348-359)."""
    if workspace._handle is None:
        return True
    step, bad = C.c_uint64(0), C.c_int(0)
    check(lib.cgpt_adamw_check(workspace._handle, C.byref(step), C.byref(bad), stream_ptr(stream)), "adamw_check")
    for s in workspace._states:
        s.step = int(step.value)
    return bad.value == 0


def adamw_last_stats(workspace: AdamWWorkspace, stream=None) -> tuple[float, float]:
    """(sum of squared unscaled gradients, clip factor) of the most recent step."""
    sq, clip = C.c_float(0), C.c_float(0)
    check(lib.cgpt_adamw_last_stats(workspace._handle, C.byref(sq), C.byref(clip), stream_ptr(stream)),
          "adamw_last_stats")
    return float(sq.value), float(clip.value)


def adamw_step(parameter, gradient, state: AdamWState, options: AdamWOptions | None = None, stream=None) -> bool:
    """Single-tensor synchronous step (include/optim/adamw.h:124-136): clip is per tensor, returns
    False when the step was skipped for non-finite gradients. CUDA tensors only."""
    options = options or AdamWOptions()
    ws = AdamWWorkspace()
    adamw_step_many_async([AdamWBatchEntry(parameter, gradient, state)], options, ws, stream)
    return adamw_check(ws, stream)


@dataclass
class LearningRateSchedulerOptions:
    """include/optim/lr_scheduler.h:9-14."""
    initial_learning_rate: float = 1.0e-4
    minimum_learning_rate: float = 0.0
    warmup_steps: int = 0
    total_steps: int = 1


class LearningRateScheduler:
    """Linear warm-up, then cosine decay to the minimum; the last step returns the minimum exactly
    (include/optim/lr_scheduler.h:16-55)."""

    def __init__(self, options: LearningRateSchedulerOptions):
        o = options
        if (not math.isfinite(o.initial_learning_rate) or not math.isfinite(o.minimum_learning_rate)
                or o.initial_learning_rate <= 0 or o.minimum_learning_rate < 0
                or o.minimum_learning_rate > o.initial_learning_rate or o.total_steps == 0
                or o.warmup_steps >= o.total_steps):
            raise _lib.CgptInvalidArgument("Invalid learning-rate scheduler options")
        self.options = o

    def learning_rate(self, step: int) -> float:
        o = self.options
        if step < o.warmup_steps:
            return o.initial_learning_rate * (float(step + 1) / float(o.warmup_steps))
        if step >= o.total_steps - 1:
            return o.minimum_learning_rate
        decay_steps = o.total_steps - o.warmup_steps
        progress = float(step - o.warmup_steps) / float(max(1, decay_steps - 1))
        cosine = 0.5 * (1.0 + math.cos(math.pi * progress))
        return o.minimum_learning_rate + (o.initial_learning_rate - o.minimum_learning_rate) * cosine
