"""One training step (forward + cut-cross-entropy loss + backward + AdamW), optionally data-parallel.

Follows the reference trainer's step (train/train.cpp:427-457, 532-556): fp16 weights and activations,
fp32 master weights, static loss scale, the step captured once into a CUDA graph and replayed.
Differences: the loss layer is the cut-cross-entropy op (no [tokens, vocab] logits); the captured graph
holds the WHOLE step, optimizer included (the learning rate is a device scalar written before each
replay; the reference launches its optimizer outside its graph because the rate is a kernel argument,
train/train.cpp:554-556); and with more than one rank the graph also holds the bucketed NCCL all-reduces,
each started on the communication stream as soon as the backward has finished the gradients of its
bucket, so they overlap the rest of the backward, and joined before the optimizer.
"""
from __future__ import annotations

import torch

from . import dp
from . import model as M
from . import optim as O


class PendingLoss:
    """A loss value on its way to the host (TrainStep.read_loss_async). At most 4 may be outstanding."""

    def __init__(self, host: torch.Tensor, done: torch.cuda.Event):
        self._host, self._done = host, done

    def value(self) -> float:
        self._done.synchronize()
        return float(self._host[0])


class TrainStep:
    def __init__(self, options: M.TransformerModelOptions, batch: int, seq: int, *, dtype=torch.float16, seed: int = 0,
                 loss_scale: float = 1024.0, adamw: O.AdamWOptions | None = None, process_group=None,
                 bucket_bytes: int = 48 << 20, use_graph: bool = True, cce_chunk_rows: int = 0, device="cuda",
                 overlap_allreduce: bool = True):
        self.options, self.batch, self.seq, self.dtype = options, batch, seq, dtype
        self.rows = batch * seq
        self.pg = process_group
        self.world = process_group.size() if process_group is not None else 1
        self.loss_scale = loss_scale
        self.adamw_options = adamw or O.AdamWOptions(3e-4, 0.9, 0.95, 1e-8, 0.1, loss_scale, 1.0)
        self.adamw_options.loss_scale = loss_scale
        self.cce_chunk_rows = cce_chunk_rows
        b = options.block_options
        self.storage = M.ModelStorage(options, dtype, seed, device=device)
        self.workspace = M.TransformerModelWorkspace(options, batch, seq, dtype, device)
        self.backward_workspace = M.TransformerModelBackwardWorkspace(options, batch, seq, dtype, device, max_seq=seq)
        self.cos, self.sin = M.rotary_cache(seq, b.rotary_dim or b.head_dim, dtype, device)
        self.token_ids = torch.zeros(self.rows, dtype=torch.int32, device=device)
        self.targets = torch.zeros(self.rows, dtype=torch.int32, device=device)
        self.loss = torch.zeros(1, dtype=torch.float32, device=device)
        pairs = self.storage.parameters_and_gradients()
        self.states = [O.AdamWState.for_parameter(p) for p, _ in pairs]
        self.entries = [O.AdamWBatchEntry(p, g, s) for (p, g), s in zip(pairs, self.states)]
        self.adamw_workspace = O.AdamWWorkspace()
        self.stream = torch.cuda.Stream(device=device)
        self.graph = None
        # With more than one rank the backward is issued piece by piece and every bucket's all-reduce starts as soon as
        # its gradients are final (overlap_allreduce=False issues all of them after the backward instead). Either way the
        # collectives are part of the captured graph.
        self.overlap_allreduce = bool(overlap_allreduce) and self.world > 1
        self.use_graph = use_graph
        self._buckets = self._make_buckets(bucket_bytes)
        self._reducer = dp.BucketReducer(self._buckets, self.pg) if self.overlap_allreduce else None
        self._keep = None
        self._loss_ring = None
        # the step's learning rate as a device scalar, fed from a small ring of pinned host values
        self.learning_rate_device = torch.full((1,), float(self.adamw_options.learning_rate), dtype=torch.float32, device=device)
        self._lr_ring = [(torch.empty(1, dtype=torch.float32).pin_memory(), torch.cuda.Event()) for _ in range(8)]
        self._lr_writes = 0
        self.adopt_default_stream_work()

    def adopt_default_stream_work(self) -> None:
        """Makes the step's stream wait for everything enqueued so far on torch's current stream. Weights, optimizer
        state and buffers are created (and checkpoints loaded, token ids written by tests) on the current stream, while
        the step runs on its own non-blocking stream: without this edge the first step could formally start before those
        kernels and copies have landed. Call it again after writing any of the step's tensors from another stream."""
        self.stream.wait_stream(torch.cuda.current_stream())

    # ------------------------------------------------------------------------------------------ pieces
    def _make_buckets(self, bucket_bytes: int):
        """Contiguous slices of the flat gradient buffer of about bucket_bytes each, in backward order."""
        return dp.make_buckets(self.storage.flat_gradients, bucket_bytes)

    def upload_batch(self, host_ids: torch.Tensor, host_targets: torch.Tensor) -> None:
        """Host (pinned) -> device copy of the step's token ids and targets on the step's stream."""
        with torch.cuda.stream(self.stream):
            self.token_ids.copy_(host_ids.view(-1), non_blocking=True)
            self.targets.copy_(host_targets.view(-1), non_blocking=True)

    def enqueue_model_step(self) -> None:
        """forward -> loss (+ LM-head gradients) -> backward on the current stream (capturable)."""
        st, ws, bw, o = self.storage, self.workspace, self.backward_workspace, self.options
        k1 = M.transformer_model_forward(None, self.token_ids, self.batch, self.seq, st, ws, self.cos, self.sin, None,
                                         None, o, scratch=bw)
        M.cut_cross_entropy_forward_backward(self.loss, bw.grad_normalized, st.g_lm_head, ws.normalized, st.lm_head,
                                             self.targets, self.rows, None, dp.gradient_scale(self.loss_scale, self.world),
                                             chunk_rows=self.cce_chunk_rows)
        if self._reducer is None:
            k2 = M.transformer_model_backward(None, self.token_ids, self.batch, self.seq, st, ws, bw, self.cos, self.sin,
                                              None, None, o)
        else:
            # backward step by step; after each, the buckets that are complete go out on the communication stream
            k2 = None
            for step in range(o.num_layers + 2):
                k2 = M.transformer_model_backward(None, self.token_ids, self.batch, self.seq, st, ws, bw, self.cos,
                                                  self.sin, None, None, o, steps=(step, step + 1))
                self._reducer.advance(st.final_gradient_elements(step + 1))
        self._keep = (k1, k2)

    def _allreduce_gradients(self) -> None:
        if self.world == 1:
            return
        if self._reducer is not None:
            self._reducer.finish()      # the collectives were started during the backward
            return
        dp.allreduce_buckets(self._buckets, group=self.pg)

    def _write_learning_rate(self, value: float) -> None:
        """Pinned host value -> device scalar on the step's stream (4 bytes; the slot is reused only after its copy ran)."""
        host, copied = self._lr_ring[self._lr_writes % len(self._lr_ring)]
        if self._lr_writes >= len(self._lr_ring):
            copied.synchronize()
        self._lr_writes += 1
        host[0] = value
        self.learning_rate_device.copy_(host, non_blocking=True)
        copied.record(self.stream)

    def enqueue_full_step(self) -> None:
        """The whole step on the current stream (capturable): model step, gradient all-reduce, AdamW with the learning
        rate read from the device scalar."""
        self.enqueue_model_step()
        self._allreduce_gradients()
        O.adamw_step_many_async(self.entries, self.adamw_options, self.adamw_workspace, learning_rate_device=self.learning_rate_device)

    def step(self, learning_rate: float | None = None) -> None:
        """One optimizer step on the batch currently in token_ids/targets. Asynchronous."""
        if learning_rate is not None:
            self.adamw_options.learning_rate = learning_rate
        with torch.cuda.stream(self.stream):
            self._write_learning_rate(float(self.adamw_options.learning_rate))
            if self.use_graph:
                if self.graph is None:
                    # Eager warm-up: sizes the library's scratch arena, binds the optimizer workspace and opens NCCL's
                    # channels. It must not change the training state, so it runs the model step and the collectives but
                    # not the optimizer (a gradient all-reduce of a repeated batch is harmless: the step that follows
                    # recomputes every gradient).
                    self.enqueue_model_step()
                    self._allreduce_gradients()
                    O.adamw_bind(self.entries, self.adamw_workspace)
                    self.stream.synchronize()
                    self.graph = torch.cuda.CUDAGraph()
                    # thread-local capture mode: NCCL's watchdog thread may query events while this thread captures
                    with torch.cuda.graph(self.graph, stream=self.stream, capture_error_mode="thread_local"):
                        self.enqueue_full_step()
                self.graph.replay()
            else:
                self.enqueue_full_step()

    def validation_loss(self) -> float:
        """Loss of the batch currently in token_ids/targets without an optimizer step (train/train.cpp:490-530 runs
        forward + loss on held-out batches). The loss layer also rewrites the LM-head and final-norm gradient buffers;
        the next training step overwrites them again."""
        st, ws, bw, o = self.storage, self.workspace, self.backward_workspace, self.options
        with torch.cuda.stream(self.stream):
            keep = M.transformer_model_forward(None, self.token_ids, self.batch, self.seq, st, ws, self.cos, self.sin, None,
                                               None, o, scratch=bw)
            M.cut_cross_entropy_forward_backward(self.loss, bw.grad_normalized, st.g_lm_head, ws.normalized, st.lm_head,
                                                 self.targets, self.rows, None, 1.0, chunk_rows=self.cce_chunk_rows)
            self.stream.synchronize()
        del keep
        return float(self.loss.item())

    def read_loss(self) -> float:
        """Device -> host read of the last step's loss (synchronises the step's stream)."""
        self.stream.synchronize()
        return float(self.loss.item())

    def read_loss_async(self) -> "PendingLoss":
        """Enqueues the device -> host copy of the last step's loss into pinned memory on the step's stream and returns
        at once; `PendingLoss.value()` waits for that copy only. A training loop that logs the loss of step i after it
        has enqueued step i + 1 never drains the stream."""
        if self._loss_ring is None:
            self._loss_ring = [(torch.empty(1, dtype=torch.float32).pin_memory(), torch.cuda.Event()) for _ in range(4)]
            self._loss_reads = 0
        host, done = self._loss_ring[self._loss_reads % len(self._loss_ring)]
        self._loss_reads += 1
        with torch.cuda.stream(self.stream):
            host.copy_(self.loss, non_blocking=True)
            done.record(self.stream)
        return PendingLoss(host, done)

    def close(self) -> None:
        """Drains the step's stream and releases the captured graph. With more than one rank the graph holds NCCL kernels
        and the events of the collectives captured into it: call this before the process group is destroyed, or the
        group's shutdown waits on work that only exists inside the graph."""
        self.stream.synchronize()
        if self.graph is not None:
            self.graph.reset()
            self.graph = None
        self._keep = None

    def check(self) -> bool:
        """Synchronises the step's stream, refreshes the host-side step counters of the optimizer states and returns
        False if a step since the last check was skipped for non-finite gradients. Raises if a tensor-core kernel's
        bounded wait ran out (device status word): its outputs are then incomplete and training must not go on."""
        from ._lib import device_status
        with torch.cuda.stream(self.stream):
            ok = O.adamw_check(self.adamw_workspace)
        status = device_status()
        if status != 0:
            raise RuntimeError(f"cgpt_b200: a kernel gave up a bounded wait (device status {status}); results are incomplete")
        return ok
