"""Whole-step CUDA graph capture.

A training step of a small model is launch-bound: several hundred kernels of tens of microseconds
each, issued from Python through autograd.  ``GraphedTrainStep`` captures ONE complete step
(gradient zeroing, forward, backward with its bucket collectives on side streams, optimizer) into a
CUDA graph and replays it, so the GPU runs back-to-back kernels with no host in the loop.

What makes the step capturable: every kernel launches on the current stream; step-dependent
scalars live in device memory (Adam's step counter and bias corrections, the epochs of the NVLink
flag barriers, the upstream gradient of the loss); allocations come from the graph's private pool;
inputs are copied into static buffers before each replay.
"""
from __future__ import annotations

import sys
from typing import Callable, Sequence

import torch

from ..ops import functional as ops


class GraphedTrainStep:
    def __init__(self, step_fn: Callable[..., torch.Tensor], example_inputs: Sequence[torch.Tensor], warmup: int = 3):
        """``step_fn(*inputs) -> loss tensor`` must run one full training step.  It is run ``warmup``
        times eagerly on a side stream (lazy initialisation, autotuning of nothing, allocator
        warm-up), then captured."""
        self.static_inputs = [t.clone() for t in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                step_fn(*self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        n0 = ops.launch_count()
        with torch.cuda.graph(self.graph):
            self.static_loss = step_fn(*self.static_inputs)
        self.launches_per_replay = ops.launch_count() - n0
        self.steps_run_eagerly = warmup   # the captured pass itself executes nothing

    def __call__(self, *inputs: torch.Tensor) -> torch.Tensor:
        for dst, src in zip(self.static_inputs, inputs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        # a fused NVLink collective of an earlier replay that gave up on a peer has left gradients
        # unreduced: stop here (the captured step refreshes the pinned status mirrors itself)
        symm = sys.modules.get("infinitrain_b200.parallel.symm")
        if symm is not None:
            symm.NvlinkContext.check_all(sync=False)
        self.graph.replay()
        ops._counters["launches"] += self.launches_per_replay
        return self.static_loss


class LaggedScalar:
    """Per-step read-back of a device scalar (the loss) that does not drain the device.

    ``float(loss)`` right after a step makes the host wait for the step and the device wait for the
    host's next launch.  Here ``push`` enqueues an asynchronous copy of the scalar into pinned host
    memory behind the step that produced it, and ``pop`` returns the OLDEST pushed value, waiting
    only for that copy.  Called as ``push(step i); pop() -> value of step i - 1`` the host stays one
    step ahead: step i is queued on the device before step i - 1's value is looked at, every step's
    value is still read, in order, one step late.  ``drain`` returns what is left at the end.
    """

    def __init__(self, depth: int = 2):
        self._slots = [torch.zeros((), dtype=torch.float32).pin_memory() for _ in range(depth)]
        self._events = [torch.cuda.Event() for _ in range(depth)]
        self._pending = []
        self._next = 0

    def push(self, value: torch.Tensor) -> None:
        if len(self._pending) == len(self._slots):
            raise RuntimeError("LaggedScalar: pop() before pushing more values than its depth")
        k = self._next
        self._next = (k + 1) % len(self._slots)
        v = value.detach()
        self._slots[k].copy_(v if v.dtype == torch.float32 else v.float(), non_blocking=True)
        self._events[k].record()
        self._pending.append(k)

    def pop(self) -> float:
        k = self._pending.pop(0)
        self._events[k].synchronize()
        return float(self._slots[k])

    def drain(self):
        return [self.pop() for _ in range(len(self._pending))]

    def __len__(self) -> int:
        return len(self._pending)
