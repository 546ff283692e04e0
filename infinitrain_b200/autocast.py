"""Autocast guard and gradient-mode guards.

Reference: infini_train/include/autocast.h:36-171 (per-op policy table applied in
``Function::Apply``), infini_train/include/autograd/grad_mode.h:8-36.  Here the policy is applied at
op granularity inside :mod:`infinitrain_b200.ops.functional`: Linear / Matmul / attention run in the
low-precision dtype with fp32 accumulation, normalisation statistics, softmax and cross-entropy
run in fp32, parameters and weight gradients stay fp32.
"""
from __future__ import annotations

import torch

from .datatype import DataType, to_torch_dtype
from .device import DeviceType
from .ops import functional as ops

# Ops that run in the low-precision dtype / are forced to fp32 (names as in the reference's table).
kLowPrecisionOps = ("Matmul", "Linear")
kFP32Ops = ("Sin", "Cos", "Tanh", "Exp", "Log", "Sqrt", "Reciprocal", "Rsqrt", "Pow", "Prod", "CrossEntropy",
            "VocabParallelCrossEntropy", "LayerNorm", "RMSNorm", "Softmax")


class AutocastGuard:
    def __init__(self, device_type=DeviceType.kCUDA, dtype=DataType.kBFLOAT16, enabled: bool = True):
        self.device_type = device_type
        self.dtype = to_torch_dtype(dtype)
        self.enabled = enabled and self.dtype != torch.float32
        self._prev = None

    def __enter__(self):
        self._prev = (ops._AutocastState.enabled, ops._AutocastState.dtype)
        ops._AutocastState.enabled = self.enabled
        ops._AutocastState.dtype = self.dtype
        return self

    def Disable(self):
        """Turns autocast off for the rest of the scope (the reference disables it before
        ``Backward``)."""
        ops._AutocastState.enabled = False

    def __exit__(self, *exc):
        ops._AutocastState.enabled, ops._AutocastState.dtype = self._prev
        return False


class NoGradGuard:
    def __enter__(self):
        self._ctx = torch.no_grad()
        self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        return self._ctx.__exit__(*exc)


def SavedTensorHooksGuard(pack, unpack):
    """Pack / unpack hooks for tensors saved for backward (reference: FunctionCtx::SavedTensorHooks,
    infini_train/include/autograd/function.h:19-37) — the enabling mechanism for activation
    off-loading or recomputation."""
    return torch.autograd.graph.saved_tensors_hooks(pack, unpack)
