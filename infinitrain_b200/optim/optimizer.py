"""Optimizers: SGD and Adam / AdamW.

Reference: infini_train/include/optimizer.h:35-68, infini_train/src/optimizer.cc:23-105 (one kernel
launch per parameter tensor, Adam without weight decay, state in the parameter dtype, ``t``
incremented even when every gradient is missing, positional state-dict keys ``adam.m.<i>``,
``adam.v.<i>``, ``adam.t``).

On CUDA with fp32 parameters the optimizer is FUSED: the parameters are moved into one flat
:class:`ParamAndGradBuffer` (fp32 master + fp32 gradients + bf16 shadow) and ``Step`` is a single
kernel launch that updates m, v and the master weights and writes the bf16 copy the GEMMs read.
``weight_decay`` adds the decoupled AdamW term (0 reproduces the reference's update exactly).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable, Dict, List, Optional, Sequence

import torch

from .. import _ext
from ..ops import functional as ops

OptimizerCreator = Callable[[Sequence[torch.nn.Parameter]], "Optimizer"]


class Optimizer:
    def __init__(self, params: Sequence[torch.nn.Parameter]):
        self.params: List[torch.nn.Parameter] = list(params)
        self._flat = None   # ParamAndGradBuffer when the fused flat path is active
        self._per_tensor_fused = False

    # ------------------------------------------------------------------ gradients
    def ZeroGrad(self, set_to_none: bool = True) -> None:
        if self._flat is not None:
            # Gradients are views of one flat buffer: a single memset; the views stay in place.
            self._flat.zero_grads()
            return
        for p in self.params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()

    def Step(self) -> None:
        raise NotImplementedError

    def StateDict(self) -> "OrderedDict[str, torch.Tensor]":
        return OrderedDict()

    def LoadStateDict(self, state_dict: Dict[str, torch.Tensor]) -> None:
        pass

    # torch-style aliases
    zero_grad = ZeroGrad
    step = Step

    # ------------------------------------------------------------------ fused path set-up
    def _maybe_flatten(self, fused: Optional[bool]):
        from ..parallel.ddp.param_and_grad_buffer import ParamAndGradBuffer

        can = (len(self.params) > 0 and all(p.is_cuda and p.dtype == torch.float32 for p in self.params)
               and _ext.available())
        if fused is None:
            fused = can
        self._per_tensor_fused = False
        if fused and can and any(getattr(p, "_itb_no_flatten", False) for p in self.params):
            # Parameters that are already slices of somebody's flat buffer (ZeRO shards) are
            # updated where they are: one fused launch per tensor.
            self._per_tensor_fused = True
            return
        if not fused:
            return
        if not can:
            raise ValueError("fused optimizer needs CUDA fp32 parameters and the native extension")
        existing = getattr(self.params[0], "_itb_flat_buffer", None)
        if existing is not None and all(getattr(p, "_itb_flat_buffer", None) is existing for p in self.params) \
                and len(existing.params) == len(self.params):
            self._flat = existing     # e.g. built by DistributedDataParallel
            return
        self._flat = ParamAndGradBuffer(self.params)
        for p in self.params:
            p._itb_flat_buffer = self._flat


class SGD(Optimizer):
    def __init__(self, params, learning_rate: float, fused: Optional[bool] = None):
        super().__init__(params)
        self.learning_rate = learning_rate
        self._maybe_flatten(fused)

    def Step(self) -> None:
        if self._flat is not None:
            C = _ext.load()
            C.sgd(self._flat.param_buffer, self._flat.grad_buffer, self._flat.shadow_buffer, self.learning_rate, 1.0)
            ops._counters["launches"] += 1
            self._flat.mark_shadows_fresh()
            return
        if self._per_tensor_fused:
            C = _ext.load()
            for p in self.params:
                if p.grad is None:
                    continue
                C.sgd(p.data, p.grad, getattr(p, "_itb_shadow", None), self.learning_rate, 1.0)
                ops._counters["launches"] += 1
            return
        with torch.no_grad():
            for p in self.params:
                if p.grad is None:
                    continue
                p.add_(p.grad.to(p.dtype), alpha=-self.learning_rate)

    @staticmethod
    def Create(learning_rate: float, **kw) -> OptimizerCreator:
        return lambda params: SGD(params, learning_rate, **kw)


class Adam(Optimizer):
    def __init__(self, params, learning_rate: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999,
                 eps: float = 1e-8, weight_decay: float = 0.0, fused: Optional[bool] = None):
        super().__init__(params)
        self.t = 0
        self.learning_rate, self.beta1, self.beta2, self.eps = learning_rate, beta1, beta2, eps
        self.weight_decay = weight_decay
        self._maybe_flatten(fused)
        if self._flat is not None:
            self._m_flat = torch.zeros_like(self._flat.param_buffer)
            self._v_flat = torch.zeros_like(self._flat.param_buffer)
            self.m = [self._m_flat[s:e].view(p.shape) for p, (s, e, _) in zip(self.params, self._flat.layout.param_ranges)]
            self.v = [self._v_flat[s:e].view(p.shape) for p, (s, e, _) in zip(self.params, self._flat.layout.param_ranges)]
        else:
            self.m = [torch.zeros_like(p) for p in self.params]
            self.v = [torch.zeros_like(p) for p in self.params]

    # ------------------------------------------------------------------ device-resident step state
    def _dev_hyper(self):
        """``[lr, 1/bc1, 1/bc2, t]`` on the device (fused paths only).  The step counter and the bias
        corrections are advanced by a one-thread kernel, so a captured training step replays with
        the right values and nothing step-dependent is passed from the host."""
        if getattr(self, "_hyper", None) is None:
            dev = self.params[0].device
            self._hyper = torch.tensor([self.learning_rate, 1.0, 1.0, float(self.t)], dtype=torch.float32, device=dev)
            self._hyper_lr = self.learning_rate
            self._prepared = False
        if self._hyper_lr != self.learning_rate:       # learning-rate change: one small synchronous copy
            self._hyper[0:1].fill_(self.learning_rate)
            self._hyper_lr = self.learning_rate
        return self._hyper

    def PrepareStep(self) -> None:
        """Advances the device-side step counter for the step about to be taken.  Fused ZeRO launches
        that run during backward need it before ``Step``; ``ZeroGrad`` of the distributed optimizer
        calls it, ``Step`` calls it when nobody did."""
        if self._flat is None and not self._per_tensor_fused:
            return
        h = self._dev_hyper()
        if not self._prepared:
            _ext.load().adam_advance(h, self.beta1, self.beta2)
            ops._counters["launches"] += 1
            self._prepared = True

    def Step(self) -> None:
        fused = self._flat is not None or self._per_tensor_fused
        if fused:
            self.PrepareStep()
            self._prepared = False
        self.t += 1
        bc1 = 1.0 - self.beta1 ** self.t
        bc2 = 1.0 - self.beta2 ** self.t
        if self._flat is not None:
            C = _ext.load()
            C.adamw(self._flat.param_buffer, self._flat.grad_buffer, self._m_flat, self._v_flat,
                    self._flat.shadow_buffer, self.learning_rate, self.beta1, self.beta2, self.eps,
                    self.weight_decay, bc1, bc2, 1.0, self._hyper)
            ops._counters["launches"] += 1
            self._flat.mark_shadows_fresh()
            return
        if self._per_tensor_fused:
            C = _ext.load()
            for p, m, v in zip(self.params, self.m, self.v):
                if p.grad is None:
                    continue
                C.adamw(p.data, p.grad, m, v, getattr(p, "_itb_shadow", None), self.learning_rate, self.beta1,
                        self.beta2, self.eps, self.weight_decay, bc1, bc2, 1.0, self._hyper)
                ops._counters["launches"] += 1
            return
        with torch.no_grad():
            for p, m, v in zip(self.params, self.m, self.v):
                if p.grad is None:
                    continue
                g = p.grad.to(p.dtype)
                m.mul_(self.beta1).add_(g, alpha=1.0 - self.beta1)
                v.mul_(self.beta2).addcmul_(g, g, value=1.0 - self.beta2)
                upd = (m / bc1) / ((v / bc2).sqrt() + self.eps)
                if self.weight_decay:
                    upd = upd + self.weight_decay * p
                p.add_(upd, alpha=-self.learning_rate)

    @staticmethod
    def Create(learning_rate: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
               weight_decay: float = 0.0, **kw) -> OptimizerCreator:
        return lambda params: Adam(params, learning_rate, beta1, beta2, eps, weight_decay, **kw)

    def StateDict(self):
        out = OrderedDict()
        for i, (m, v) in enumerate(zip(self.m, self.v)):
            out[f"adam.m.{i}"] = m
            out[f"adam.v.{i}"] = v
        out["adam.t"] = torch.tensor(self.t, dtype=torch.int64)
        return out

    def NamedStateDict(self, model) -> "OrderedDict[str, torch.Tensor]":
        """The same state keyed by parameter NAME (``adam.m.transformer.h.0.attn.c_attn.weight``): it
        survives a change of parameter order or a frozen subset; ``LoadStateDict`` takes either form."""
        names = self._param_names(model)
        out = OrderedDict()
        for i, (m, v) in enumerate(zip(self.m, self.v)):
            out[f"adam.m.{names[i]}"] = m
            out[f"adam.v.{names[i]}"] = v
        out["adam.t"] = torch.tensor(self.t, dtype=torch.int64)
        return out

    def _param_names(self, model):
        by_id = {}
        named = model.NamedParameters() if hasattr(model, "NamedParameters") else model.named_parameters()
        for name, p in named:
            by_id.setdefault(id(p), name)
        missing = [i for i, p in enumerate(self.params) if id(p) not in by_id]
        if missing:
            raise KeyError(f"optimizer parameter {missing[0]} is not a parameter of the model")
        return [by_id[id(p)] for p in self.params]

    def LoadStateDict(self, state_dict, model=None):
        names = self._param_names(model) if model is not None else None
        for i, (m, v) in enumerate(zip(self.m, self.v)):
            for kind, dst in (("m", m), ("v", v)):
                key = f"adam.{kind}.{i}"
                if key not in state_dict and names is not None:
                    key = f"adam.{kind}.{names[i]}"
                if key not in state_dict:
                    raise KeyError(f"Missing optimizer state: {key}")
                with torch.no_grad():
                    dst.copy_(state_dict[key].to(dst.device))
        if "adam.t" not in state_dict:
            raise KeyError("Missing optimizer state: adam.t")
        self.t = int(state_dict["adam.t"].item())
        if getattr(self, "_hyper", None) is not None:
            self._hyper[3:4].fill_(float(self.t))
            self._prepared = False


AdamW = Adam
