"""Precision checker: per-module / per-function tensor summaries for cross-framework alignment.

Reference: infini_train/src/utils/precision_checker.cc:31-473, precision_check_config.cc,
precision_check_context.h, docs/precision_checker_guide.md.  Levels OFF / MODULE / FUNCTION; formats
``simple`` (min / max / mean / first six values / NaN and Inf counts) or ``md5`` (hash of the raw
fp32 bytes, optionally quantised to a tolerance first); optional ``.npy`` dumps; one log per rank;
a context (micro-batch / layer) and counters that reset every iteration so file names repeat across
steps.  MODULE level hooks every :class:`infinitrain_b200.nn.Module` call through the global hook
registry; FUNCTION level additionally records every fused op of :mod:`ops.functional`.
"""
from __future__ import annotations

import enum
import hashlib
import os
import time
from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np
import torch

from .global_module_hook_registry import GlobalModuleHookRegistry


class PrecisionCheckLevel(enum.IntEnum):
    OFF = 0
    MODULE = 1
    FUNCTION = 2


@dataclass
class PrecisionCheckConfig:
    level: PrecisionCheckLevel = PrecisionCheckLevel.OFF
    output_path: str = "./log_precision_check"
    format: str = "simple"
    save_tensors: bool = False
    md5_tolerance: float = 0.0

    @staticmethod
    def Parse(config_str: str) -> "PrecisionCheckConfig":
        """``"level=1,format=md5,path=./out,save_tensors=true,md5_tolerance=1e-3"``"""
        cfg = PrecisionCheckConfig()
        kv = {}
        for part in (config_str or "").split(","):
            if "=" in part:
                k, v = part.split("=", 1)
                kv[k.strip()] = v.strip()
        if "level" in kv:
            cfg.level = PrecisionCheckLevel(int(kv["level"]))
        if "path" in kv:
            cfg.output_path = kv["path"]
        if "format" in kv:
            cfg.format = kv["format"]
        if "save_tensors" in kv:
            cfg.save_tensors = kv["save_tensors"] in ("true", "1")
        if "md5_tolerance" in kv:
            cfg.md5_tolerance = float(kv["md5_tolerance"])
        return cfg


class PrecisionCheckContext:
    """Where in the step the checker is (micro-batch index, layer); part of every record key."""

    gas_step = 0
    layer = ""

    @classmethod
    def Set(cls, gas_step: int = 0, layer: str = ""):
        cls.gas_step, cls.layer = gas_step, layer

    @classmethod
    def Key(cls) -> str:
        return f"[GAS-{cls.gas_step}]" + (f"[{cls.layer}]" if cls.layer else "")


class PrecisionCheckEnv:
    _instance = None

    def __init__(self):
        self.config = PrecisionCheckConfig()
        self.timestamped_path = ""
        self._counters: Dict[str, int] = {}
        self._handles = []

    @classmethod
    def Instance(cls) -> "PrecisionCheckEnv":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def Init(self, config: PrecisionCheckConfig, rank: int = 0) -> None:
        self.Shutdown()
        self.config = config
        self.rank = rank
        if config.level == PrecisionCheckLevel.OFF:
            return
        self.timestamped_path = os.path.join(config.output_path, time.strftime("%Y%m%d_%H%M%S"))
        os.makedirs(self.timestamped_path, exist_ok=True)
        reg = GlobalModuleHookRegistry.Instance()
        self._handles = [reg.RegisterModuleForwardHook(PrecisionChecker.ModuleForwardHook),
                         reg.RegisterModuleFullBackwardHook(PrecisionChecker.ModuleBackwardHook)]
        if config.level >= PrecisionCheckLevel.FUNCTION:
            PrecisionChecker.InstallFunctionHooks()

    def Shutdown(self):
        for h in self._handles:
            h.Remove()
        self._handles = []
        PrecisionChecker.RemoveFunctionHooks()
        self.config = PrecisionCheckConfig()

    def GetConfig(self):
        return self.config

    def GetOutputPath(self):
        return self.timestamped_path

    def GetAndIncrementCounter(self, key: str) -> int:
        v = self._counters.get(key, 0)
        self._counters[key] = v + 1
        return v

    def ResetCounters(self):
        self._counters.clear()


def ComputeMD5(t: torch.Tensor, tolerance: float = 0.0) -> str:
    a = t.detach().float().cpu().contiguous().numpy()
    if tolerance > 0:
        a = (np.round(a / tolerance) * tolerance).astype(np.float32)
    return hashlib.md5(a.tobytes()).hexdigest()


def Summarize(t: torch.Tensor) -> str:
    f = t.detach().float()
    flat = f.reshape(-1)
    first = ", ".join(f"{v:.6g}" for v in flat[:6].cpu().tolist())
    nan, inf = int(torch.isnan(flat).sum()), int(torch.isinf(flat).sum())
    if flat.numel() == 0:
        return "empty"
    return (f"shape={tuple(t.shape)} dtype={str(t.dtype).replace('torch.', '')} min={flat.min().item():.6g} "
            f"max={flat.max().item():.6g} mean={flat.mean().item():.6g} first6=[{first}] nan={nan} inf={inf}")


class PrecisionChecker:
    _name_map: Dict[int, str] = {}
    _orig_fns = {}

    @classmethod
    def BuildNameMap(cls, model, prefix: str = "") -> None:
        cls._name_map = {}
        named = model.NamedModules() if hasattr(model, "NamedModules") else list(model.named_modules())
        for name, mod in named:
            cls._name_map.setdefault(id(mod), name or prefix or type(mod).__name__)

    @classmethod
    def ResetCounters(cls):
        PrecisionCheckEnv.Instance().ResetCounters()

    @classmethod
    def _record(cls, kind: str, name: str, idx: int, t: torch.Tensor):
        env = PrecisionCheckEnv.Instance()
        cfg = env.config
        if cfg.level == PrecisionCheckLevel.OFF or not isinstance(t, torch.Tensor) or not t.is_floating_point():
            return
        key = f"{PrecisionCheckContext.Key()}[{kind}] {name} #{idx}"
        n = env.GetAndIncrementCounter(key)
        body = ComputeMD5(t, cfg.md5_tolerance) if cfg.format == "md5" else Summarize(t)
        with open(os.path.join(env.timestamped_path, f"precision_check_rank_{env.rank}.log"), "a") as f:
            f.write(f"{key} ({n}): {body}\n")
        if cfg.save_tensors:
            safe = key.replace("/", "_").replace(" ", "_").replace("[", "").replace("]", "_").replace("#", "")
            d = os.path.join(env.timestamped_path, f"rank_{env.rank}")
            os.makedirs(d, exist_ok=True)
            np.save(os.path.join(d, f"{safe}_{n}.npy"), t.detach().float().cpu().numpy())

    @classmethod
    def ModuleForwardHook(cls, module, inputs, outputs):
        name = cls._name_map.get(id(module), type(module).__name__)
        outs = outputs if isinstance(outputs, (tuple, list)) else (outputs,)
        for i, o in enumerate(outs):
            cls._record("Forward Output", name, i, o)

    @classmethod
    def ModuleBackwardHook(cls, module, grad_outputs, grad_inputs):
        name = cls._name_map.get(id(module), type(module).__name__)
        for i, g in enumerate(grad_outputs or ()):
            cls._record("Backward GradOutput", name, i, g)

    @classmethod
    def InstallFunctionHooks(cls):
        from ..ops import functional as ops

        for fname in ("linear", "mlp_gelu", "layernorm", "rmsnorm", "gelu", "swiglu", "attention_packed", "embedding",
                      "cross_entropy"):
            if fname in cls._orig_fns:
                continue
            orig = getattr(ops, fname)
            cls._orig_fns[fname] = orig

            def wrapped(*a, _orig=orig, _n=fname, **k):
                out = _orig(*a, **k)
                cls._record("Function Output", _n, 0, out)
                return out

            setattr(ops, fname, wrapped)

    @classmethod
    def RemoveFunctionHooks(cls):
        from ..ops import functional as ops

        for fname, orig in cls._orig_fns.items():
            setattr(ops, fname, orig)
        cls._orig_fns = {}
