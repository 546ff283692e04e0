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
    layer = 0
    layer_name = ""

    @classmethod
    def Set(cls, gas_step: int = 0, layer: int = 0, layer_name: str = ""):
        cls.gas_step, cls.layer, cls.layer_name = gas_step, layer, layer_name

    @classmethod
    def Key(cls) -> str:
        """``[GAS-g] [L-l] name`` (reference: src/utils/precision_check_context.cc:22-29)."""
        return f"[GAS-{cls.gas_step}] [L-{cls.layer}]" + (f" {cls.layer_name}" if cls.layer_name else "")


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
        # the reference's quantisation, bit for bit (src/utils/precision_checker.cc:249-260): double
        # arithmetic, round half away from zero, back to fp32
        x = a.astype(np.float64) * (1.0 / tolerance)
        a = (np.sign(x) * np.floor(np.abs(x) + 0.5) * tolerance).astype(np.float32)
    return hashlib.md5(a.tobytes()).hexdigest()


def _g(v: float) -> str:
    """A float the way a C++ stream prints it by default (six significant digits)."""
    return f"{v:.6g}"


def _dtype_name(t: torch.Tensor) -> str:
    return str(t.dtype).replace("torch.", "")


def Summarize(t: torch.Tensor) -> str:
    """``dtype=float32 shape=(4,64,96) min=.. max=.. mean=.. [v0, .., v5, ...] [NaN:0 Inf:0]``: the
    body of the reference's ``simple`` line (src/utils/precision_checker.cc:352-371)."""
    flat = t.detach().float().reshape(-1)
    shape = "(" + ",".join(str(d) for d in t.shape) + ")"
    head = f"dtype={_dtype_name(t)} shape={shape} "
    if flat.numel() == 0:
        return head + "min=0 max=0 mean=0 [] [NaN:0 Inf:0]"
    nan, inf = int(torch.isnan(flat).sum()), int(torch.isinf(flat).sum())
    first = ", ".join(_g(v) for v in flat[:6].cpu().tolist()) + (", ..." if flat.numel() > 6 else "")
    return (head + f"min={_g(flat.min().item())} max={_g(flat.max().item())} mean={_g(flat.double().mean().item())} "
            f"[{first}] [NaN:{nan} Inf:{inf}]")


class PrecisionChecker:
    _name_map: Dict[int, str] = {}
    _orig_fns = {}

    @classmethod
    def BuildNameMap(cls, model, prefix: str = "") -> None:
        """Module -> dotted path, as the reference builds it (src/utils/precision_checker.cc:397-418):
        the root and the pipeline-internal ``__pp*`` subtrees are skipped, so layers carry their
        state-dict paths (``transformer.h.0.attn.c_attn``) and the stage wrappers their type names."""
        cls._name_map = {}
        named = (model.NamedModules(remove_duplicate=False) if hasattr(model, "NamedModules")
                 else list(model.named_modules(remove_duplicate=False)))
        for name, mod in named:
            if not name or name.startswith("__pp"):
                continue
            cls._name_map.setdefault(id(mod), (prefix + "." if prefix else "") + name)

    @classmethod
    def ResetCounters(cls):
        PrecisionCheckEnv.Instance().ResetCounters()

    @classmethod
    def _record(cls, stage: str, name: str, i: int, t: torch.Tensor):
        """One line ``<context> <name>[_<n>]_<forward|backward> tensor[<i>]: ...`` and, when asked, one
        ``rank_<r>/<name>[_<n>]_<stage>.npy``; ``n`` counts the records of this (name, stage) since the
        last ``ResetCounters`` (reference: src/utils/precision_checker.cc:281-371)."""
        env = PrecisionCheckEnv.Instance()
        cfg = env.config
        if cfg.level == PrecisionCheckLevel.OFF or not isinstance(t, torch.Tensor) or not t.is_floating_point():
            return
        short = "forward" if "Forward" in stage else "backward"
        n = env.GetAndIncrementCounter(f"{name}_{short}")
        log_name = name + (f"_{n}" if n > 0 else "") + "_" + short
        if cfg.format == "md5":
            shape = "(" + ",".join(str(d) for d in t.shape) + ")"
            body = f"dtype={_dtype_name(t)} shape={shape} md5={ComputeMD5(t, cfg.md5_tolerance)}"
        else:
            body = Summarize(t)
        with open(os.path.join(env.timestamped_path, f"precision_check_rank_{env.rank}.log"), "a") as f:
            f.write(f"{PrecisionCheckContext.Key()} {log_name} tensor[{i}]: {body}\n")
        if cfg.save_tensors:
            d = os.path.join(env.timestamped_path, f"rank_{env.rank}")
            os.makedirs(d, exist_ok=True)
            np.save(os.path.join(d, f"{log_name}.npy"), t.detach().float().cpu().numpy())

    @classmethod
    def ModuleForwardHook(cls, module, inputs, outputs):
        name = cls._name_map.get(id(module), getattr(module, "kType", None) or type(module).__name__)
        outs = outputs if isinstance(outputs, (tuple, list)) else (outputs,)
        for i, o in enumerate(outs):
            cls._record("Forward Output", name, i, o)

    @classmethod
    def ModuleBackwardHook(cls, module, grad_outputs, grad_inputs):
        name = cls._name_map.get(id(module), getattr(module, "kType", None) or type(module).__name__)
        for i, g in enumerate(grad_outputs or ()):
            cls._record("GradOutputs", name, i, g)

    # fused op -> record name, after the reference's ``<kType>Function`` names where an op of that
    # type exists there (src/autograd/*.cc); the fused ops have no finer-grained records
    _FUNCTION_NAMES = {"linear": "LinearFunction", "mlp_gelu": "MlpGeluFunction", "layernorm": "LayerNormFunction",
                       "rmsnorm": "RMSNormFunction", "gelu": "GeluFunction", "swiglu": "SwiGLUFunction",
                       "attention_packed": "AttentionFunction", "embedding": "EmbeddingFunction",
                       "cross_entropy": "CrossEntropyFunction"}

    @classmethod
    def InstallFunctionHooks(cls):
        """FUNCTION level: every fused op of ``ops.functional`` records its tensor inputs and its output
        under ``<Name>Function_forward`` and the gradient that reaches its output under
        ``<Name>Function_backward`` (reference: RegisterForFunction, src/utils/precision_checker.cc:420-446)."""
        from ..ops import functional as ops

        for fname, rec in cls._FUNCTION_NAMES.items():
            if fname in cls._orig_fns:
                continue
            orig = getattr(ops, fname)
            cls._orig_fns[fname] = orig

            def wrapped(*a, _orig=orig, _n=rec, **k):
                for i, t in enumerate(x for x in a if isinstance(x, torch.Tensor)):
                    cls._record("Forward Input", _n, i, t)
                out = _orig(*a, **k)
                cls._record("Forward Output", _n, 0, out)
                if isinstance(out, torch.Tensor) and out.requires_grad:
                    out.register_hook(lambda g, _n=_n: cls._record("Backward Input", _n, 0, g))
                return out

            setattr(ops, fname, wrapped)

    @classmethod
    def RemoveFunctionHooks(cls):
        from ..ops import functional as ops

        for fname, orig in cls._orig_fns.items():
            setattr(ops, fname, orig)
        cls._orig_fns = {}
