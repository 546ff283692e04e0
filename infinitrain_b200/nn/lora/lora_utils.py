"""LoRA model utilities: injection, freezing, merging, state dict and adapter files.

Reference: infini_train/src/nn/lora/lora_utils.cc:23-462.  Adapter file: little-endian
``uint32 magic 0x4C4F5241 ("LORA"), uint32 version 1, uint32 count`` then per tensor
``uint32 name_len, name, uint32 ndim, int64 dims..., float32 data``.
"""
from __future__ import annotations

import struct
from collections import OrderedDict
from typing import Dict, List

import numpy as np
import torch

from ...parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear
from ..layers import Linear
from ..module import Module
from .lora_config import LoRAConfig, ParseLoRATargetModules  # noqa: F401
from .lora_layers import LoRAColumnParallelLinear, LoRALinear, LoRARowParallelLinear

kLoRAMagic = 0x4C4F5241
_LORA_TYPES = (LoRALinear, LoRAColumnParallelLinear, LoRARowParallelLinear)


def _is_lora(m) -> bool:
    return isinstance(m, _LORA_TYPES)


def _wrap(m, config: LoRAConfig):
    if _is_lora(m):
        return None
    if isinstance(m, ColumnParallelLinear):
        return LoRAColumnParallelLinear(m, config)
    if isinstance(m, RowParallelLinear):
        return LoRARowParallelLinear(m, config)
    if isinstance(m, Linear):
        return LoRALinear(config=config, base_module=m)
    return None


def _named_children_paths(model):
    """(path, parent, child name, child) for every module below ``model``; shared children (the
    pipeline aliases) are visited once per parent so every alias is replaced."""
    out = []
    seen_parent = set()

    def walk(mod, prefix):
        if id(mod) in seen_parent:
            return
        seen_parent.add(id(mod))
        for name, child in list(mod._modules.items()):
            if child is None:
                continue
            path = prefix + ("." if prefix else "") + name
            out.append((path, mod, name, child))
            walk(child, path)

    walk(model, "")
    return out


def ReplaceModuleByPath(model: Module, path: str, new_module: Module) -> None:
    parts = path.split(".")
    cur = model
    for p in parts[:-1]:
        cur = cur._modules[p]
    cur._modules[parts[-1]] = new_module


def InjectLoRALayers(model: Module, config: LoRAConfig) -> Module:
    """Replaces every matching linear by its LoRA variant (structure only, no freezing).  A root
    module that is itself a plain ``Linear`` matches by type name when its path is empty."""
    root_type = model.type() if isinstance(model, Module) else ""
    if isinstance(model, Linear) and not _is_lora(model) and (config.ShouldApplyLoRA(root_type) or
                                                              root_type in config.target_modules):
        return _wrap(model, config)
    replaced: Dict[int, Module] = {}
    for path, parent, name, child in _named_children_paths(model):
        clean = ".".join(p for p in path.split(".") if not p.startswith("__pp"))
        if not config.ShouldApplyLoRA(clean) and not config.ShouldApplyLoRA(path):
            continue
        if id(child) in replaced:
            parent._modules[name] = replaced[id(child)]
            continue
        new = _wrap(child, config)
        if new is not None:
            replaced[id(child)] = new
            parent._modules[name] = new
    return model


def FreezeBaseModel(model: Module) -> None:
    for p in model.parameters():
        p.requires_grad_(False)
    for p in GetLoRAParameters(model):
        p.requires_grad_(True)


def UnfreezeModel(model: Module) -> None:
    for p in model.parameters():
        p.requires_grad_(True)


def GetLoRAModel(model: Module, config: LoRAConfig) -> Module:
    model = InjectLoRALayers(model, config)
    FreezeBaseModel(model)
    return model


def _lora_modules(model) -> List[Module]:
    out, seen = [], set()
    for m in model.modules():
        if _is_lora(m) and id(m) not in seen:
            seen.add(id(m))
            out.append(m)
    return out


def GetLoRAParameters(model: Module) -> List[torch.nn.Parameter]:
    out = []
    for m in _lora_modules(model):
        out += m.LoRAParameters()
    return out


def GetBaseParameters(model: Module) -> List[torch.nn.Parameter]:
    lora = {id(p) for p in GetLoRAParameters(model)}
    return [p for p in model.parameters() if id(p) not in lora]


def MergeLoRAWeights(model: Module) -> None:
    for m in _lora_modules(model):
        m.MergeWeights()


def UnmergeLoRAWeights(model: Module) -> None:
    for m in _lora_modules(model):
        m.UnmergeWeights()


def _unwrap(m):
    if isinstance(m, LoRAColumnParallelLinear):
        base = ColumnParallelLinear.__new__(ColumnParallelLinear)
        Module.__init__(base, ColumnParallelLinear.kType)
        keys = ("in_features", "out_features", "output_size_per_partition", "has_bias", "gather_output",
                "input_is_parallel", "skip_bias_add", "sequence_parallel")
    elif isinstance(m, LoRARowParallelLinear):
        base = RowParallelLinear.__new__(RowParallelLinear)
        Module.__init__(base, RowParallelLinear.kType)
        keys = ("in_features", "out_features", "input_size_per_partition", "has_bias", "reduce_output",
                "input_is_parallel", "skip_bias_add", "sequence_parallel")
    else:
        base = Linear.__new__(Linear)
        Module.__init__(base, Linear.kType)
        keys = ("in_features", "out_features")
    for k in keys:
        setattr(base, k, getattr(m, k))
    base.weight, base.bias = m.weight, m.bias
    return base


def MergeAndUnload(model: Module) -> Module:
    """Folds every adapter into its base weight and replaces the LoRA modules by plain base modules
    that share the merged weight / bias; afterwards no LoRA parameter exists and every parameter
    is trainable."""
    MergeLoRAWeights(model)
    if _is_lora(model):
        model = _unwrap(model)
    else:
        replaced = {}
        for path, parent, name, child in _named_children_paths(model):
            if _is_lora(child):
                if id(child) not in replaced:
                    replaced[id(child)] = _unwrap(child)
                parent._modules[name] = replaced[id(child)]
    UnfreezeModel(model)
    return model


def LoRAStateDict(model: Module) -> "OrderedDict[str, torch.Tensor]":
    sd = model.StateDict() if isinstance(model, Module) else model.state_dict(keep_vars=True)
    return OrderedDict((k, v) for k, v in sd.items() if k.endswith(".lora_A") or k.endswith(".lora_B") or
                       k in ("lora_A", "lora_B"))


def LoadLoRAStateDict(model: Module, state_dict: Dict[str, torch.Tensor]) -> None:
    own = model.StateDict()
    for k, v in state_dict.items():
        if k in own:
            with torch.no_grad():
                own[k].copy_(v.to(own[k].device, own[k].dtype))
        else:
            import warnings

            warnings.warn(f"LoRA parameter not found in model: {k}")


def ShardedLoRAPath(filepath: str) -> str:
    """The adapter file of THIS rank.  With tensor or pipeline parallelism a rank holds a shard of
    the adapters (its slice of the sharded factors, the layers of its stage under their local
    names), so every (tp, pp) coordinate has a file of its own, ``<path>.tp<i>.pp<j>``; data-parallel
    replicas share it.  Without model parallelism the path is returned unchanged.  (In the reference
    every rank writes the one path it was given: example/gpt2/main.cc:531-534.)"""
    from ...parallel import global_env as genv

    tp, pp = genv.GetTensorParallelSize(), genv.GetPipelineParallelSize()
    if tp <= 1 and pp <= 1:
        return filepath
    return f"{filepath}.tp{genv.GetTensorParallelRank()}.pp{genv.GetPipelineParallelRank()}"


def SaveLoRAWeights(model: Module, filepath: str) -> None:
    sd = LoRAStateDict(model)
    with open(filepath, "wb") as f:
        f.write(struct.pack("<III", kLoRAMagic, 1, len(sd)))
        for name, t in sd.items():
            nb = name.encode()
            f.write(struct.pack("<I", len(nb)))
            f.write(nb)
            f.write(struct.pack("<I", t.dim()))
            for d in t.shape:
                f.write(struct.pack("<q", d))
            f.write(t.detach().float().cpu().contiguous().numpy().tobytes())


def LoadLoRAWeights(model: Module, filepath: str) -> None:
    with open(filepath, "rb") as f:
        magic, version, count = struct.unpack("<III", f.read(12))
        if magic != kLoRAMagic:
            raise ValueError("Invalid LoRA file format")
        if version != 1:
            raise ValueError(f"Unsupported LoRA file version: {version}")
        sd = {}
        for _ in range(count):
            (nlen,) = struct.unpack("<I", f.read(4))
            name = f.read(nlen).decode()
            (ndim,) = struct.unpack("<I", f.read(4))
            dims = [struct.unpack("<q", f.read(8))[0] for _ in range(ndim)]
            n = int(np.prod(dims)) if dims else 1
            data = np.frombuffer(f.read(4 * n), dtype="<f4").reshape(dims).copy()
            sd[name] = torch.from_numpy(data)
    LoadLoRAStateDict(model, sd)


def CountTrainableParameters(model: Module) -> int:
    return sum(p.numel() for p in model.parameters() if p.requires_grad)


def CountTotalParameters(model: Module) -> int:
    return sum(p.numel() for p in model.parameters())


def PrintLoRASummary(model: Module, print_fn=print) -> str:
    tr, tot = CountTrainableParameters(model), CountTotalParameters(model)
    lines = ["========== LoRA Model Summary ==========",
             f"Total parameters:     {tot}",
             f"Trainable parameters: {tr}",
             f"Frozen parameters:    {tot - tr}",
             f"Trainable ratio:      {100.0 * tr / max(tot, 1):.4f}%",
             f"LoRA modules:         {len(_lora_modules(model))}",
             "========================================"]
    text = "\n".join(lines)
    if print_fn:
        print_fn(text)
    return text
