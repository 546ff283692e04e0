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


def _adapter_generator(config: LoRAConfig, global_path: str):
    """``config.seed`` and the FNV-1a hash of the module's whole-model path seed the adapter's own generator."""
    if not config.seed:
        return None
    h = 2166136261
    for c in global_path.encode():
        h = ((h ^ c) * 16777619) & 0xFFFFFFFF
    return torch.Generator().manual_seed((config.seed ^ h) & 0xFFFFFFFF)


def _wrap(m, config: LoRAConfig, generator=None):
    if _is_lora(m):
        return None
    if isinstance(m, ColumnParallelLinear):
        return LoRAColumnParallelLinear(m, config, generator)
    if isinstance(m, RowParallelLinear):
        return LoRARowParallelLinear(m, config, generator)
    if isinstance(m, Linear):
        return LoRALinear(config=config, base_module=m, generator=generator)
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
    # a module's whole-model name: its state-dict path (the pipeline's chunk aliases name the same modules under
    # shorter paths) with the stage's local layer number turned into the global one
    local_to_global = dict(enumerate(_global_layer_indices(model)))
    state_path = {}
    if config.seed:
        for n, m in _modules_by_state_dict_path(model).items():
            if not any(part.startswith("__pp") for part in n.split(".")):
                state_path.setdefault(id(m), n)
    for path, parent, name, child in _named_children_paths(model):
        clean = ".".join(p for p in path.split(".") if not p.startswith("__pp"))
        if not config.ShouldApplyLoRA(clean) and not config.ShouldApplyLoRA(path):
            continue
        if id(child) in replaced:
            parent._modules[name] = replaced[id(child)]
            continue
        whole = state_path.get(id(child), clean)
        new = _wrap(child, config, _adapter_generator(config, _rename_layer(whole, local_to_global) if local_to_global else whole))
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


# --------------------------------------------------------------------------- topology-independent adapters
def _global_layer_indices(model) -> List[int]:
    """Global index of every layer this rank holds, in the order of its local ``transformer.h.<i>`` names."""
    info = getattr(model, "stage_info", None)
    if info is None:
        return []
    out: List[int] = []
    for s, e in sorted(info.layer_ranges_per_chunk):
        out += list(range(s, e))
    return out


def _rename_layer(name: str, mapping: Dict[int, int]) -> str:
    parts = name.split(".")
    if len(parts) > 2 and parts[0] == "transformer" and parts[1] == "h" and parts[2].isdigit():
        parts[2] = str(mapping[int(parts[2])])
    return ".".join(parts)


def _qkv_split(model, name: str):
    """(q_rows, kv_rows) of the full fused projection when ``name`` is an attention ``c_attn``, else None."""
    cfg = getattr(model, "config", None)
    if cfg is None or not name.endswith("attn.c_attn.lora_B"):
        return None
    d = cfg.head_dim()
    return cfg.n_head * d, cfg.n_kv_head * d


def _modules_by_state_dict_path(model) -> Dict[str, Module]:
    """path -> module with the paths state-dict keys use (``transformer.h.0.attn.c_attn``)."""
    if hasattr(model, "NamedModules"):
        return {n: m for n, m in model.NamedModules(remove_duplicate=False)}
    return dict(model.named_modules(remove_duplicate=False))


def GatherFullLoRAStateDict(model: Module) -> "OrderedDict[str, torch.Tensor]":
    """The adapters of the WHOLE model under global names, assembled from every tensor- and
    pipeline-parallel rank (a collective over all ranks of the job; every rank gets the result).
    Column-parallel B factors are concatenated along the output rows (a fused QKV projection back into
    its Q | K | V order), row-parallel A factors along the input columns, replicated factors are taken
    from tensor-parallel rank 0, and a stage's local layer numbers become global ones."""
    import torch.distributed as dist

    from ...parallel import global_env as genv

    tp, tp_rank = genv.GetTensorParallelSize(), genv.GetTensorParallelRank()
    local_to_global = dict(enumerate(_global_layer_indices(model)))
    mine = {}
    mods = _modules_by_state_dict_path(model)
    for name, t in LoRAStateDict(model).items():
        owner = mods.get(name.rsplit(".", 1)[0])
        kind = "rep"
        if isinstance(owner, LoRAColumnParallelLinear) and name.endswith("lora_B") and tp > 1:
            kind = "rows"
        elif isinstance(owner, LoRARowParallelLinear) and name.endswith("lora_A") and tp > 1:
            kind = "cols"
        mine[_rename_layer(name, local_to_global) if local_to_global else name] = (kind, tp_rank, t.detach().float().cpu())
    if dist.is_initialized() and dist.get_world_size() > 1:
        everyone = [None] * dist.get_world_size()
        dist.all_gather_object(everyone, mine if genv.GetDataParallelRank() == 0 else {})
    else:
        everyone = [mine]
    pieces: Dict[str, Dict[int, torch.Tensor]] = {}
    kinds: Dict[str, str] = {}
    for d in everyone:
        for name, (kind, r, t) in d.items():
            pieces.setdefault(name, {})[r] = t
            kinds[name] = kind
    out = OrderedDict()
    for name in sorted(pieces):
        shards = [pieces[name][r] for r in sorted(pieces[name])]
        if kinds[name] == "rep":
            out[name] = shards[0]
        elif kinds[name] == "cols":
            out[name] = torch.cat(shards, dim=1)
        else:
            split = _qkv_split(model, name)
            if split is None:
                out[name] = torch.cat(shards, dim=0)
            else:
                q, kv = split[0] // len(shards), split[1] // len(shards)
                out[name] = torch.cat([s[:q] for s in shards] + [s[q:q + kv] for s in shards] + [s[q + kv:] for s in shards], 0)
    return out


def ScatterFullLoRAStateDict(model: Module, full: Dict[str, torch.Tensor]) -> int:
    """Loads this rank's part of a whole-model adapter dict (global names, unsharded factors): the
    inverse of :func:`GatherFullLoRAStateDict`.  Returns the number of tensors loaded."""
    from ...parallel import global_env as genv

    tp, tp_rank = genv.GetTensorParallelSize(), genv.GetTensorParallelRank()
    local_to_global = dict(enumerate(_global_layer_indices(model)))
    mods = _modules_by_state_dict_path(model)
    n = 0
    for name, dst in LoRAStateDict(model).items():
        gname = _rename_layer(name, local_to_global) if local_to_global else name
        if gname not in full:
            raise KeyError(f"adapter file has no tensor '{gname}'")
        src = full[gname].float()
        owner = mods.get(name.rsplit(".", 1)[0])
        if tp > 1 and isinstance(owner, LoRAColumnParallelLinear) and name.endswith("lora_B"):
            split = _qkv_split(model, name)
            if split is None:
                k = src.shape[0] // tp
                src = src[tp_rank * k:(tp_rank + 1) * k]
            else:
                qr, kvr = split
                q, k_, v = src[:qr], src[qr:qr + kvr], src[qr + kvr:]
                src = torch.cat([t[tp_rank * (t.shape[0] // tp):(tp_rank + 1) * (t.shape[0] // tp)] for t in (q, k_, v)], 0)
        elif tp > 1 and isinstance(owner, LoRARowParallelLinear) and name.endswith("lora_A"):
            k = src.shape[1] // tp
            src = src[:, tp_rank * k:(tp_rank + 1) * k]
        if tuple(src.shape) != tuple(dst.shape):
            raise ValueError(f"adapter tensor '{gname}' has shape {tuple(src.shape)}, this rank needs {tuple(dst.shape)}")
        with torch.no_grad():
            dst.copy_(src.to(dst.device, dst.dtype))
        n += 1
    return n


def _write_lora_file(sd: Dict[str, torch.Tensor], filepath: str) -> None:
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


def _read_lora_file(filepath: str) -> Dict[str, torch.Tensor]:
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
            sd[name] = torch.from_numpy(np.frombuffer(f.read(4 * n), dtype="<f4").reshape(dims).copy())
    return sd


def SaveFullLoRAWeights(model: Module, filepath: str) -> None:
    """One adapter file for the whole model, whatever the parallel layout it was trained in (collective
    over all ranks; global rank 0 writes).  The file is an ordinary adapter file: a single-rank run,
    the C++ frontend and the reference read it."""
    import torch.distributed as dist

    full = GatherFullLoRAStateDict(model)
    if not dist.is_initialized() or dist.get_rank() == 0:
        _write_lora_file(full, filepath)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def LoadFullLoRAWeights(model: Module, filepath: str) -> None:
    """Loads a whole-model adapter file into this rank's shard of the model (any parallel layout)."""
    ScatterFullLoRAStateDict(model, _read_lora_file(filepath))


def SaveLoRAWeights(model: Module, filepath: str) -> None:
    """This rank's adapter tensors under their local names (the reference's file: magic 0x4C4F5241,
    version 1, fp32; src/nn/lora/lora_utils.cc:309-358)."""
    _write_lora_file(LoRAStateDict(model), filepath)


def LoadLoRAWeights(model: Module, filepath: str) -> None:
    LoadLoRAStateDict(model, _read_lora_file(filepath))


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
