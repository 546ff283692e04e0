"""``nn.Module`` with the reference's API shape on top of ``torch.nn.Module``.

Reference: infini_train/include/nn/modules/module.h:28-124, infini_train/src/nn/modules/module.cc.
Differences kept on purpose: parameters are registered in a deterministic order (the reference
iterates ``unordered_map``s), ``To(device)`` moves parameters in place so tied weights and hooks
survive, and ``StateDict`` skips the pipeline alias children named ``__pp*`` exactly as the
reference does.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch

from ..common.hook import HookHandle
from ..utils.global_module_hook_registry import GlobalModuleHookRegistry

kPPFirstStageName = "__pp_first_stage"
kPPLastStageName = "__pp_last_stage"
kPPChunkNamePrefix = "__pp_chunk_"


def _as_list(x):
    if x is None:
        return []
    if isinstance(x, (list, tuple)):
        return list(x)
    return [x]


class Module(torch.nn.Module):
    kUndefinedType = "Undefined"

    def __init__(self, type: str = kUndefinedType):
        super().__init__()
        self._type = type
        self._fwd_pre_hooks: list = []
        self._fwd_post_hooks: list = []
        self._bwd_pre_hooks: list = []
        self._bwd_post_hooks: list = []

    # ------------------------------------------------------------------ identity
    def type(self, *args, **kwargs):  # noqa: A003 - the reference names it ``type()``
        if args or kwargs:
            return super().type(*args, **kwargs)
        return self._type

    # ------------------------------------------------------------------ parameters / buffers
    def Parameters(self) -> List[torch.nn.Parameter]:
        """All parameters of the subtree, de-duplicated by identity, in registration order."""
        return list(self.parameters())

    def has_parameter(self, name: str) -> bool:
        return name in self._parameters and self._parameters[name] is not None

    def parameter(self, name: str) -> torch.nn.Parameter:
        return self._parameters[name]

    def mutable_parameter(self, name: str):
        return self._parameters[name]

    def set_parameter(self, name: str, value: torch.nn.Parameter) -> None:
        self._parameters[name] = value

    def Buffers(self) -> List[torch.Tensor]:
        return list(self.buffers())

    def modules_list(self) -> List["Module"]:
        """Direct and indirect sub-modules excluding ``self`` (the reference's ``modules()``)."""
        return [m for _, m in self.NamedModules() if m is not self]

    def mutable_module(self, name: str):
        return self._modules[name]

    def GetModule(self, name: str):
        """The reference's ``module(name)`` accessor (that name is left free for child modules called
        "module", which DistributedDataParallel and PipelineParallel use)."""
        return self._modules[name]

    def NamedModules(self, memory: Optional[set] = None, prefix: str = "", remove_duplicate: bool = True):
        """Pre-order list of ``(qualified name, module)`` with children visited in sorted-name order."""
        memory = set() if memory is None else memory
        out = []
        if remove_duplicate and id(self) in memory:
            return out
        memory.add(id(self))
        out.append((prefix, self))
        for name in sorted(self._modules.keys()):
            child = self._modules[name]
            if child is None:
                continue
            sub = prefix + ("." if prefix else "") + name
            if isinstance(child, Module):
                out += child.NamedModules(memory, sub, remove_duplicate)
            else:
                for n, m in child.named_modules(prefix=sub):
                    if not remove_duplicate or id(m) not in memory:
                        memory.add(id(m))
                        out.append((n, m))
        return out

    # ------------------------------------------------------------------ state dict
    def StateDict(self) -> "OrderedDict[str, torch.Tensor]":
        out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        self._state_dict_into(out, "")
        return out

    def _state_dict_into(self, out, prefix):
        for name, p in self._parameters.items():
            if p is not None:
                out[prefix + name] = p
        for name, b in self._buffers.items():
            if b is not None:
                out[prefix + name] = b
        for name, child in self._modules.items():
            if child is None or name.startswith("__pp"):
                continue
            if isinstance(child, Module):
                child._state_dict_into(out, prefix + name + ".")
            else:
                for k, v in child.state_dict(keep_vars=True).items():
                    out[prefix + name + "." + k] = v

    def LoadStateDict(self, state_dict: Dict[str, torch.Tensor]) -> None:
        """Strict on missing keys / shape / dtype; unexpected keys are ignored with a warning."""
        own = self.StateDict()
        for k, dst in own.items():
            if k not in state_dict:
                raise KeyError(f"LoadStateDict: missing key '{k}'")
            src = state_dict[k]
            if tuple(src.shape) != tuple(dst.shape):
                raise ValueError(f"LoadStateDict: shape mismatch for '{k}': {tuple(src.shape)} vs {tuple(dst.shape)}")
            if src.dtype != dst.dtype:
                raise ValueError(f"LoadStateDict: dtype mismatch for '{k}': {src.dtype} vs {dst.dtype}")
            with torch.no_grad():
                dst.copy_(src)
        extra = [k for k in state_dict if k not in own]
        if extra:
            import warnings

            warnings.warn(f"LoadStateDict: ignoring {len(extra)} unexpected key(s), e.g. '{extra[0]}'")

    # ------------------------------------------------------------------ call + hooks
    def Forward(self, *inputs):
        raise NotImplementedError("Forward function not implemented for this module")

    def forward(self, *inputs, **kwargs):
        return self.Forward(*inputs, **kwargs)

    def __call__(self, *inputs, **kwargs):
        reg = GlobalModuleHookRegistry.Instance()
        if reg.forward_pre_hooks:
            reg.CallModuleForwardPreHooks(self, inputs)
        for h in self._fwd_pre_hooks:
            h(self, inputs)
        outputs = super().__call__(*inputs, **kwargs)
        for h in self._fwd_post_hooks:
            h(self, inputs, outputs)
        if reg.forward_hooks:
            reg.CallModuleForwardHooks(self, inputs, outputs)
        if self._bwd_pre_hooks or self._bwd_post_hooks or reg.backward_hooks:
            self._install_backward_hooks(outputs, reg)
        return outputs

    def _install_backward_hooks(self, outputs, reg):
        for out in _as_list(outputs):
            if not isinstance(out, torch.Tensor) or out.grad_fn is None:
                continue
            fn = out.grad_fn
            if self._bwd_pre_hooks:
                fn.register_prehook(lambda grad_outputs, m=self: [h(m, grad_outputs) for h in m._bwd_pre_hooks] and None)
            if self._bwd_post_hooks or reg.backward_hooks:

                def post(grad_inputs, grad_outputs, m=self, reg=reg):
                    for h in m._bwd_post_hooks:
                        h(m, grad_inputs, grad_outputs)
                    if reg.backward_hooks:
                        reg.CallModuleFullBackwardHooks(m, grad_outputs, grad_inputs)

                fn.register_hook(post)

    def RegisterForwardPreHook(self, hook: Callable) -> HookHandle:
        self._fwd_pre_hooks.append(hook)
        return HookHandle(self._fwd_pre_hooks, hook)

    def RegisterForwardPostHook(self, hook: Callable) -> HookHandle:
        self._fwd_post_hooks.append(hook)
        return HookHandle(self._fwd_post_hooks, hook)

    def RegisterBackwardPreHook(self, hook: Callable) -> HookHandle:
        self._bwd_pre_hooks.append(hook)
        return HookHandle(self._bwd_pre_hooks, hook)

    def RegisterBackwardPostHook(self, hook: Callable) -> HookHandle:
        self._bwd_post_hooks.append(hook)
        return HookHandle(self._bwd_post_hooks, hook)

    # ------------------------------------------------------------------ training entry (pipeline)
    def TrainStep(self, inputs, targets, optimizer, loss_fn, dtype) -> float:
        return 0.0

    # ------------------------------------------------------------------ device / dtype
    def To(self, target) -> "Module":
        """``To(device)`` or ``To(dtype)``; parameters are moved in place (tying is preserved)."""
        from ..device import Device
        from ..datatype import DataType, to_torch_dtype

        if isinstance(target, Device):
            self.to(target.torch_device())
        elif isinstance(target, DataType):
            self.to(to_torch_dtype(target))
        else:
            self.to(target)
        return self

    def Apply(self, fn: Callable[["Module"], None]) -> None:
        """Children first, then ``self`` (reference: module.cc Apply)."""
        for child in self._modules.values():
            if child is None:
                continue
            if isinstance(child, Module):
                child.Apply(fn)
            else:
                child.apply(fn)
        fn(self)

    def ReplicateForDataParallel(self, device_idx: int) -> "Module":
        import copy

        rep = copy.deepcopy(self)
        rep.to(torch.device("cuda", device_idx) if torch.cuda.is_available() else torch.device("cpu"))
        return rep


class CloneableModule(Module):
    """Kept for API parity: every Module here is already replicable."""
