"""Tensor helpers in the reference's API shape.

The framework's tensor IS ``torch.Tensor`` (storage, views, dtype promotion, autograd metadata);
this module adds the reference's constructor form and the few methods PyTorch names differently
(reference: infini_train/include/tensor.h:62-240, infini_train/src/tensor.cc:674-975).
"""
from __future__ import annotations

import struct
from typing import Optional, Sequence

import numpy as np
import torch

from .datatype import DataType, from_torch_dtype, to_torch_dtype
from .device import Device


def Tensor(dims: Sequence[int], dtype=DataType.kFLOAT32, device: Optional[Device] = None,
           requires_grad: bool = False) -> torch.Tensor:
    """Uninitialised tensor of shape ``dims`` (``Tensor(dims, dtype, device, requires_grad)``)."""
    dev = device.torch_device() if isinstance(device, Device) else (device or "cpu")
    return torch.empty(tuple(dims), dtype=to_torch_dtype(dtype), device=dev, requires_grad=requires_grad)


def Dims(t: torch.Tensor):
    return list(t.shape)


def NumElements(t: torch.Tensor) -> int:
    return t.numel()


def SizeInBytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def Dtype(t: torch.Tensor) -> DataType:
    return from_torch_dtype(t.dtype)


def GetDevice(t: torch.Tensor) -> Device:
    return Device.from_torch(t.device)


def To(t: torch.Tensor, target) -> torch.Tensor:
    if isinstance(target, Device):
        return t.to(target.torch_device())
    if isinstance(target, DataType):
        return t.to(to_torch_dtype(target))
    return t.to(target)


def Fill(t: torch.Tensor, value) -> torch.Tensor:
    with torch.no_grad():
        return t.fill_(getattr(value, "value", value))


def MaskedFill(t: torch.Tensor, mask: torch.Tensor, value) -> torch.Tensor:
    return t.masked_fill(mask.bool(), value)


def RepeatInterleave(t: torch.Tensor, repeats: int, dim: int) -> torch.Tensor:
    return t.repeat_interleave(repeats, dim)


def Slice(t: torch.Tensor, dim: int, start: int, end: int, step: int = 1) -> torch.Tensor:
    idx = [slice(None)] * t.dim()
    idx[dim] = slice(start, end, step)
    return t[tuple(idx)]


def Split(t: torch.Tensor, split_size: int, dim: int = 0):
    return list(t.split(split_size, dim))


def Outer(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return torch.outer(a, b)


def SaveAsNpy(t: torch.Tensor, path: str) -> None:
    """NumPy ``.npy`` v1.0 file of the tensor converted to fp32 (what the reference writes)."""
    np.save(path if path.endswith(".npy") else path + ".npy", t.detach().float().cpu().numpy())


def Print(t: torch.Tensor, file=None) -> None:
    """torch-style text of the tensor (the reference prints in that style too, src/tensor.cc:784-975); the
    options of :func:`SetPrintOptions` apply."""
    print(t, file=file)


def SetPrintOptions(precision: Optional[int] = None, threshold: Optional[int] = None, edge_items: Optional[int] = None,
                    linewidth: Optional[int] = None, profile: Optional[str] = None, sci_mode: Optional[bool] = None) -> None:
    """``Tensor::SetPrintOptions`` (include/tensor.h:195-198): digits after the point, the element count
    above which a tensor is summarised, how many items each end of a summarised dimension keeps, the line
    width, a named profile (``default`` / ``short`` / ``full``) applied before the other arguments, and
    scientific notation on, off or chosen by the values (``None``)."""
    if profile is not None:
        torch.set_printoptions(profile=profile)
    kw = {k: v for k, v in (("precision", precision), ("threshold", threshold), ("edgeitems", edge_items),
                            ("linewidth", linewidth)) if v is not None}
    if kw or sci_mode is not None:
        torch.set_printoptions(sci_mode=sci_mode, **kw)


def RegisterPostAccumulateGradHook(t: torch.Tensor, hook):
    from .common.hook import TorchHookHandle

    return TorchHookHandle(t.register_post_accumulate_grad_hook(hook))
