"""Functional wrappers (reference: infini_train/include/nn/functional.h:25-184)."""
from __future__ import annotations

from typing import Sequence

import torch

from ..ops import functional as ops


def Tril(x, diagonal=0):
    return torch.tril(x, diagonal)


def Triu(x, diagonal=0):
    return torch.triu(x, diagonal)


def Ones(shape, dtype=torch.float32, device=None):
    return torch.ones(tuple(shape), dtype=dtype, device=device)


def Reciprocal(x):
    return torch.reciprocal(x)


def Sin(x):
    return torch.sin(x)


def Cos(x):
    return torch.cos(x)


def Tanh(x):
    return torch.tanh(x)


def Pow(a, b):
    """``Pow(tensor, exponent)`` or ``Pow(base_scalar, tensor)``."""
    return torch.pow(a, b)


def Rsqrt(x):
    return torch.rsqrt(x)


def Mean(x, dim, keep_dim=False):
    return x.mean(dim, keepdim=keep_dim)


def Sum(x, dim, keep_dim=False):
    return x.sum(dim, keepdim=keep_dim)


def Min(x, dim, keep_dim=False):
    return x.min(dim, keepdim=keep_dim).values


def Max(x, dim, keep_dim=False):
    return x.max(dim, keepdim=keep_dim).values


def Sigmoid(x):
    return torch.sigmoid(x)


def Softmax(x, dim=-1):
    return torch.softmax(x.float(), dim).to(x.dtype)


def Slice(x, starts: Sequence[int], ends: Sequence[int], steps: Sequence[int]):
    idx = tuple(slice(s, e, st) for s, e, st in zip(starts, ends, steps))
    return x[idx]


def Stack(tensors, dim=0):
    return torch.stack(list(tensors), dim)


def Concat(tensors, dim=0):
    return torch.cat(list(tensors), dim)


def Linear(x, weight, bias=None):
    return ops.linear(x, weight, bias)


def LayerNorm(x, weight, bias=None, eps=1e-5):
    return ops.layernorm(x, weight, bias, eps)


def RMSNorm(x, weight, eps=1e-6):
    return ops.rmsnorm(x, weight, eps)


def NewGELU(x):
    return ops.gelu(x)


def SwiGLU(a, b):
    return ops.swiglu(a, b)


def CrossEntropy(logits, target):
    return ops.cross_entropy(logits, target)
