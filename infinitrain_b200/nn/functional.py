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


# --------------------------------------------------------------------------- the rest of the reference's op catalogue
# (infini_train/include/autograd/{elementwise,transform,gather,scatter,outer,matmul}.h): thin names over
# PyTorch ops with the reference's conventions.
def Neg(x):
    return torch.neg(x)


def Exp(x):
    return torch.exp(x)


def Log(x):
    return torch.log(x)


def Matmul(a, b):
    return torch.matmul(a, b)


def Outer(a, b):
    return torch.outer(a, b)


def Transpose(x, dim0: int, dim1: int):
    return x.transpose(dim0, dim1).contiguous()          # the reference materialises the copy


def _as_input_dtype(mask, x):
    return mask.to(x.dtype)


def Equals(a, b):
    """Comparisons give 0 / 1 in the INPUT dtype, not bool (reference: src/kernels/cpu/elementwise.cc)."""
    return _as_input_dtype(a == b, a)


def Lt(a, b):
    return _as_input_dtype(a < b, a)


def Le(a, b):
    return _as_input_dtype(a <= b, a)


def Gt(a, b):
    return _as_input_dtype(a > b, a)


def Ge(a, b):
    return _as_input_dtype(a >= b, a)


def And(a, b):
    return _as_input_dtype((a != 0) & (b != 0), a)


def Or(a, b):
    return _as_input_dtype((a != 0) | (b != 0), a)


def Mask(x, mask, value: float):
    """masked_fill with a mask that may cover only the trailing (or leading) dimensions of ``x``."""
    m = mask.to(torch.bool)
    if m.dim() < x.dim() and tuple(x.shape[:m.dim()]) == tuple(m.shape) and tuple(x.shape[-m.dim():]) != tuple(m.shape):
        m = m.reshape(*m.shape, *([1] * (x.dim() - m.dim())))          # lead-aligned
    return x.masked_fill(m, value)


def Gather(x, dim: int, index):
    return torch.gather(x, dim, index)


def Scatter(values, indices, out_dims: Sequence[int]):
    """Top-k scatter (reference: src/kernels/cpu/scatter.cc:13-47): ``values`` and ``indices`` are
    ``[..., k]``; row r of the zero-filled output ``[..., n]`` gets ``values[r, j]`` at column
    ``indices[r, j]``.  The gradient gathers the same positions back."""
    out = torch.zeros(tuple(out_dims), dtype=values.dtype, device=values.device)
    return out.scatter(-1, indices, values)
