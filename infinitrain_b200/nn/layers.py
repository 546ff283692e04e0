"""Basic layers and containers.

Reference: infini_train/src/nn/modules/{linear,sparse,normalization,activations,loss,container}.cc.
Initialisation follows the reference (Linear: Kaiming-uniform with a = sqrt(5) for the weight and
U(-1/sqrt(fan_in), 1/sqrt(fan_in)) for the bias; Embedding: N(0, 1); norms: ones / zeros).
"""
from __future__ import annotations

import math
from collections import OrderedDict
from typing import Iterable, Optional

import torch

from ..ops import functional as ops
from . import init
from .module import Module


class Linear(Module):
    kType = "Linear"
    kParamWeightName = "weight"
    kParamBiasName = "bias"

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None):
        super().__init__(self.kType)
        self.in_features, self.out_features = in_features, out_features
        self.weight = torch.nn.Parameter(torch.empty(out_features, in_features, device=device))
        self.bias = torch.nn.Parameter(torch.empty(out_features, device=device)) if bias else None
        self.ResetParameters()

    def ResetParameters(self):
        init.KaimingUniform(self.weight, a=math.sqrt(5.0))
        if self.bias is not None:
            bound = 1.0 / math.sqrt(self.in_features) if self.in_features > 0 else 0.0
            init.Uniform(self.bias, -bound, bound)

    def Forward(self, x):
        return ops.linear(x, self.weight, self.bias)


class Embedding(Module):
    kType = "Embedding"
    kParamWeightName = "weight"

    def __init__(self, num_embeddings: int, embedding_dim: int, device=None):
        super().__init__(self.kType)
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = torch.nn.Parameter(torch.empty(num_embeddings, embedding_dim, device=device))
        init.Normal(self.weight)

    def Forward(self, idx):
        if idx.dim() == 2:
            return ops.embedding(idx, self.weight)
        return torch.nn.functional.embedding(idx, self.weight)


class LayerNorm(Module):
    kType = "LayerNorm"

    def __init__(self, normalized_shape, eps: float = 1e-5, device=None):
        super().__init__(self.kType)
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(normalized_shape)
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(self.normalized_shape, device=device))
        self.bias = torch.nn.Parameter(torch.zeros(self.normalized_shape, device=device))

    def Forward(self, x, skip: bool = False):
        """``skip=True`` returns ``(y, x)``: hand the second output to the ``residual`` argument of the
        projection that closes the residual branch (see :func:`ops.functional.layernorm_skip`)."""
        if skip:
            return ops.layernorm_skip(x, self.weight, self.bias, self.eps)
        return ops.layernorm(x, self.weight, self.bias, self.eps)


class RMSNorm(Module):
    kType = "RMSNorm"

    def __init__(self, dim: int, eps: float = 1e-6, device=None):
        super().__init__(self.kType)
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(dim, device=device))

    def Forward(self, x, skip: bool = False):
        if skip:
            return ops.rmsnorm_skip(x, self.weight, self.eps)
        return ops.rmsnorm(x, self.weight, self.eps)


class Sigmoid(Module):
    kType = "Sigmoid"

    def __init__(self):
        super().__init__(self.kType)

    def Forward(self, x):
        return torch.sigmoid(x)


class NewGELU(Module):
    kType = "NewGELU"

    def __init__(self):
        super().__init__(self.kType)

    def Forward(self, x):
        return ops.gelu(x)


class SwiGLU(Module):
    """``x * sigmoid(x)`` — the reference's "SwiGLU" module is the SiLU part of the gate
    (infini_train/src/nn/modules/activations.cc:21-23)."""

    kType = "SwiGLU"

    def __init__(self):
        super().__init__(self.kType)

    def Forward(self, x):
        return x * torch.sigmoid(x)


class CrossEntropyLoss(Module):
    kType = "CrossEntropyLoss"

    def __init__(self):
        super().__init__(self.kType)

    def Forward(self, logits, target):
        return ops.cross_entropy(logits, target)


class Sequential(Module):
    kType = "Sequential"

    def __init__(self, *layers):
        super().__init__(self.kType)
        if len(layers) == 1 and isinstance(layers[0], (list, tuple)):
            layers = tuple(layers[0])
        for i, layer in enumerate(layers):
            self.add_module(str(i), layer)

    def __len__(self):
        return len(self._modules)

    def __iter__(self):
        return iter(self._modules.values())

    def __getitem__(self, i):
        return list(self._modules.values())[i]

    def Forward(self, *inputs):
        x = inputs
        for layer in self._modules.values():
            x = layer(*x) if isinstance(x, tuple) else layer(x)
        return x


class ModuleDict(Module):
    kType = "ModuleDict"

    def __init__(self, modules: Optional[dict] = None):
        super().__init__(self.kType)
        for k, v in (modules or {}).items():
            self.add_module(k, v)

    def __getitem__(self, k):
        return self._modules[k]

    def __setitem__(self, k, v):
        self.add_module(k, v)

    def __contains__(self, k):
        return k in self._modules

    def keys(self):
        return self._modules.keys()

    def items(self):
        return self._modules.items()

    def values(self):
        return self._modules.values()

    def __len__(self):
        return len(self._modules)


class ModuleList(Module):
    kType = "ModuleList"

    def __init__(self, modules: Optional[Iterable] = None):
        super().__init__(self.kType)
        for m in modules or []:
            self.append(m)

    def append(self, m):
        self.add_module(str(len(self._modules)), m)
        return self

    def __getitem__(self, i):
        if isinstance(i, slice):
            return list(self._modules.values())[i]
        return self._modules[str(i if i >= 0 else len(self._modules) + i)]

    def __iter__(self):
        return iter(self._modules.values())

    def __len__(self):
        return len(self._modules)
