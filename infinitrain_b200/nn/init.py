"""Parameter initialisers (reference: infini_train/src/nn/init.cc).

The reference draws on the host from a global ``std::mt19937(42)`` (one generator per OpenMP thread,
so its streams depend on the thread count) and copies to the device.  Here one ``torch.Generator``
seeded with 42 on the host is the single stream, which makes initialisation independent of thread
count and of the target device; parity runs exchange weights through llm.c files instead.
"""
from __future__ import annotations

import math

import torch

_GEN = torch.Generator(device="cpu")
_GEN.manual_seed(42)


def manual_seed(seed: int) -> None:
    _GEN.manual_seed(seed)


def _fill(t: torch.Tensor, host: torch.Tensor) -> torch.Tensor:
    with torch.no_grad():
        t.copy_(host.to(t.dtype))
    return t


def Normal(t: torch.Tensor, mean: float = 0.0, std: float = 1.0, generator=None) -> torch.Tensor:
    host = torch.empty(t.shape, dtype=torch.float32, device="cpu").normal_(mean, std, generator=generator or _GEN)
    return _fill(t, host)


def Uniform(t: torch.Tensor, a: float = 0.0, b: float = 1.0, generator=None) -> torch.Tensor:
    host = torch.empty(t.shape, dtype=torch.float32, device="cpu").uniform_(a, b, generator=generator or _GEN)
    return _fill(t, host)


def _fan_in_out(t: torch.Tensor):
    if t.dim() < 2:
        raise ValueError("fan in/out need at least 2 dimensions")
    rf = 1
    for s in t.shape[2:]:
        rf *= s
    return t.shape[1] * rf, t.shape[0] * rf


def CalculateGain(nonlinearity: str = "leaky_relu", param: float = 0.0) -> float:
    if nonlinearity in ("linear", "sigmoid"):
        return 1.0
    if nonlinearity == "tanh":
        return 5.0 / 3.0
    if nonlinearity == "relu":
        return math.sqrt(2.0)
    if nonlinearity == "leaky_relu":
        return math.sqrt(2.0 / (1.0 + param * param))
    raise ValueError(nonlinearity)


def KaimingUniform(t: torch.Tensor, a: float = 0.0, mode: str = "fan_in", nonlinearity: str = "leaky_relu",
                   generator=None) -> torch.Tensor:
    fan_in, fan_out = _fan_in_out(t)
    fan = fan_in if mode == "fan_in" else fan_out
    bound = math.sqrt(3.0) * CalculateGain(nonlinearity, a) / math.sqrt(fan)
    return Uniform(t, -bound, bound, generator)


def Ones(t: torch.Tensor) -> torch.Tensor:
    with torch.no_grad():
        return t.fill_(1)


def Zeros(t: torch.Tensor) -> torch.Tensor:
    with torch.no_grad():
        return t.zero_()


def Arange(start: int, end: int, dtype=torch.int64, device=None) -> torch.Tensor:
    return torch.arange(start, end, dtype=dtype, device=device)
