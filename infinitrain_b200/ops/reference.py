"""Plain PyTorch fp32 implementations of every fused op.

They are the CPU path of the framework and the numerical oracle of the kernel tests; each restates
the math of the reference's CPU kernels (infini_train/src/kernels/cpu/*.cc) with autograd doing the
backward pass.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def linear(x, weight, bias=None, residual=None, gelu=False):
    y = F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))
    if gelu:
        y = new_gelu(y)
    if residual is not None:
        y = y + residual
    return y


def new_gelu(x):
    # tanh approximation (reference: infini_train/src/nn/modules/activations.cc:15-19)
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x.pow(3))))


def swiglu(a, b):
    # reference gate order: c_fc(x) * silu(c_fc2(x)) (infini_train/src/nn/modules/transformer/mlp.cc:84-90)
    return a * (b * torch.sigmoid(b))


def layernorm(x, gamma, beta, eps):
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = (xf - mean).pow(2).mean(-1, keepdim=True)
    y = (xf - mean) * torch.rsqrt(var + eps) * gamma
    if beta is not None:
        y = y + beta
    return y.to(x.dtype)


def rmsnorm(x, gamma, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma
    return y.to(x.dtype)


def precompute_freqs_cis(head_dim: int, end: int, theta: float = 10000.0, device=None):
    """[end, head_dim/2, 2] table of (cos, sin) (reference: infini_train/src/nn/modules/transformer/utils.cc:9-29)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    t = torch.arange(end, dtype=torch.float32, device=device)
    ang = torch.outer(t, inv)
    return torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous()


def apply_rope(x, freqs, pos0=0):
    """x [B, T, H, D] with interleaved (even, odd) pairs; freqs [T_max, D/2, 2]."""
    B, T, H, D = x.shape
    xf = x.float().reshape(B, T, H, D // 2, 2)
    c = freqs[pos0:pos0 + T, :, 0].view(1, T, 1, D // 2)
    s = freqs[pos0:pos0 + T, :, 1].view(1, T, 1, D // 2)
    out = torch.stack([xf[..., 0] * c - xf[..., 1] * s, xf[..., 0] * s + xf[..., 1] * c], dim=-1)
    return out.reshape(B, T, H, D).to(x.dtype)


def attention(q, k, v, causal=True, scale=None):
    """q [B,T,H,D], k/v [B,T,KV,D] -> [B,T,H,D]; softmax in fp32, GQA by head repetition."""
    B, T, H, D = q.shape
    KV = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf, kf, vf = q.float(), k.float(), v.float()
    if KV != H:
        kf = kf.repeat_interleave(H // KV, dim=2)
        vf = vf.repeat_interleave(H // KV, dim=2)
    s = torch.einsum("bthd,bshd->bhts", qf, kf) * scale
    if causal:
        mask = torch.ones(T, T, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = s.softmax(-1)
    return torch.einsum("bhts,bshd->bthd", p, vf).to(q.dtype)


def embedding(idx, wte, wpe=None, pos0=0, vocab_start=0):
    V = wte.shape[0]
    local = idx - vocab_start
    own = (local >= 0) & (local < V)
    out = wte[local.clamp(0, V - 1)] * own.unsqueeze(-1).to(wte.dtype)
    if wpe is not None:
        T = idx.shape[1]
        out = out + wpe[pos0:pos0 + T]
    return out


def cross_entropy(logits, target):
    """Mean over all rows (reference: infini_train/src/kernels/cpu/cross_entropy.cc:17-98)."""
    return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), target.reshape(-1))
