"""Fused ops behind ``torch.autograd.Function``: the CUDA path launches the hand-written sm_100a
kernels of ``infinitrain_b200._C``; the CPU path (and any dtype the kernels do not cover) runs the
PyTorch implementations of :mod:`infinitrain_b200.ops.reference`.

Mixed precision follows the reference's autocast policy at module granularity
(infini_train/include/autocast.h:36-71): Linear/Matmul run in bf16 with fp32 accumulation and emit
bf16, normalisation and softmax statistics are fp32, weight gradients are fp32.  The casts are not
materialised: weights have a bf16 shadow that the fused optimizer refreshes, and activations stay
bf16 between the fused kernels.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _ext
from . import reference as ref

_counters = {"launches": 0}


def launch_count() -> int:
    """Number of native kernel launches issued through this module (for benchmarks)."""
    return _counters["launches"]


def _C():
    mod = _ext.load()
    if mod is None:
        raise RuntimeError("infinitrain_b200 native extension is not available")
    return mod


# --------------------------------------------------------------------------- autocast state
class _AutocastState:
    enabled = False
    dtype = torch.bfloat16


def autocast_enabled() -> bool:
    return _AutocastState.enabled


def autocast_dtype() -> torch.dtype:
    return _AutocastState.dtype


def _use_fused(x: torch.Tensor) -> bool:
    """Fused kernels run on CUDA when the activation is bf16 or bf16 autocast is on."""
    return x.is_cuda and (x.dtype == torch.bfloat16 or (_AutocastState.enabled and _AutocastState.dtype == torch.bfloat16))


# --------------------------------------------------------------------------- bf16 weight shadows
def weight_lp(weight: torch.Tensor) -> torch.Tensor:
    """bf16 copy of an fp32 weight, cached on the tensor.

    The fused optimizers write the shadow in the same kernel as the fp32 update and stamp it with
    the weight's version; any other in-place change bumps the version and triggers a re-cast.
    """
    if weight.dtype == torch.bfloat16:
        return weight.detach()
    sh = getattr(weight, "_itb_shadow", None)
    ver = weight._version
    if sh is not None and getattr(weight, "_itb_shadow_version", -1) == ver and sh.device == weight.device:
        return sh
    if sh is None or sh.shape != weight.shape or sh.device != weight.device:
        sh = torch.empty_like(weight, dtype=torch.bfloat16)
    if weight.is_cuda and weight.is_contiguous():
        _C().cast_into(weight.detach(), sh)
        _counters["launches"] += 1
    else:
        sh.copy_(weight.detach())
    weight._itb_shadow = sh
    weight._itb_shadow_version = ver
    return sh


def mark_shadow_fresh(weight: torch.Tensor) -> None:
    """Called by fused optimizers after they wrote ``weight._itb_shadow`` themselves."""
    weight._itb_shadow_version = weight._version


def _pad_cols(n: int) -> int:
    return (n + 63) // 64 * 64


def _as_bf16_2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.dtype != torch.bfloat16:
        x2 = x2.to(torch.bfloat16)
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) or (x2.data_ptr() % 16):
        x2 = x2.contiguous()
    return x2


# --------------------------------------------------------------------------- linear
class _LinearFn(torch.autograd.Function):
    """y = x W^T (+ bias) (+ residual), optionally y = gelu(x W^T + bias).

    Forward, dgrad and wgrad are three launches of the tcgen05 GEMM; bias / residual / GELU live in
    its epilogue, the weight gradient is accumulated in fp32 with split-K atomics, the bias
    gradient is a two-stage column sum.
    """

    @staticmethod
    def forward(ctx, x, weight, bias, residual, gelu):
        C = _C()
        K = x.shape[-1]
        N = weight.shape[0]
        x2 = _as_bf16_2d(x)
        M = x2.shape[0]
        w = weight_lp(weight)
        out_f32 = residual is not None and residual.dtype == torch.float32
        ld = _pad_cols(N)
        out = torch.empty((M, ld), device=x.device, dtype=torch.float32 if out_f32 else torch.bfloat16)
        flags = 0
        if out_f32:
            flags |= C.GEMM_OUT_F32
        if bias is not None:
            flags |= C.GEMM_BIAS
        res2 = None
        if residual is not None:
            res2 = residual.reshape(M, N)
            if res2.stride(-1) != 1:
                res2 = res2.contiguous()
            flags |= C.GEMM_RESIDUAL
        pre = None
        if gelu:
            assert residual is None, "gelu and residual epilogues are not combined"
            pre = torch.empty((M, ld), device=x.device, dtype=torch.bfloat16)
            flags |= C.GEMM_GELU_DUAL
            C.gemm(x2, False, w, False, M, N, K, pre, out, bias, None, None, flags, 0)
        else:
            C.gemm(x2, False, w, False, M, N, K, out, None, bias, res2, None, flags, 0)
        _counters["launches"] += 1
        ctx.save_for_backward(x2, weight, pre if gelu else None)
        ctx.bias_param = bias            # the Parameter itself: its gradient may go straight to a flat buffer
        ctx.bias_elsewhere = claim_bias_grad(residual, bias)
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.gelu = gelu
        ctx.x_shape = x.shape
        ctx.x_dtype = x.dtype
        ctx.res_dtype = residual.dtype if residual is not None else None
        ctx.N, ctx.K, ctx.M, ctx.ld = N, K, M, ld
        y = out[:, :N] if ld != N else out
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        C = _C()
        x2, weight, pre = ctx.saved_tensors
        M, N, K = ctx.M, ctx.N, ctx.K
        d_res = dy if ctx.has_res else None
        if d_res is not None and d_res.dtype != ctx.res_dtype:
            d_res = d_res.to(ctx.res_dtype)
        dy2 = dy.reshape(M, N)
        if dy2.dtype != torch.bfloat16:
            dy2 = dy2.to(torch.bfloat16)
        if dy2.stride(-1) != 1 or (dy2.stride(0) % 8) or (dy2.data_ptr() % 16):
            dy2 = dy2.contiguous()
        if ctx.gelu:
            # dy is the gradient of the activation output: fold gelu'(h) in with one pointwise pass.
            dyc = dy2 if dy2.is_contiguous() else dy2.contiguous()
            prec = pre[:, :N] if ctx.ld != N else pre
            prec = prec if prec.is_contiguous() else prec.contiguous()
            dy2 = C.gelu_bwd(dyc, prec)
            _counters["launches"] += 1
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            w = weight_lp(weight)
            dx2 = torch.empty((M, K), device=dy.device, dtype=torch.bfloat16)
            C.gemm(dy2, False, w, True, M, K, N, dx2, None, None, None, None, 0, 0)
            _counters["launches"] += 1
            dx = dx2.view(ctx.x_shape)
            if ctx.x_dtype != torch.bfloat16:
                dx = dx.to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = _wgrad(C, dy2, x2, weight, N, K, M)
        if ctx.has_bias and ctx.needs_input_grad[2] and not ctx.bias_elsewhere:
            db = _bias_grad(C, dy2, N, ctx.bias_param)
        return dx, dw, db, d_res, None


def _wgrad(C, dy2, x2, weight, N, K, M):
    """dW[N,K] = dy^T x in fp32.  Accumulates straight into ``weight.main_grad`` when the parameter
    has one (flat DDP / ZeRO gradient buffers) and then fires its grad-ready hooks."""
    main = getattr(weight, "main_grad", None)
    if main is None and getattr(weight, "_itb_main_grad_fn", None) is not None:
        main = weight._itb_main_grad_fn()
    if getattr(weight, "_itb_shared", False):
        # A parameter used by several ops (tied embedding / head) receives the rest of its gradient
        # through autograd; its ready hook must fire once, after the last contribution.
        main = None
    if main is not None:
        C.gemm(dy2, True, x2, True, N, K, M, main, None, None, None, None, C.GEMM_OUT_F32 | C.GEMM_ATOMIC, 0)
        _counters["launches"] += 1
        for hook in getattr(weight, "_itb_grad_ready_hooks", ()):
            hook(weight)
        return None
    dw = torch.zeros((N, K), device=dy2.device, dtype=torch.float32)
    C.gemm(dy2, True, x2, True, N, K, M, dw, None, None, None, None, C.GEMM_OUT_F32 | C.GEMM_ATOMIC, 0)
    _counters["launches"] += 2
    return dw if weight.dtype == torch.float32 else dw.to(weight.dtype)


def _main_grad_of(p: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """The fp32 slot of ``p`` in a flat gradient buffer that a kernel may accumulate into directly, or
    None (no flat buffer, or a parameter shared by several ops whose ready hook must fire once)."""
    if p is None or getattr(p, "_itb_shared", False):
        return None
    if getattr(p, "_itb_sp_hooked", False) or getattr(p, "_backward_hooks", None):
        return None      # a tensor hook must see this gradient (e.g. the sum over the tensor-parallel group)
    main = getattr(p, "main_grad", None)
    if main is None and getattr(p, "_itb_main_grad_fn", None) is not None:
        main = p._itb_main_grad_fn()
    if main is None or main.dtype != torch.float32 or not main.is_contiguous():
        return None
    return main


def autograd_ready_hook(fn):
    """Wraps a grad-ready callback for ``register_post_accumulate_grad_hook``: the call autograd makes
    for a parameter whose gradient another op will write later in this backward pass (see
    ``claim_bias_grad``) is dropped; that op reports the parameter through ``_itb_grad_ready_hooks``."""
    def hook(p):
        if getattr(p, "_itb_grad_elsewhere", False):
            return None
        return fn(p)
    return hook


def _grad_written(p: torch.Tensor) -> None:
    """A kernel has added ``p``'s gradient to its flat-buffer slot: tell the reducer / ZeRO group."""
    if getattr(p, "_itb_grad_elsewhere", False):
        p._itb_grad_elsewhere = False
    for hook in getattr(p, "_itb_grad_ready_hooks", ()):
        hook(p)


def _bias_grad(C, dy2, N, bias=None):
    """Column sums of dY.  With a flat gradient buffer behind ``bias`` they are added straight into
    its slot (no gradient tensor, no separate accumulation launch) and None is returned."""
    if N % 8 == 0 and dy2.data_ptr() % 16 == 0:
        _counters["launches"] += 2
        main = _main_grad_of(bias)
        if main is not None:
            C.colsum(dy2, main)
            _grad_written(bias)
            return None
        return C.colsum(dy2)
    return dy2.float().sum(0)


def linear(x, weight, bias=None, residual=None, gelu=False):
    """``x @ weight.T + bias`` with optional fused residual add or tanh-GELU."""
    K = x.shape[-1]
    if _use_fused(x) and K % 8 == 0 and weight.is_cuda:
        return _LinearFn.apply(x, weight, bias, residual, gelu)
    if _AutocastState.enabled and x.dtype == torch.float32 and not x.is_cuda:
        # CPU emulation of the bf16 autocast of Linear: bf16-rounded operands, fp32 accumulate.
        y = ref.linear(x.to(_AutocastState.dtype).float(), weight.to(_AutocastState.dtype).float(), bias, None, gelu)
        return y if residual is None else y + residual
    return ref.linear(x, weight, bias, residual, gelu)


# --------------------------------------------------------------------------- fused GELU MLP
class _MlpGeluFn(torch.autograd.Function):
    """out = residual + gelu(x Wfc^T + bfc) Wproj^T + bproj as four GEMM launches forward+backward
    activations: the GELU is stored by the first GEMM's epilogue and its derivative is applied in the
    epilogue of the dgrad GEMM of the projection (reference composition:
    infini_train/src/nn/modules/transformer/mlp.cc:70-79)."""

    @staticmethod
    def forward(ctx, x, w_fc, b_fc, w_proj, b_proj, residual):
        C = _C()
        Cd = x.shape[-1]
        F = w_fc.shape[0]
        x2 = _as_bf16_2d(x)
        M = x2.shape[0]
        wfc, wpr = weight_lp(w_fc), weight_lp(w_proj)
        h = torch.empty((M, F), device=x.device, dtype=torch.bfloat16)
        g = torch.empty((M, F), device=x.device, dtype=torch.bfloat16)
        flags = C.GEMM_GELU_DUAL | (C.GEMM_BIAS if b_fc is not None else 0)
        C.gemm(x2, False, wfc, False, M, F, Cd, h, g, b_fc, None, None, flags, 0)
        out_f32 = residual is not None and residual.dtype == torch.float32
        out = torch.empty((M, Cd), device=x.device, dtype=torch.float32 if out_f32 else torch.bfloat16)
        flags = (C.GEMM_OUT_F32 if out_f32 else 0) | (C.GEMM_BIAS if b_proj is not None else 0)
        res2 = None
        if residual is not None:
            res2 = residual.reshape(M, Cd)
            res2 = res2 if res2.stride(-1) == 1 else res2.contiguous()
            flags |= C.GEMM_RESIDUAL
        C.gemm(g, False, wpr, False, M, Cd, F, out, None, b_proj, res2, None, flags, 0)
        _counters["launches"] += 2
        ctx.save_for_backward(x2, h, g, w_fc, w_proj)
        ctx.bias_params = (b_fc, b_proj)
        ctx.bias_elsewhere = claim_bias_grad(residual, b_proj)
        ctx.meta = (M, Cd, F, x.shape, x.dtype, b_fc is not None, b_proj is not None,
                    residual.dtype if residual is not None else None)
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        C = _C()
        x2, h, g, w_fc, w_proj = ctx.saved_tensors
        M, Cd, F, x_shape, x_dtype, has_bfc, has_bpr, res_dtype = ctx.meta
        d_res = None
        if res_dtype is not None:
            d_res = dy if dy.dtype == res_dtype else dy.to(res_dtype)
        dy2 = _as_bf16_2d(dy)
        # dh = (dy Wproj) * gelu'(h): derivative applied in the GEMM epilogue.
        dh = torch.empty((M, F), device=dy.device, dtype=torch.bfloat16)
        C.gemm(dy2, False, weight_lp(w_proj), True, M, F, Cd, dh, None, None, None, h, C.GEMM_DGELU, 0)
        _counters["launches"] += 1
        dw_proj = _wgrad(C, dy2, g, w_proj, Cd, F, M) if ctx.needs_input_grad[3] else None
        b_fc, b_proj = ctx.bias_params
        db_proj = None
        if has_bpr and ctx.needs_input_grad[4] and not ctx.bias_elsewhere:
            db_proj = _bias_grad(C, dy2, Cd, b_proj)
        dx = None
        if ctx.needs_input_grad[0]:
            dx2 = torch.empty((M, Cd), device=dy.device, dtype=torch.bfloat16)
            C.gemm(dh, False, weight_lp(w_fc), True, M, Cd, F, dx2, None, None, None, None, 0, 0)
            _counters["launches"] += 1
            dx = dx2.view(x_shape)
            if x_dtype != torch.bfloat16:
                dx = dx.to(x_dtype)
        dw_fc = _wgrad(C, dh, x2, w_fc, F, Cd, M) if ctx.needs_input_grad[1] else None
        db_fc = _bias_grad(C, dh, F, b_fc) if has_bfc and ctx.needs_input_grad[2] else None
        return dx, dw_fc, db_fc, dw_proj, db_proj, d_res


def mlp_gelu(x, w_fc, b_fc, w_proj, b_proj, residual=None):
    if _use_fused(x) and x.shape[-1] % 8 == 0 and w_fc.shape[0] % 8 == 0:
        return _MlpGeluFn.apply(x, w_fc, b_fc, w_proj, b_proj, residual)
    hmid = linear(x, w_fc, b_fc, gelu=True)
    return linear(hmid, w_proj, b_proj, residual=residual)


# --------------------------------------------------------------------------- normalisation
class _SkipHolder:
    """Travels on the skip tensor of a residual norm to the projection that adds it back in: that
    projection's bias gradient is the column sum of the skip's gradient, which the norm's backward
    kernel reads anyway."""

    __slots__ = ("bias",)

    def __init__(self):
        self.bias = None


def claim_bias_grad(residual, bias) -> bool:
    """Called by a linear whose epilogue adds ``residual``: True when the norm that produced
    ``residual`` as its skip output will compute ``bias``'s gradient (straight into the flat
    gradient buffer) in its own backward pass, so the linear must not."""
    holder = getattr(residual, "_itb_skip_holder", None)
    if holder is None or bias is None or holder.bias is not None or _main_grad_of(bias) is None:
        return False
    holder.bias = bias
    # Until that norm's backward has run, nothing may report this parameter's gradient as complete:
    # autograd still visits its accumulator (with an undefined gradient, because the linear returns
    # none) and fires the parameter's post-accumulate hook there, long before the norm writes the slot.
    bias._itb_grad_elsewhere = True
    return True


def _norm_param_grads(params, outs):
    """Gradient tensors for autograd, or None for parameters whose gradient the kernel has already
    added to their flat-buffer slot."""
    res = []
    for p, slot, g in zip(params, outs[0], outs[1]):
        if p is None:
            res.append(None)
        elif slot is not None:
            _grad_written(p)
            res.append(None)
        else:
            res.append(g)
    return res


class _LayerNormFn(torch.autograd.Function):
    """LayerNorm; with ``skip=True`` also returns the input as a second output, so that the residual
    connection around the normalised branch starts HERE: backward then receives the branch's
    gradient and the skip's gradient together and one kernel computes norm'(dy) + dskip (and the
    column sums of dskip for the bias of the projection that adds the skip back in)."""

    @staticmethod
    def forward(ctx, x, gamma, beta, eps, out_dtype, holder=None):
        C = _C()
        xc = x if x.is_contiguous() else x.contiguous()
        y, mean, rstd = C.layernorm_fwd(xc, gamma, beta, eps, out_dtype)
        _counters["launches"] += 1
        ctx.save_for_backward(xc, mean, rstd)
        ctx.params = (gamma, beta)
        ctx.holder = holder
        if holder is None:
            return y
        return y, xc.view_as(xc)

    @staticmethod
    def backward(ctx, dy, dskip=None):
        C = _C()
        x, mean, rstd = ctx.saved_tensors
        gamma, beta = ctx.params
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        if dyc.dtype == torch.float32 and x.dtype == torch.bfloat16:
            dyc = dyc.to(torch.bfloat16)
        if dskip is not None:
            dskip = dskip if dskip.dtype == x.dtype else dskip.to(x.dtype)
            dskip = dskip if dskip.is_contiguous() else dskip.contiguous()
        bias = ctx.holder.bias if (ctx.holder is not None and dskip is not None) else None
        slots = (_main_grad_of(gamma), _main_grad_of(beta), _main_grad_of(bias))
        dx, dg, db, _ = C.layernorm_bwd(dyc, x, gamma, mean, rstd, beta is not None, dskip, slots[0],
                                        slots[1] if beta is not None else None, slots[2], False)
        _counters["launches"] += 2
        if bias is not None:
            _grad_written(bias)
        dgamma, dbeta = _norm_param_grads((gamma, beta), (slots, (dg, db)))
        return dx, dgamma, dbeta, None, None, None


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, eps, out_dtype, holder=None):
        C = _C()
        xc = x if x.is_contiguous() else x.contiguous()
        y, rstd = C.rmsnorm_fwd(xc, gamma, eps, out_dtype)
        _counters["launches"] += 1
        ctx.save_for_backward(xc, rstd)
        ctx.params = (gamma,)
        ctx.holder = holder
        if holder is None:
            return y
        return y, xc.view_as(xc)

    @staticmethod
    def backward(ctx, dy, dskip=None):
        C = _C()
        x, rstd = ctx.saved_tensors
        (gamma,) = ctx.params
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        if dyc.dtype == torch.float32 and x.dtype == torch.bfloat16:
            dyc = dyc.to(torch.bfloat16)
        if dskip is not None:
            dskip = dskip if dskip.dtype == x.dtype else dskip.to(x.dtype)
            dskip = dskip if dskip.is_contiguous() else dskip.contiguous()
        bias = ctx.holder.bias if (ctx.holder is not None and dskip is not None) else None
        slots = (_main_grad_of(gamma), _main_grad_of(bias))
        dx, dg, _ = C.rmsnorm_bwd(dyc, x, gamma, rstd, dskip, slots[0], slots[1], False)
        _counters["launches"] += 2
        if bias is not None:
            _grad_written(bias)
        (dgamma,) = _norm_param_grads((gamma,), ((slots[0],), (dg,)))
        return dx, dgamma, None, None, None


def _norm_out_dtype(x):
    if x.dtype == torch.bfloat16 or (_AutocastState.enabled and _AutocastState.dtype == torch.bfloat16):
        return torch.bfloat16
    return torch.float32


def _norm_fused(x, gamma) -> bool:
    C_ = x.shape[-1]
    return (x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and gamma.dtype == torch.float32 and C_ % 8 == 0
            and C_ <= 6144 and _ext.available())


def layernorm(x, gamma, beta=None, eps=1e-5):
    if _norm_fused(x, gamma):
        return _LayerNormFn.apply(x, gamma, beta, eps, _norm_out_dtype(x))
    return ref.layernorm(x, gamma, beta, eps)


def rmsnorm(x, gamma, eps=1e-6):
    if _norm_fused(x, gamma):
        return _RMSNormFn.apply(x, gamma, eps, _norm_out_dtype(x))
    return ref.rmsnorm(x, gamma, eps)


def layernorm_skip(x, gamma, beta=None, eps=1e-5):
    """``(layernorm(x), x)``: the second output is the start of the residual connection around the
    normalised branch.  Adding it back in through a fused linear's ``residual`` argument lets the
    backward pass add the skip's gradient inside the norm's backward kernel (no separate add) and
    take that linear's bias gradient from the same pass."""
    if _norm_fused(x, gamma):
        holder = _SkipHolder()
        y, xs = _LayerNormFn.apply(x, gamma, beta, eps, _norm_out_dtype(x), holder)
        xs._itb_skip_holder = holder
        return y, xs
    return ref.layernorm(x, gamma, beta, eps), x


def rmsnorm_skip(x, gamma, eps=1e-6):
    """``(rmsnorm(x), x)``; see :func:`layernorm_skip`."""
    if _norm_fused(x, gamma):
        holder = _SkipHolder()
        y, xs = _RMSNormFn.apply(x, gamma, eps, _norm_out_dtype(x), holder)
        xs._itb_skip_holder = holder
        return y, xs
    return ref.rmsnorm(x, gamma, eps), x


# --------------------------------------------------------------------------- activations
class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x if x.is_contiguous() else x.contiguous()
        ctx.save_for_backward(xc)
        _counters["launches"] += 1
        return _C().gelu_fwd(xc)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dyc = dy.to(x.dtype)
        dyc = dyc if dyc.is_contiguous() else dyc.contiguous()
        _counters["launches"] += 1
        return _C().gelu_bwd(dyc, x)


def gelu(x):
    if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and _ext.available():
        return _GeluFn.apply(x)
    return ref.new_gelu(x)


class _SwiGLUFn(torch.autograd.Function):
    """out = a * silu(b) for a, b the two column halves of one [rows, 2F] matrix."""

    @staticmethod
    def forward(ctx, ab):
        C = _C()
        F = ab.shape[-1] // 2
        ab2 = ab.reshape(-1, 2 * F)
        ab2 = ab2 if ab2.stride(-1) == 1 else ab2.contiguous()
        out = C.swiglu_fwd(ab2[:, :F], ab2[:, F:])
        _counters["launches"] += 1
        ctx.save_for_backward(ab2)
        ctx.shape = ab.shape
        return out.view(*ab.shape[:-1], F)

    @staticmethod
    def backward(ctx, dout):
        C = _C()
        (ab2,) = ctx.saved_tensors
        F = ab2.shape[-1] // 2
        d2 = dout.reshape(-1, F).to(ab2.dtype)
        d2 = d2 if d2.stride(-1) == 1 else d2.contiguous()
        dab = C.swiglu_bwd(d2, ab2[:, :F], ab2[:, F:])
        _counters["launches"] += 1
        return dab.view(ctx.shape)


def swiglu_packed(ab):
    """``ab[..., :F] * silu(ab[..., F:])`` for a packed [..., 2F] tensor."""
    F = ab.shape[-1] // 2
    if ab.is_cuda and ab.dtype in (torch.float32, torch.bfloat16) and F % 8 == 0 and _ext.available():
        return _SwiGLUFn.apply(ab)
    return ref.swiglu(ab[..., :F], ab[..., F:])


def swiglu(a, b):
    if a.is_cuda and a.dtype in (torch.float32, torch.bfloat16) and a.shape[-1] % 8 == 0 and _ext.available():
        return _SwiGLUFn.apply(torch.cat([a, b], dim=-1))
    return ref.swiglu(a, b)


# --------------------------------------------------------------------------- attention
class _AttentionFn(torch.autograd.Function):
    """Causal flash attention over a packed [B, T, (H + 2 KV) D] bf16 projection, with RoPE applied
    in place to the q and k heads first (and un-applied on their gradients)."""

    @staticmethod
    def forward(ctx, qkv, H, KV, D, freqs, pos0, causal):
        C = _C()
        B, T, _ = qkv.shape
        if qkv.dtype != torch.bfloat16:
            qkv = qkv.to(torch.bfloat16)
        if freqs is not None:
            qkv = qkv.clone() if not qkv.is_contiguous() else qkv
            C.rope_inplace(qkv, freqs, B, T, H + KV, D, qkv.stride(1), pos0, False)
            _counters["launches"] += 1
        q = qkv[..., : H * D].unflatten(-1, (H, D))
        k = qkv[..., H * D : (H + KV) * D].unflatten(-1, (KV, D))
        v = qkv[..., (H + KV) * D :].unflatten(-1, (KV, D))
        scale = 1.0 / math.sqrt(D)
        o, lse = C.flash_attn_fwd(q, k, v, scale, causal)
        _counters["launches"] += 1
        ctx.save_for_backward(qkv, o, lse, freqs)
        ctx.meta = (H, KV, D, pos0, causal, scale)
        return o.view(B, T, H * D)

    @staticmethod
    def backward(ctx, dout):
        C = _C()
        qkv, o, lse, freqs = ctx.saved_tensors
        H, KV, D, pos0, causal, scale = ctx.meta
        B, T, _ = qkv.shape
        q = qkv[..., : H * D].unflatten(-1, (H, D))
        k = qkv[..., H * D : (H + KV) * D].unflatten(-1, (KV, D))
        v = qkv[..., (H + KV) * D :].unflatten(-1, (KV, D))
        dqkv = torch.empty_like(qkv)
        dq = dqkv[..., : H * D].unflatten(-1, (H, D))
        dk = dqkv[..., H * D : (H + KV) * D].unflatten(-1, (KV, D))
        dv = dqkv[..., (H + KV) * D :].unflatten(-1, (KV, D))
        do = dout.reshape(B, T, H, D)
        if do.dtype != torch.bfloat16:
            do = do.to(torch.bfloat16)
        do = do if do.is_contiguous() else do.contiguous()
        C.flash_attn_bwd(do, q, k, v, o, lse, dq, dk, dv, scale, causal)
        _counters["launches"] += 4
        if freqs is not None:
            C.rope_inplace(dqkv, freqs, B, T, H + KV, D, dqkv.stride(1), pos0, True)
            _counters["launches"] += 1
        return dqkv, None, None, None, None, None, None


def attention_packed(qkv, n_head, n_kv_head, head_dim, freqs=None, pos0=0, causal=True):
    """Self-attention on a packed QKV projection ``[B, T, (H + 2 KV) D]`` -> ``[B, T, H D]``.

    ``freqs`` is the ``[T_max, D/2, 2]`` (cos, sin) table for rotary embedding or ``None``.
    On CUDA the packed buffer is rotated in place.
    """
    H, KV, D = n_head, n_kv_head, head_dim
    if qkv.is_cuda and D in (64, 128) and _use_fused(qkv):
        return _AttentionFn.apply(qkv, H, KV, D, freqs, pos0, causal)
    B, T, _ = qkv.shape
    q = qkv[..., : H * D].reshape(B, T, H, D)
    k = qkv[..., H * D : (H + KV) * D].reshape(B, T, KV, D)
    v = qkv[..., (H + KV) * D :].reshape(B, T, KV, D)
    if freqs is not None:
        q = ref.apply_rope(q, freqs, pos0)
        k = ref.apply_rope(k, freqs, pos0)
    return ref.attention(q, k, v, causal).reshape(B, T, H * D)


# --------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, wte, wpe, pos0, vocab_start, out_dtype):
        C = _C()
        idx = idx if idx.is_contiguous() else idx.contiguous()
        out = C.embedding_fwd(idx, wte, wpe, pos0, vocab_start, out_dtype)
        _counters["launches"] += 1
        ctx.save_for_backward(idx, wte, wpe)
        ctx.meta = (pos0, vocab_start)
        return out

    @staticmethod
    def backward(ctx, dout):
        C = _C()
        idx, wte, wpe = ctx.saved_tensors
        pos0, vocab_start = ctx.meta
        dout = dout if dout.is_contiguous() else dout.contiguous()
        dwte = torch.zeros_like(wte, dtype=torch.float32) if ctx.needs_input_grad[1] else None
        dwpe = torch.zeros_like(wpe, dtype=torch.float32) if (wpe is not None and ctx.needs_input_grad[2]) else None
        C.embedding_bwd(idx, dout, dwte, dwpe, pos0, vocab_start)
        _counters["launches"] += 2 + (dwte is not None) + (dwpe is not None)
        return None, dwte, dwpe, None, None, None


def embedding(idx, wte, wpe=None, pos0=0, vocab_start=0):
    """Token (+ position) embedding; ids outside ``[vocab_start, vocab_start + len(wte))`` give zero rows."""
    if wte.is_cuda and wte.dtype == torch.float32 and wte.shape[1] % 8 == 0 and idx.dim() == 2 and _ext.available():
        out_dtype = torch.bfloat16 if (_AutocastState.enabled and _AutocastState.dtype == torch.bfloat16) else torch.float32
        return _EmbeddingFn.apply(idx, wte, wpe, pos0, vocab_start, out_dtype)
    return ref.embedding(idx, wte, wpe, pos0, vocab_start)


# --------------------------------------------------------------------------- cross entropy
class _CrossEntropyFn(torch.autograd.Function):
    """Mean softmax cross-entropy; the backward pass overwrites the logits buffer with dlogits."""

    @staticmethod
    def forward(ctx, logits, target):
        C = _C()
        V = logits.shape[-1]
        l2 = logits.reshape(-1, V) if logits.dim() != 2 else logits
        if l2.stride(-1) != 1:
            l2 = l2.contiguous()
        t = target.reshape(-1)
        t = t if t.is_contiguous() else t.contiguous()
        loss, lse, _ = C.ce_fwd(l2, t, V)
        _counters["launches"] += 1
        ctx.save_for_backward(l2, t, lse)
        ctx.shape = logits.shape
        return loss.reshape(())

    @staticmethod
    def backward(ctx, g):
        C = _C()
        l2, t, lse = ctx.saved_tensors
        V = l2.shape[-1]
        C.ce_bwd(l2, t, lse, g.reshape(1).float(), V, True)
        _counters["launches"] += 1
        return l2.view(ctx.shape), None


def cross_entropy(logits, target):
    """Mean cross-entropy over all rows.  On CUDA the logits tensor is consumed: after backward it
    holds the gradient."""
    if logits.is_cuda and logits.dtype in (torch.float32, torch.bfloat16) and _ext.available():
        return _CrossEntropyFn.apply(logits, target)
    return ref.cross_entropy(logits, target)
