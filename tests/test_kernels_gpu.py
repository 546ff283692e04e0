"""Numerics of every single-GPU sm_100a kernel against a plain PyTorch fp32 reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["pair", "single"])
def C(request):
    """Every kernel test runs with both GEMM kernels: CTA pairs (cta_group::2) and single CTAs."""
    from infinitrain_b200 import _ext

    mod = _ext.load(required=True)
    old = mod.get_gemm_mode()
    mod.set_gemm_mode(1 if request.param == "pair" else 0)
    yield mod
    mod.set_gemm_mode(old)
    assert mod.kernel_status() == 0, "a kernel wait timed out"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


GEMM_SHAPES = [(128, 256, 64), (256, 512, 128), (200, 264, 72), (1024, 768, 768), (384, 2304, 768),
               (130, 50264, 64)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_forward_layout(C, M, N, K):
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    C.gemm(a, False, b, False, M, N, K, c, None, None, None, None, 0, 0)
    ref = a.float() @ b.float().t()
    assert _rel(c, ref) < 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 512, 128), (200, 264, 72), (1024, 768, 3072)])
def test_gemm_dgrad_layout(C, M, N, K):
    # dx[M,K'] = dy[M,N'] @ W[N',K'] : A K-major (contraction N'), B MN-major.
    torch.manual_seed(1)
    dy = torch.randn(M, K, device="cuda").bfloat16()          # contraction length K
    w = torch.randn(K, N, device="cuda").bfloat16()           # stored [contraction, out]
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    C.gemm(dy, False, w, True, M, N, K, c, None, None, None, None, 0, 0)
    ref = dy.float() @ w.float()
    assert _rel(c, ref) < 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 512, 128), (264, 200, 520), (768, 3072, 4096)])
def test_gemm_wgrad_layout_splitk(C, M, N, K):
    # dW[M,N] = dy[K,M]^T @ x[K,N] : both MN-major, fp32 output accumulated with atomics.
    torch.manual_seed(2)
    dy = torch.randn(K, M, device="cuda").bfloat16()
    x = torch.randn(K, N, device="cuda").bfloat16()
    c = torch.zeros(M, N, device="cuda", dtype=torch.float32)
    C.gemm(dy, True, x, True, M, N, K, c, None, None, None, None, C.GEMM_OUT_F32 | C.GEMM_ATOMIC, 0)
    ref = dy.float().t() @ x.float()
    assert _rel(c, ref) < 1e-3
    c2 = torch.empty(M, N, device="cuda", dtype=torch.float32)
    C.gemm(dy, True, x, True, M, N, K, c2, None, None, None, None, C.GEMM_OUT_F32, 0)
    assert _rel(c2, ref) < 1e-3


def test_gemm_epilogues(C):
    torch.manual_seed(3)
    M, N, K = 512, 768, 256
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = (torch.randn(N, K, device="cuda") / math.sqrt(K)).bfloat16()
    bias = torch.randn(N, device="cuda")
    res = torch.randn(M, N, device="cuda").bfloat16()
    ref = a.float() @ b.float().t() + bias
    # bias + residual, bf16 out
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    C.gemm(a, False, b, False, M, N, K, c, None, bias, res, None, C.GEMM_BIAS | C.GEMM_RESIDUAL, 0)
    assert _rel(c, ref + res.float()) < 1e-2
    # gelu dual store
    h = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    g = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    C.gemm(a, False, b, False, M, N, K, h, g, bias, None, None, C.GEMM_BIAS | C.GEMM_GELU_DUAL, 0)
    assert _rel(h, ref) < 1e-2
    assert _rel(g, torch.nn.functional.gelu(h.float(), approximate="tanh")) < 1e-2
    # dgelu epilogue
    hh = h.float().requires_grad_(True)
    torch.nn.functional.gelu(hh, approximate="tanh").sum().backward()
    d = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    C.gemm(a, False, b, False, M, N, K, d, None, None, None, h, C.GEMM_DGELU, 0)
    assert _rel(d, (a.float() @ b.float().t()) * hh.grad) < 1e-2
    # fp32 out with residual and accumulate
    r32 = torch.randn(M, N, device="cuda")
    c32 = torch.empty(M, N, device="cuda")
    C.gemm(a, False, b, False, M, N, K, c32, None, bias, r32, None,
           C.GEMM_OUT_F32 | C.GEMM_BIAS | C.GEMM_RESIDUAL, 0)
    assert _rel(c32, ref + r32) < 1e-3
    acc = r32.clone()
    C.gemm(a, False, b, False, M, N, K, acc, None, None, None, None, C.GEMM_OUT_F32 | C.GEMM_ACCUM, 0)
    assert _rel(acc, r32 + a.float() @ b.float().t()) < 1e-3


@pytest.mark.parametrize("rows,Cdim", [(64, 768), (1000, 768), (33, 2048), (16, 4096)])
@pytest.mark.parametrize("xdt", [torch.float32, torch.bfloat16])
def test_layernorm(C, rows, Cdim, xdt):
    torch.manual_seed(4)
    x = torch.randn(rows, Cdim, device="cuda").to(xdt)
    g = torch.randn(Cdim, device="cuda")
    b = torch.randn(Cdim, device="cuda")
    y, mean, rstd = C.layernorm_fwd(x, g, b, 1e-5, torch.bfloat16)
    xr = x.float().requires_grad_(True)
    gr = g.clone().requires_grad_(True)
    br = b.clone().requires_grad_(True)
    ref = torch.nn.functional.layer_norm(xr, (Cdim,), gr, br, 1e-5)
    assert _rel(y, ref) < 1e-2
    assert torch.allclose(mean, xr.mean(-1), atol=1e-4)
    dy = torch.randn(rows, Cdim, device="cuda").bfloat16()
    ref.backward(dy.float())
    dx, dg, db, _ = C.layernorm_bwd(dy, x, g, mean, rstd, True)
    assert dx.dtype == x.dtype
    assert _rel(dx, xr.grad) < (1e-2 if xdt == torch.bfloat16 else 1e-4)
    assert _rel(dg, gr.grad) < 1e-3 and _rel(db, br.grad) < 1e-3
    # on a residual stream: dx = norm'(dy) + dres, column sums of dres, gradients accumulated into given slots
    dres = torch.randn(rows, Cdim, device="cuda").to(xdt)
    slot_g, slot_b, slot_s = (torch.full((Cdim,), 0.5, device="cuda") for _ in range(3))
    dx2, dg2, db2, ds2 = C.layernorm_bwd(dy, x, g, mean, rstd, True, dres, slot_g, slot_b, slot_s)
    assert dg2.data_ptr() == slot_g.data_ptr() and ds2.data_ptr() == slot_s.data_ptr()
    assert _rel(dx2.float(), xr.grad + dres.float()) < (1e-2 if xdt == torch.bfloat16 else 1e-4)
    assert _rel(slot_g, gr.grad + 0.5) < 1e-3 and _rel(slot_b, br.grad + 0.5) < 1e-3
    assert _rel(slot_s, dres.float().sum(0) + 0.5) < 1e-3
    _, _, _, ds3 = C.layernorm_bwd(dy, x, g, mean, rstd, True, dres, None, None, None, True)
    assert _rel(ds3, dres.float().sum(0)) < 1e-3


@pytest.mark.parametrize("rows,Cdim", [(64, 768), (257, 2048), (48, 4096)])
@pytest.mark.parametrize("xdt", [torch.float32, torch.bfloat16])
def test_rmsnorm(C, rows, Cdim, xdt):
    torch.manual_seed(5)
    x = torch.randn(rows, Cdim, device="cuda").to(xdt)
    g = torch.randn(Cdim, device="cuda")
    y, rstd = C.rmsnorm_fwd(x, g, 1e-5, torch.bfloat16)
    xr = x.float().requires_grad_(True)
    gr = g.clone().requires_grad_(True)
    ref = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * gr
    assert _rel(y, ref) < 1e-2
    dy = torch.randn(rows, Cdim, device="cuda").bfloat16()
    ref.backward(dy.float())
    dx, dg, _ = C.rmsnorm_bwd(dy, x, g, rstd)
    assert _rel(dx, xr.grad) < (1e-2 if xdt == torch.bfloat16 else 1e-4)
    assert _rel(dg, gr.grad) < 1e-3
    dres = torch.randn(rows, Cdim, device="cuda").to(xdt)
    slot_g = torch.full((Cdim,), 0.25, device="cuda")
    dx2, dg2, ds2 = C.rmsnorm_bwd(dy, x, g, rstd, dres, slot_g, None, True)
    assert _rel(dx2.float(), xr.grad + dres.float()) < (1e-2 if xdt == torch.bfloat16 else 1e-4)
    assert _rel(slot_g, gr.grad + 0.25) < 1e-3 and _rel(ds2, dres.float().sum(0)) < 1e-3


def test_residual_norm_block_matches_plain_autograd(C):
    """``(y, skip) = norm_skip(x)`` followed by a fused linear that adds ``skip`` back in: the backward
    pass of the norm takes the skip's gradient (no separate add), the bias gradient of that linear comes
    out of the same kernel, and parameter gradients land in their flat-buffer slots."""
    from infinitrain_b200.autocast import AutocastGuard
    from infinitrain_b200.datatype import DataType
    from infinitrain_b200.device import DeviceType
    from infinitrain_b200.ops import functional as ops

    torch.manual_seed(11)
    B, T, Cd = 2, 96, 256
    x0 = (torch.randn(B, T, Cd, device="cuda") * 0.5).bfloat16()
    gamma, beta = torch.randn(Cd, device="cuda") * 0.2 + 1, torch.randn(Cd, device="cuda") * 0.1
    w, b = torch.randn(Cd, Cd, device="cuda") * 0.05, torch.randn(Cd, device="cuda") * 0.1
    up = torch.randn(B, T, Cd, device="cuda").bfloat16()

    def run(fused):
        ps = [t.clone().requires_grad_(True) for t in (gamma, beta, w, b)]
        if fused:
            for p in ps:                  # flat-buffer slots, as DDP / the fused optimizer set them up
                p.main_grad = torch.zeros_like(p)
                p.grad = p.main_grad
        x = x0.clone().requires_grad_(True)
        with AutocastGuard(DeviceType.kCUDA, DataType.kBFLOAT16):
            if fused:
                y, skip = ops.layernorm_skip(x, ps[0], ps[1])
                out = ops.linear(y, ps[2], ps[3], residual=skip)
            else:
                out = ops.linear(ops.layernorm(x, ps[0], ps[1]), ps[2], ps[3]) + x
        out.backward(up)
        grads = [p.main_grad if fused else p.grad for p in ps]
        return out, x.grad, grads

    o1, dx1, g1 = run(True)
    o0, dx0, g0 = run(False)
    assert _rel(o1, o0) < 1e-2 and _rel(dx1, dx0) < 2e-2
    for a, r in zip(g1, g0):
        assert _rel(a, r) < 2e-2
    assert C.kernel_status() == 0


def test_gelu_swiglu(C):
    torch.manual_seed(6)
    x = torch.randn(1000, 520, device="cuda").bfloat16()
    xr = x.float().requires_grad_(True)
    ref = torch.nn.functional.gelu(xr, approximate="tanh")
    assert _rel(C.gelu_fwd(x), ref) < 1e-2
    dy = torch.randn_like(x)
    ref.backward(dy.float())
    assert _rel(C.gelu_bwd(dy, x), xr.grad) < 1e-2
    F = 264
    ab = torch.randn(300, 2 * F, device="cuda").bfloat16()
    a, b = ab[:, :F], ab[:, F:]
    ar, br = a.float().requires_grad_(True), b.float().requires_grad_(True)
    ref = ar * torch.nn.functional.silu(br)
    out = C.swiglu_fwd(a, b)
    assert _rel(out, ref) < 1e-2
    do = torch.randn(300, F, device="cuda").bfloat16()
    ref.backward(do.float())
    dab = C.swiglu_bwd(do, a, b)
    assert _rel(dab[:, :F], ar.grad) < 1e-2 and _rel(dab[:, F:], br.grad) < 1e-2


def test_rope(C):
    torch.manual_seed(7)
    B, T, H, KV, D = 2, 48, 4, 2, 64
    qkv = torch.randn(B, T, (H + 2 * KV) * D, device="cuda").bfloat16()
    orig = qkv.clone()
    pos = torch.arange(2 * T, device="cuda").float()
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.outer(pos, inv)
    freqs = torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous()  # [2T, D/2, 2]
    C.rope_inplace(qkv, freqs, B, T, H + KV, D, qkv.stride(1), 3, False)
    x = orig[..., : (H + KV) * D].float().view(B, T, H + KV, D // 2, 2)
    c = freqs[3 : 3 + T, :, 0].view(1, T, 1, D // 2)
    s = freqs[3 : 3 + T, :, 1].view(1, T, 1, D // 2)
    ref = torch.stack([x[..., 0] * c - x[..., 1] * s, x[..., 0] * s + x[..., 1] * c], -1)
    got = qkv[..., : (H + KV) * D].float().view(B, T, H + KV, D // 2, 2)
    assert _rel(got, ref) < 1e-2
    assert torch.equal(qkv[..., (H + KV) * D :], orig[..., (H + KV) * D :])  # v untouched
    C.rope_inplace(qkv, freqs, B, T, H + KV, D, qkv.stride(1), 3, True)
    assert _rel(qkv, orig) < 1e-2


def test_embedding(C):
    torch.manual_seed(8)
    B, T, Cd, V = 3, 40, 768, 1000
    idx = torch.randint(0, V, (B, T), device="cuda")
    wte = torch.randn(V, Cd, device="cuda")
    wpe = torch.randn(64, Cd, device="cuda")
    out = C.embedding_fwd(idx, wte, wpe, 0, 0, torch.bfloat16)
    ref = wte[idx] + wpe[:T]
    assert _rel(out, ref) < 1e-2
    dout = torch.randn(B, T, Cd, device="cuda").bfloat16()
    dwte = torch.zeros_like(wte)
    dwpe = torch.zeros_like(wpe)
    C.embedding_bwd(idx, dout, dwte, dwpe, 0, 0)
    rw = torch.zeros_like(wte).index_add_(0, idx.view(-1), dout.float().view(-1, Cd))
    assert _rel(dwte, rw) < 1e-4
    assert _rel(dwpe[:T], dout.float().sum(0)) < 1e-4
    # vocabulary shard: only ids in [500, 1000) are owned
    out2 = C.embedding_fwd(idx, wte[500:], None, 0, 500, torch.float32)
    ref2 = torch.where((idx >= 500).unsqueeze(-1), wte[idx], torch.zeros(1, device="cuda"))
    assert torch.allclose(out2, ref2)


@pytest.mark.parametrize("rows,V,ld,dtype", [(64, 50257, 50304, torch.bfloat16), (37, 1000, 1000, torch.float32),
                                              (16, 999, 1008, torch.bfloat16)])
def test_cross_entropy(C, rows, V, ld, dtype):
    torch.manual_seed(9)
    buf = (torch.randn(rows, ld, device="cuda") * 3).to(dtype)
    logits = buf[:, :V]
    tgt = torch.randint(0, V, (rows,), device="cuda")
    lr = logits.float().clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lr, tgt)
    loss, lse, row_loss = C.ce_fwd(buf, tgt, V)
    assert abs(loss.item() - ref.item()) < 1e-3 * max(1.0, abs(ref.item()))
    (ref * 0.5).backward()
    C.ce_bwd(buf, tgt, lse, torch.full((1,), 0.5, device="cuda"), V, True)
    assert _rel(buf[:, :V], lr.grad) < (2e-2 if dtype == torch.bfloat16 else 1e-4)
    if ld > V:
        assert buf[:, V:].abs().max().item() == 0


@pytest.mark.parametrize("gdt", [torch.float32, torch.bfloat16])
def test_adamw_sgd(C, gdt):
    torch.manual_seed(10)
    n = 100003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda").to(gdt)
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    sh = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pr = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([pr], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        pr.grad = g.float() * 0.5
        opt.step()
        C.adamw(p, g, m, v, sh, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1 - 0.9 ** step, 1 - 0.95 ** step, 0.5)
    assert torch.allclose(p, pr.detach(), atol=1e-5, rtol=1e-4)
    assert torch.equal(sh, p.bfloat16())
    p2 = p.clone()
    C.sgd(p2, g, sh, 0.1, 2.0)
    assert torch.allclose(p2, p - 0.2 * g.float(), atol=1e-6)


def test_cast_colsum(C):
    x = torch.randn(1000, 776, device="cuda")
    y = torch.empty_like(x, dtype=torch.bfloat16)
    C.cast_into(x, y)
    assert torch.equal(y, x.bfloat16())
    assert _rel(C.colsum(y), y.float().sum(0)) < 1e-4


def _attn_ref(q, k, v, causal):
    B, T, H, D = q.shape
    KV = k.shape[2]
    qf, kf, vf = q.float(), k.float(), v.float()
    kf = kf.repeat_interleave(H // KV, dim=2)
    vf = vf.repeat_interleave(H // KV, dim=2)
    s = torch.einsum("bthd,bshd->bhts", qf, kf) / math.sqrt(D)
    if causal:
        mask = torch.ones(T, T, device=q.device, dtype=torch.bool).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = s.softmax(-1)
    return torch.einsum("bhts,bshd->bthd", p, vf)


@pytest.mark.parametrize("attn_mode", [3, 0], ids=["tcgen05", "mma_sync"])
@pytest.mark.parametrize("B,T,H,KV,D", [(2, 128, 4, 4, 64), (1, 200, 4, 2, 64), (2, 96, 8, 2, 128),
                                         (1, 1024, 2, 2, 64), (2, 384, 8, 2, 128), (1, 2048, 4, 1, 128)])
def test_flash_attention(C, B, T, H, KV, D, attn_mode):
    torch.manual_seed(11)
    default_mode = C.get_attn_mode()
    C.set_attn_mode(attn_mode)
    qkv = torch.randn(B, T, (H + 2 * KV) * D, device="cuda").bfloat16()
    q = qkv[..., : H * D].view(B, T, H, D)
    k = qkv[..., H * D : (H + KV) * D].view(B, T, KV, D)
    v = qkv[..., (H + KV) * D :].view(B, T, KV, D)
    o, lse = C.flash_attn_fwd(q, k, v, 1.0 / math.sqrt(D), True)
    qr, kr, vr = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    ref = _attn_ref(qr, kr, vr, True)
    assert _rel(o, ref) < 2e-2
    dout = torch.randn_like(o)
    ref.backward(dout.float())
    dqkv = torch.empty_like(qkv)
    dq = dqkv[..., : H * D].view(B, T, H, D)
    dk = dqkv[..., H * D : (H + KV) * D].view(B, T, KV, D)
    dv = dqkv[..., (H + KV) * D :].view(B, T, KV, D)
    C.flash_attn_bwd(dout, q, k, v, o, lse, dq, dk, dv, 1.0 / math.sqrt(D), True)
    C.set_attn_mode(default_mode)
    assert C.kernel_status() == 0
    assert _rel(dv, vr.grad) < 3e-2
    assert _rel(dk, kr.grad) < 3e-2
    assert _rel(dq, qr.grad) < 3e-2


def test_bounded_wait_gives_up_with_a_status_code(C):
    """A wait on a flag that nothing sets runs out of polls, records its code and returns; the
    context stays usable.  A flag that is already set passes with status 0."""
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    C.wait_flag(flag, 1, 1 << 12, 77, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 77
    from infinitrain_b200.utils.fault_tolerance import KernelTimeout, check_kernel_status

    with pytest.raises(KernelTimeout):
        check_kernel_status(lambda: int(err.item()), "flag wait")
    err.zero_()
    flag.fill_(5)
    C.wait_flag(flag, 3, 1 << 12, 77, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert torch.ones(8, device="cuda").sum().item() == 8.0
