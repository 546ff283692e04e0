"""Functional wrappers, tensor helpers and the fp32 oracle ops on CPU, each against an independent
PyTorch formulation (the per-op forward/backward files of the reference's tests/autograd/)."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from infinitrain_b200 import tensor as T
from infinitrain_b200.datatype import DataType
from infinitrain_b200.nn import functional as fn
from infinitrain_b200.ops import functional as ops
from infinitrain_b200.ops import reference as ref


def test_functional_wrappers_match_torch():
    x = torch.randn(3, 4, 5).abs() + 0.1
    assert torch.equal(fn.Tril(x[0], 0), x[0].tril()) and torch.equal(fn.Triu(x[0], 1), x[0].triu(1))
    assert fn.Ones((2, 3)).sum() == 6
    for a, b in ((fn.Reciprocal, torch.reciprocal), (fn.Sin, torch.sin), (fn.Cos, torch.cos), (fn.Tanh, torch.tanh),
                 (fn.Rsqrt, torch.rsqrt), (fn.Sigmoid, torch.sigmoid)):
        assert torch.equal(a(x), b(x))
    assert torch.equal(fn.Pow(x, 2.0), x ** 2) and torch.equal(fn.Pow(2.0, x), 2.0 ** x)
    assert fn.Mean(x, 1).shape == (3, 5) and fn.Sum(x, 1, True).shape == (3, 1, 5)
    assert torch.equal(fn.Max(x, 2), x.max(2).values) and torch.equal(fn.Min(x, 0, True), x.min(0, keepdim=True).values)
    assert torch.allclose(fn.Softmax(x, 1).sum(1), torch.ones(3, 5))
    assert torch.equal(fn.Slice(x, (0, 1, 0), (3, 4, 5), (1, 2, 1)), x[:, 1:4:2, :])
    assert fn.Stack([x, x], 1).shape == (3, 2, 4, 5) and fn.Concat([x, x], 2).shape == (3, 4, 10)


def test_tensor_helpers(tmp_path, capsys):
    t = T.Tensor([2, 3], DataType.kFLOAT32)
    assert T.Dims(t) == [2, 3] and T.NumElements(t) == 6 and T.SizeInBytes(t) == 24 and T.Dtype(t) == DataType.kFLOAT32
    T.Fill(t, 2.5)
    assert float(t.sum()) == 15.0
    assert T.Dtype(T.To(t, DataType.kBFLOAT16)) == DataType.kBFLOAT16
    m = torch.tensor([[True, False, False], [False, False, True]])
    assert float(T.MaskedFill(t, m, 0.0).sum()) == 10.0
    assert T.RepeatInterleave(torch.arange(3), 2, 0).tolist() == [0, 0, 1, 1, 2, 2]
    assert T.Slice(torch.arange(10), 0, 2, 8, 3).tolist() == [2, 5]
    assert [p.shape[0] for p in T.Split(torch.zeros(7, 2), 3, 0)] == [3, 3, 1]
    assert torch.equal(T.Outer(torch.tensor([1., 2.]), torch.tensor([3., 4.])), torch.tensor([[3., 4.], [6., 8.]]))
    path = str(tmp_path / "t.npy")
    T.SaveAsNpy(t, path)
    assert np.load(path).shape == (2, 3) and float(np.load(path).sum()) == 15.0
    T.Print(t)
    assert "2.5" in capsys.readouterr().out
    seen = []
    p = torch.zeros(2, requires_grad=True)
    T.RegisterPostAccumulateGradHook(p, lambda q: seen.append(q.grad.clone()))
    (p * 3).sum().backward()
    assert len(seen) == 1 and seen[0].tolist() == [3.0, 3.0]


def test_oracle_norms_gelu_swiglu():
    x = torch.randn(4, 7, 48, dtype=torch.float64)
    g, b = torch.randn(48, dtype=torch.float64), torch.randn(48, dtype=torch.float64)
    assert torch.allclose(ref.layernorm(x, g, b, 1e-5).double(), F.layer_norm(x, (48,), g, b, 1e-5), atol=1e-5)
    want = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6) * g
    assert torch.allclose(ref.rmsnorm(x, g, 1e-6).double(), want, atol=1e-5)
    assert torch.allclose(ref.new_gelu(x), F.gelu(x, approximate="tanh"), atol=1e-12)
    assert torch.allclose(ref.swiglu(x, 2 * x), x * F.silu(2 * x))


def test_oracle_rope_equals_complex_rotation():
    B, Tn, H, D = 2, 9, 3, 16
    x = torch.randn(B, Tn, H, D)
    fr = ref.precompute_freqs_cis(D, 32, 500000.0)
    got = ref.apply_rope(x, fr, pos0=4)
    xc = torch.view_as_complex(x.reshape(B, Tn, H, D // 2, 2))
    rot = torch.view_as_complex(fr[4:4 + Tn].contiguous()).view(1, Tn, 1, D // 2)
    want = torch.view_as_real(xc * rot).reshape(B, Tn, H, D)
    assert torch.allclose(got, want, atol=1e-6)
    # a rotation keeps the norm of every pair
    assert torch.allclose(got.pow(2).sum(-1), x.pow(2).sum(-1), rtol=1e-5)


@pytest.mark.parametrize("kv", [4, 2, 1])
def test_oracle_attention_equals_sdpa_with_gqa(kv):
    B, Tn, H, D = 2, 11, 4, 8
    q, k, v = torch.randn(B, Tn, H, D), torch.randn(B, Tn, kv, D), torch.randn(B, Tn, kv, D)
    got = ref.attention(q, k, v, causal=True)
    kk, vv = k.repeat_interleave(H // kv, 2), v.repeat_interleave(H // kv, 2)
    want = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), is_causal=True)
    assert torch.allclose(got, want.transpose(1, 2), atol=1e-5)


def test_oracle_embedding_with_vocab_shard_and_positions():
    wte, wpe = torch.randn(10, 4), torch.randn(16, 4)
    idx = torch.tensor([[0, 9, 10, 19, 25]])
    out = ref.embedding(idx, wte, None, 0, vocab_start=10)          # this shard owns ids 10..19
    assert torch.equal(out[0, 2], wte[0]) and torch.equal(out[0, 3], wte[9])
    assert float(out[0, [0, 1, 4]].abs().sum()) == 0.0
    out = ref.embedding(idx, torch.randn(30, 4), wpe, pos0=3)
    assert out.shape == (1, 5, 4)
    full = torch.randn(30, 4)
    assert torch.allclose(ref.embedding(idx, full, wpe, 3), full[idx] + wpe[3:8])


def test_packed_attention_and_fused_entry_points_fall_back_on_cpu():
    """The public ops take the same arguments on CPU and give the oracle's numbers, with gradients."""
    B, Tn, H, KV, D = 2, 6, 4, 2, 8
    qkv = torch.randn(B, Tn, (H + 2 * KV) * D, requires_grad=True)
    fr = ref.precompute_freqs_cis(D, 16)
    y = ops.attention_packed(qkv, H, KV, D, fr, 0, True)
    q, k, v = qkv.split([H * D, KV * D, KV * D], -1)
    want = ref.attention(ref.apply_rope(q.view(B, Tn, H, D), fr), ref.apply_rope(k.view(B, Tn, KV, D), fr),
                         v.view(B, Tn, KV, D))
    assert torch.allclose(y.reshape(B, Tn, H, D), want, atol=1e-5)
    y.sum().backward()
    assert qkv.grad is not None and torch.isfinite(qkv.grad).all()

    x = torch.randn(5, 12, requires_grad=True)
    w, b, r = torch.randn(7, 12, requires_grad=True), torch.randn(7), torch.randn(5, 7)
    out = ops.linear(x, w, b, residual=r, gelu=True)
    assert torch.allclose(out, F.gelu(F.linear(x, w, b), approximate="tanh") + r, atol=1e-5)
    logits, tgt = torch.randn(6, 11, requires_grad=True), torch.randint(0, 11, (6,))
    loss = ops.cross_entropy(logits, tgt)
    assert torch.allclose(loss, F.cross_entropy(logits, tgt), atol=1e-6)
    loss.backward()
    want_g = (logits.detach().softmax(-1) - F.one_hot(tgt, 11)) / 6
    assert torch.allclose(logits.grad, want_g, atol=1e-6)


def test_autograd_engine_contracts():
    """What the reference's engine tests assert (tests/autograd/test_autograd.cc:110-195), on the
    engine this framework uses: needs_input_grad is visible to the function, outputs marked
    non-differentiable carry no graph, saved tensors go through pack / unpack hooks."""
    seen = {}

    class Fn(torch.autograd.Function):
        @staticmethod
        def forward(ctx, a, b):
            seen["needs"] = tuple(ctx.needs_input_grad)
            ctx.save_for_backward(a)
            idx = torch.zeros(1, dtype=torch.long)
            ctx.mark_non_differentiable(idx)
            return a * b, idx

        @staticmethod
        def backward(ctx, g, _):
            (a,) = ctx.saved_tensors
            return None, g * a

    a, b = torch.randn(3), torch.randn(3, requires_grad=True)
    packed = []

    def pack(t):
        packed.append(t.shape)
        return t.clone()

    with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
        y, idx = Fn.apply(a, b)
    assert seen["needs"] == (False, True) and not idx.requires_grad and packed == [a.shape]
    y.sum().backward()
    assert torch.equal(b.grad, a)
    with torch.no_grad():
        assert not (b * 2).requires_grad


def test_remaining_catalogue_ops():
    a, b = torch.tensor([1.0, 2.0, 0.0]), torch.tensor([1.0, 3.0, 5.0])
    for f, want in ((fn.Equals, [1, 0, 0]), (fn.Lt, [0, 1, 1]), (fn.Le, [1, 1, 1]), (fn.Gt, [0, 0, 0]), (fn.Ge, [1, 0, 0]),
                    (fn.And, [1, 1, 0]), (fn.Or, [1, 1, 1])):
        out = f(a, b)
        assert out.dtype == torch.float32 and out.tolist() == [float(v) for v in want]        # 0 / 1 in the input dtype
    assert fn.Equals(a.bfloat16(), 1.0).dtype == torch.bfloat16
    x = torch.randn(2, 3, 4)
    assert torch.equal(fn.Neg(x), -x) and torch.allclose(fn.Log(fn.Exp(x)), x, atol=1e-6)
    assert fn.Transpose(x, 0, 2).shape == (4, 3, 2) and fn.Transpose(x, 0, 2).is_contiguous()
    assert fn.Matmul(x, x.transpose(1, 2)).shape == (2, 3, 3) and fn.Outer(a, b).shape == (3, 3)
    tail = torch.tensor([[False, True, False, False]] * 3)
    assert fn.Mask(x, tail, -1.0)[1, 2, 1] == -1.0 and fn.Mask(x, tail, -1.0)[1, 2, 0] == x[1, 2, 0]
    lead = torch.tensor([[True, False, False], [False, False, True]])
    assert bool((fn.Mask(x, lead, 9.0)[0, 0] == 9.0).all()) and fn.Mask(x, lead, 9.0)[0, 1, 0] == x[0, 1, 0]
    assert torch.equal(fn.Gather(x, 2, torch.zeros(2, 3, 1, dtype=torch.long)), x[..., :1])
    vals = torch.tensor([[0.7, 0.3], [0.6, 0.4]], requires_grad=True)
    idx = torch.tensor([[2, 0], [1, 3]])
    out = fn.Scatter(vals, idx, (2, 4))
    assert out.tolist() == [[0.3, 0.0, 0.7, 0.0], [0.0, 0.6, 0.0, 0.4]] or torch.allclose(
        out, torch.tensor([[0.3, 0.0, 0.7, 0.0], [0.0, 0.6, 0.0, 0.4]]))
    (out * torch.arange(8.0).view(2, 4)).sum().backward()
    assert torch.allclose(vals.grad, torch.tensor([[2.0, 0.0], [5.0, 7.0]]))                  # gathered back


def test_autograd_hook_of_a_gradient_written_elsewhere_is_dropped():
    """A linear whose bias gradient is produced by the norm's backward returns no gradient for the bias;
    autograd still fires the bias's post-accumulate hook (with an undefined gradient) at that point.
    That call must not reach the reducer: the bucket would be reduced before the norm has written it."""
    import torch

    from infinitrain_b200.ops import functional as F

    class _Lin(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x, b):
            return x + b

        @staticmethod
        def backward(ctx, g):
            return g, None          # the bias gradient comes from elsewhere

    x = torch.randn(4, requires_grad=True)
    b = torch.zeros(4, requires_grad=True)
    b.main_grad = torch.zeros(4)
    ready = []
    b.register_post_accumulate_grad_hook(F.autograd_ready_hook(lambda p: ready.append("autograd")))
    b._itb_grad_ready_hooks = [lambda p: ready.append("written")]
    holder = F._SkipHolder()
    res = torch.zeros(4)
    res._itb_skip_holder = holder
    assert F.claim_bias_grad(res, b) and holder.bias is b
    _Lin.apply(x, b).sum().backward()
    assert ready == []                      # autograd's call was dropped
    F._grad_written(b)                      # the norm's backward reports the slot
    assert ready == ["written"] and not b._itb_grad_elsewhere
    # a parameter nobody claimed is reported by autograd as before
    _Lin.apply(x, b).sum().backward()
    assert ready == ["written", "autograd"]


def test_print_options_apply_to_print():
    import io

    t = torch.tensor([1.23456, 20000.5])
    try:
        T.SetPrintOptions(precision=2, sci_mode=False)
        buf = io.StringIO()
        T.Print(t, file=buf)
        assert "1.23," in buf.getvalue() and "20000.50" in buf.getvalue()
        T.SetPrintOptions(sci_mode=True)
        buf = io.StringIO()
        T.Print(t, file=buf)
        assert "e+04" in buf.getvalue()
        T.SetPrintOptions(threshold=3, edge_items=1)
        buf = io.StringIO()
        T.Print(torch.arange(10.0), file=buf)
        assert "..." in buf.getvalue()
    finally:
        T.SetPrintOptions(profile="default", sci_mode=None)
