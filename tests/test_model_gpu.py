"""Model-level numerics on a GPU: the fused bf16 path against the fp32 PyTorch path of the same
model with the same weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup():
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory

    genv.InitAllEnv(world_size=1, rank=0)
    ProcessGroupFactory.Instance().Init()


def _run(model, x, y, autocast, steps=1, opt=None):
    from infinitrain_b200.autocast import AutocastGuard
    from infinitrain_b200.datatype import DataType
    from infinitrain_b200.device import DeviceType
    from infinitrain_b200.nn import CrossEntropyLoss

    loss_fn = CrossEntropyLoss()
    losses = []
    for _ in range(steps):
        if opt is not None:
            opt.ZeroGrad()
        with AutocastGuard(DeviceType.kCUDA, DataType.kBFLOAT16, enabled=autocast):
            loss = loss_fn(model(x), y)
        loss.backward()
        if opt is not None:
            opt.Step()
        losses.append(loss.item())
    return losses


@pytest.mark.parametrize("family", ["gpt2", "llama3"])
@pytest.mark.parametrize("residual", [torch.bfloat16, torch.float32])
def test_fused_matches_fp32_reference(family, residual):
    import copy

    from infinitrain_b200 import _ext
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel

    _setup()
    torch.manual_seed(0)
    if family == "gpt2":
        cfg = TransformerConfig.GPT2(n_layer=2, n_embd=256, n_head=4, n_kv_head=4, vocab_size=1001,
                                     original_vocab_size=1001, block_size=128, residual_dtype=residual)
    else:
        cfg = TransformerConfig.LLaMA3(n_layer=2, n_embd=256, n_head=4, n_kv_head=2, vocab_size=1000,
                                       original_vocab_size=1000, block_size=128, multiple_of=64,
                                       residual_dtype=residual)
    ref_model = TransformerModel(cfg)
    with torch.no_grad():
        for p in ref_model.parameters():
            if p.dim() >= 2:
                p.normal_(0, 0.02)
    gpu_model = copy.deepcopy(ref_model).cuda()
    x = torch.randint(0, 1000, (2, 128))
    y = torch.randint(0, 1000, (2, 128))
    l_ref = _run(ref_model, x, y, autocast=False)[0]
    l_gpu = _run(gpu_model, x.cuda(), y.cuda(), autocast=True)[0]
    assert abs(l_ref - l_gpu) < 1e-2, (l_ref, l_gpu)
    ref_grads = dict((n, p.grad) for n, p in ref_model.named_parameters())
    for n, p in gpu_model.named_parameters():
        g, r = p.grad.float().cpu(), ref_grads[n]
        rel = (g - r).norm() / (r.norm() + 1e-12)
        assert rel < 6e-2, (n, rel.item())
    assert _ext.load().kernel_status() == 0


def test_training_reduces_loss_with_fused_optimizer():
    from infinitrain_b200.models import GPT2
    from infinitrain_b200.optim import Adam

    _setup()
    torch.manual_seed(0)
    model = GPT2("gpt2", n_layer=2, block_size=128).cuda()
    opt = Adam(model.Parameters(), 1e-3)
    assert opt._flat is not None, "fused flat-buffer optimizer expected on CUDA"
    x = torch.randint(0, 50257, (4, 128), device="cuda")
    y = torch.randint(0, 50257, (4, 128), device="cuda")
    losses = _run(model, x, y, autocast=True, steps=8, opt=opt)
    assert losses[-1] < losses[0] - 0.5, losses
    # the bf16 shadow the GEMMs read is the rounded fp32 master
    w = model.lm_head.weight
    assert torch.equal(w._itb_shadow, w.detach().bfloat16())


@pytest.mark.parametrize("family", ["gpt2", "llama3"])
def test_same_seed_runs_are_bit_identical_where_the_algorithm_is(family):
    """Two runs from the same seed on the same inputs.  The forward pass uses fixed reduction orders
    throughout (GEMM tiles, attention, norms), so the logits must agree bit for bit.  Three reductions
    are unordered fp32 sums and make what follows them reproducible only to rounding: the mean of the
    row losses (atomics), the dQ accumulation of the attention backward over key tiles (bulk
    add-reductions) and the token-table gradient (atomics on shared ids).  Loss and gradients are
    therefore compared with a tight tolerance instead."""
    from infinitrain_b200.autocast import AutocastGuard
    from infinitrain_b200.datatype import DataType
    from infinitrain_b200.device import DeviceType
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel

    _setup()

    def once():
        from infinitrain_b200.nn import init

        init.manual_seed(123)   # the framework's one initialisation stream
        torch.manual_seed(123)
        if family == "gpt2":
            cfg = TransformerConfig.GPT2(n_layer=2, n_embd=256, n_head=4, n_kv_head=4, vocab_size=1001,
                                         original_vocab_size=1001, block_size=256)
        else:
            cfg = TransformerConfig.LLaMA3(n_layer=2, n_embd=256, n_head=4, n_kv_head=2, vocab_size=1000,
                                           original_vocab_size=1000, block_size=256, multiple_of=64)
        model = TransformerModel(cfg).cuda()
        g = torch.Generator().manual_seed(5)
        x = torch.randint(0, 1000, (4, 256), generator=g).cuda()
        y = torch.randint(0, 1000, (4, 256), generator=g).cuda()
        with torch.no_grad(), AutocastGuard(DeviceType.kCUDA, DataType.kBFLOAT16, enabled=True):
            logits = model(x).detach().clone()
        losses = _run(model, x, y, autocast=True, steps=1)
        grads = {n: p.grad.detach().float().clone() for n, p in model.named_parameters()}
        return logits, losses[0], grads

    o1, l1, g1 = once()
    o2, l2, g2 = once()
    assert torch.equal(o1, o2)
    assert abs(l1 - l2) <= 2e-6 * abs(l1), (l1, l2)
    for n in g1:
        rel = (g1[n] - g2[n]).norm() / (g1[n].norm() + 1e-20)
        assert rel < 1e-4, (n, rel.item())


def test_lagged_scalar_returns_every_value_in_order_one_step_late():
    from infinitrain_b200.utils.cuda_graph import LaggedScalar

    reader = LaggedScalar()
    seen = []
    static = torch.zeros((), device="cuda")
    for i in range(5):
        static.fill_(float(i) + 0.5)         # the producer overwrites one static tensor, as a replayed graph does
        reader.push(static)
        if i >= 1:
            seen.append(reader.pop())
    seen += reader.drain()
    assert seen == [0.5, 1.5, 2.5, 3.5, 4.5]
    assert len(reader) == 0
    reader.push(static)
    reader.push(static.bfloat16())
    with pytest.raises(RuntimeError):
        reader.push(static)
