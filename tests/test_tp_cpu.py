"""Tensor / sequence parallel training on CPU ranks (gloo) against the unpartitioned model."""
import os

import pytest
import torch

from dist_utils import run_ranks
from infinitrain_b200.models import llmc
from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel


def _cfg(family):
    if family == "gpt2":
        return TransformerConfig.GPT2(n_layer=2, n_embd=32, n_head=4, n_kv_head=4, vocab_size=96, original_vocab_size=90,
                                      block_size=16)
    return TransformerConfig.LLaMA3(n_layer=2, n_embd=32, n_head=4, n_kv_head=2, vocab_size=96, original_vocab_size=90,
                                    block_size=16, multiple_of=16)


def _data():
    g = torch.Generator().manual_seed(3)
    return torch.randint(0, 90, (2, 16), generator=g), torch.randint(0, 90, (2, 16), generator=g)


def _tp_train_worker(rank, world, family, path, ref_losses):
    from infinitrain_b200.optim import SGD
    from infinitrain_b200.parallel.tensor_parallel import AllReduceSequenceParallelGrads, VocabParallelCrossEntropyLoss

    m = llmc.GPT2FromLLMC(path) if family == "gpt2" else llmc.LLaMA3FromLLMC(path)
    opt = SGD(m.Parameters(), 0.05)
    loss_fn = VocabParallelCrossEntropyLoss(90)
    x, y = _data()
    for s in range(3):
        opt.ZeroGrad()
        loss = loss_fn(m(x), y)
        loss.backward()
        AllReduceSequenceParallelGrads(m)
        opt.Step()
        assert abs(loss.item() - ref_losses[s]) < 2e-5, (s, loss.item(), ref_losses[s])


@pytest.mark.parametrize("family,sp", [("llama3", False), ("llama3", True), ("gpt2", True)])
def test_tp2_training_matches_unpartitioned(tmp_path, family, sp):
    from infinitrain_b200.optim import SGD
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory
    from infinitrain_b200.parallel.tensor_parallel import VocabParallelCrossEntropyLoss

    genv.InitAllEnv(world_size=1, rank=0)
    ProcessGroupFactory.Reset()
    ProcessGroupFactory.Instance().Init()
    torch.manual_seed(2)
    cfg = _cfg(family)
    m = TransformerModel(cfg)
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.05)
        # padded vocabulary rows (>= original vocab) are zero in llm.c files
        m.lm_head.weight[90:].zero_()
    path = os.path.join(tmp_path, "w.bin")
    if family == "gpt2":
        llmc.write_gpt2_llmc(path, cfg, llmc.full_state_dict(m), padded_vocab_size=96)
    else:
        llmc.write_llama3_llmc(path, cfg, llmc.full_state_dict(m))
    opt = SGD(m.Parameters(), 0.05)
    loss_fn = VocabParallelCrossEntropyLoss(90)
    x, y = _data()
    ref = []
    for _ in range(3):
        opt.ZeroGrad()
        loss = loss_fn(m(x), y)
        loss.backward()
        opt.Step()
        ref.append(loss.item())
    run_ranks(_tp_train_worker, 2, args=(family, path, ref), tp=2, sp=sp)


def test_fused_tp_launch_bookkeeping_without_a_gpu():
    """The host side of the fused tensor-parallel launches: workspace reuse distances ("lag"), which
    hooks a launch enables, and the reuse of a gathered activation -- with the kernel call replaced by
    a recorder."""
    import torch

    from infinitrain_b200.parallel import symm

    class FakeC:
        TP_PUSH, TP_GATE_A, TP_SCATTER, TP_BROADCAST = 1, 2, 4, 8

        def __init__(self):
            self.calls = []

        def tp_gemm(self, a, a_mn, b, b_mn, M, N, K, c, c2, bias, aux, flags, tp, err):
            self.calls.append(dict(tp))

    class FakeNvl:
        rank, world, device = 1, 4, torch.device("cpu")
        err = torch.zeros(1, dtype=torch.int32)

    class FakeBuf:
        def __init__(self, n):
            self.t = torch.zeros(n)
            self.ptrs, self.mc = [10, 20, 30, 40], 99
            self.arrive_ptrs, self.my_arrive = [1, 2, 3, 4], 2
            self.total = torch.zeros(1, dtype=torch.int32)
            self.last_use, self.content = None, None

        holds = symm._SymBuf.holds

    tp = object.__new__(symm.TpFusedContext)
    tp.nvl, tp.C, tp.rank, tp.world = FakeNvl(), FakeC(), 1, 4
    tp.flag_ptrs = [100, 200, 300, 400]
    tp.launch_ctr = torch.zeros(1, dtype=torch.int32)
    tp.cta_done = torch.zeros(1, dtype=torch.int32)
    tp.launch_index, tp._bufs = 0, {}
    gather, slab = FakeBuf(16), FakeBuf(16)
    x = torch.zeros(4, 4)
    a = b = torch.zeros(2, 2)
    never = 1 << 24
    tp.launch(a, False, b, False, 8, 8, 8, None, None, None, None, 0, batch=1, T=8, push=gather, push_src=x, gate=gather)
    tp.launch(a, False, b, False, 8, 8, 8, None, None, None, None, 0, batch=1, T=8, slab=slab, rs_out=x)
    tp.launch(a, False, b, False, 8, 8, 8, None, None, None, None, 0, batch=1, T=8, push=gather, push_src=x, gate=gather)
    tp.launch(a, False, b, False, 8, 8, 8, None, None, None, None, 0, batch=1, T=8, slab=slab, rs_out=x, bcast=gather)
    c = tp.C.calls
    assert [d["mode"] for d in c] == [1 | 2, 4, 1 | 2, 4 | 8]
    assert c[0]["push_lag"] == never and c[2]["push_lag"] == 2          # reused two launches later
    assert c[1]["rs_lag"] == never and c[3]["rs_lag"] == 2
    assert c[3]["ar_lag"] == 1 and c[3]["ar_out"] == gather.ptrs and c[3]["ar_mc"] == 99
    assert c[0]["Tl"] == 2 and c[0]["rank"] == 1 and c[0]["world"] == 4 and c[0]["started"] == tp.flag_ptrs
    assert tp.launch_index == 4 and gather.last_use == 3 and slab.last_use == 3
    # the gathered copy is reused only for the very tensor that was pushed, unmodified
    assert gather.holds(x)
    assert not gather.holds(torch.zeros(4, 4))
    x.add_(1)
    assert not gather.holds(x)
