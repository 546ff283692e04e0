"""Token files, loaders, tokenizer, checkpoint files and resume (CPU)."""
import os

import numpy as np
import pytest
import torch

from infinitrain_b200 import nn
from infinitrain_b200.checkpoint import Checkpoint, ResumeFromCheckpoint, SaveCheckpoint, TrainerState
from infinitrain_b200.data import (DataLoader, DistributedDataLoader, TinyShakespeareDataset, Tokenizer,
                                   write_token_file, write_tokenizer_file)
from infinitrain_b200.data.tokenizer import RandomF32, RandomU32
from infinitrain_b200.optim import SGD, Adam


@pytest.fixture(autouse=True)
def _env():
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory

    genv.InitAllEnv(world_size=1, rank=0)
    ProcessGroupFactory.Reset()
    ProcessGroupFactory.Instance().Init()


@pytest.mark.parametrize("llama3", [False, True])
def test_token_dataset_and_loaders(tmp_path, llama3):
    toks = np.arange(1000) % (60000 if not llama3 else 100000)
    path = os.path.join(tmp_path, "tok.bin")
    write_token_file(path, toks, llama3)
    ds = TinyShakespeareDataset(path, 16)
    assert ds.Size() == 1000 // 16 - 1
    x, y = ds[3]
    assert x.dtype == torch.int64 and x.tolist() == list(range(48, 64)) and y.tolist() == list(range(49, 65))
    dl = DataLoader(ds, 4)
    xb, yb = next(iter(dl))
    assert xb.shape == (4, 16) and xb[1, 0].item() == 16 and yb[1, 0].item() == 17
    # rank r of 2 reads batches r, r+2, ...
    for r in range(2):
        it = iter(DistributedDataLoader(ds, 4, r, 2, pin_memory=False))
        b0, _ = next(it)
        b1, _ = next(it)
        assert b0[0, 0].item() == r * 4 * 16 and b1[0, 0].item() == (r + 2) * 4 * 16
    n0 = sum(1 for _ in DistributedDataLoader(ds, 4, 0, 2, pin_memory=False))
    n1 = sum(1 for _ in DistributedDataLoader(ds, 4, 1, 2, pin_memory=False))
    assert n0 + n1 == ds.Size() // 4


def test_tokenizer_and_sampler(tmp_path):
    path = os.path.join(tmp_path, "tok.tokenizer")
    write_tokenizer_file(path, [b"a", b"bc", b" d"], magic=20240328, version=2, eot=2)
    t = Tokenizer(path)
    assert t.vocab_size == 3 and t.GetEndOfText() == 2 and t.Decode(1) == "bc" and t.Decode(9) == "[INVALID_TOKEN]"
    s = [1337]
    a, b = RandomU32(s), RandomU32(s)
    assert a != b and 0 <= RandomF32(s) < 1.0
    s2 = [1337]
    assert RandomU32(s2) == a        # deterministic stream


def test_state_dict_file_roundtrip(tmp_path):
    sd = {"w": torch.randn(3, 5), "b": torch.arange(7, dtype=torch.int64), "h": torch.randn(4).bfloat16(),
          "s": torch.tensor(3.5)}
    p = os.path.join(tmp_path, "x.ckpt")
    Checkpoint.SaveStateDict(p, sd)
    with open(p, "rb") as f:
        assert int.from_bytes(f.read(4), "little") == 0x54504B43 and int.from_bytes(f.read(4), "little") == 1
    back = Checkpoint.LoadStateDict(p)
    assert list(back.keys()) == list(sd.keys())
    for k in sd:
        assert back[k].dtype == sd[k].dtype and torch.equal(back[k], sd[k])
    with open(p, "r+b") as f:        # corrupt the magic: the reader must refuse
        f.write(b"\0\0\0\0")
    with pytest.raises(RuntimeError):
        Checkpoint.LoadStateDict(p)


def test_trainer_state_json_tolerant(tmp_path):
    p = os.path.join(tmp_path, "trainer_state.json")
    Checkpoint.SaveTrainerState(p, TrainerState(global_step=30, consumed_batches=120, last_lr=1e-4, n_layer=12, vocab_size=50257))
    import json

    assert json.load(open(p))["global_step"] == 30          # valid JSON
    # the reference's writer forgets the comma after vocab_size: still readable
    open(p, "w").write('{\n  "n_layer": 12,\n  "vocab_size": 50257\n  "global_step": 31,\n  "last_lr": 0.0001\n}\n')
    st = Checkpoint.LoadTrainerState(p)
    assert st.global_step == 31 and st.vocab_size == 50257 and abs(st.last_lr - 1e-4) < 1e-12


def test_checkpoint_resume_continues_identically(tmp_path):
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel

    cfg = TransformerConfig.GPT2(n_layer=2, n_embd=32, n_head=2, n_kv_head=2, vocab_size=64, original_vocab_size=64,
                                 block_size=16)
    torch.manual_seed(0)
    x = torch.randint(0, 64, (4, 16))

    def steps(model, opt, n):
        out = []
        for _ in range(n):
            opt.ZeroGrad()
            loss = nn.CrossEntropyLoss()(model(x), x)
            loss.backward()
            opt.Step()
            out.append(loss.item())
        return out

    m = TransformerModel(cfg)
    opt = Adam(m.Parameters(), 1e-2)
    steps(m, opt, 3)
    root = os.path.join(tmp_path, "ck")
    SaveCheckpoint(root, 3, m, opt, cfg, consumed_batches=3, last_lr=1e-2, max_checkpoint_keep=2)
    cont = steps(m, opt, 2)
    m2 = TransformerModel(cfg)
    opt2 = Adam(m2.Parameters(), 1e-2)
    res = ResumeFromCheckpoint(os.path.join(root, "checkpoint_step_000003"), m2, opt2, cfg)
    assert res.global_step == 3 and res.consumed_batches == 3 and opt2.t == 3
    assert steps(m2, opt2, 2) == pytest.approx(cont, abs=1e-6)
    # Adam's t advances even when no gradient exists; SGD has no state
    opt2.ZeroGrad()
    opt2.Step()
    assert int(opt2.StateDict()["adam.t"]) == 6 and SGD(m2.Parameters(), 0.1).StateDict() == {}
    # pruning keeps the newest two
    for s in (4, 5, 6):
        SaveCheckpoint(root, s, m, opt, cfg, max_checkpoint_keep=2)
    assert sorted(os.listdir(root)) == ["checkpoint_step_000005", "checkpoint_step_000006"]
    # topology / shape validation
    bad = TransformerConfig.GPT2(n_layer=3, n_embd=32, n_head=2, n_kv_head=2, vocab_size=64, original_vocab_size=64, block_size=16)
    with pytest.raises((ValueError, KeyError)):
        ResumeFromCheckpoint(os.path.join(root, "checkpoint_step_000006"), TransformerModel(bad), None, bad, False)


def test_zero_optimizer_state_resharding():
    """State saved by 4 data-parallel ranks, resumed on 2 and on 3: every parameter's moments end up
    at the offsets the new flat layout gives them."""
    import torch

    from infinitrain_b200.checkpoint.reshard import gather_full_optimizer_state, reshard_zero_optimizer_state
    from infinitrain_b200.parallel.ddp.param_and_grad_buffer import plan_flat_layout

    torch.manual_seed(0)
    numels = [130, 4096, 77, 250_000, 1_200_000, 64, 900_000, 31]
    truth = [{"adam.m": torch.randn(n), "adam.v": torch.rand(n)} for n in numels]

    def shards_for(dp):
        lay = plan_flat_layout(numels, dp, shard=True)
        states = [dict() for _ in range(dp)]
        for key in ("adam.m", "adam.v"):
            flat = torch.zeros(lay.numel)
            for (s, e, _), t in zip(lay.param_ranges, truth):
                flat[s:e] = t[key]
            for b, (bs, be) in enumerate(lay.bucket_ranges):
                n = (be - bs) // dp
                for r in range(dp):
                    states[r][f"{key}.{b}"] = flat[bs + r * n: bs + (r + 1) * n].clone()
        for r in range(dp):
            states[r]["adam.t"] = torch.tensor(7)
        return states

    old = shards_for(4)
    for new_dp in (2, 3, 1, 8):
        want = shards_for(new_dp)
        for r in range(new_dp):
            got = reshard_zero_optimizer_state(old, numels, new_dp, r)
            assert set(got) == set(want[r])
            for k in want[r]:
                assert torch.equal(got[k], want[r][k]), (new_dp, r, k)
    full = gather_full_optimizer_state(old, numels)
    for f, t in zip(full, truth):
        assert torch.equal(f["adam.m"], t["adam.m"]) and torch.equal(f["adam.v"], t["adam.v"])


def test_optimizer_state_by_parameter_name():
    """Adam state keyed by parameter name loads into an optimizer whose parameters come in another
    order; the positional keys of the reference keep working."""
    from infinitrain_b200 import nn
    from infinitrain_b200.optim import Adam

    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(4, 3), nn.Linear(3, 2))
    opt = Adam(m.Parameters(), 1e-2)
    for _ in range(2):
        opt.ZeroGrad()
        m(torch.randn(5, 4)).sum().backward()
        opt.Step()
    named = opt.NamedStateDict(m)
    assert "adam.m.0.weight" in named and "adam.v.1.bias" in named and int(named["adam.t"]) == 2
    other = Adam(list(reversed(m.Parameters())), 1e-2)
    other.LoadStateDict(named, model=m)
    for p, mm in zip(other.params, other.m):
        i = [id(q) for q in opt.params].index(id(p))
        assert torch.equal(mm, opt.m[i])
    assert other.t == 2
    again = Adam(m.Parameters(), 1e-2)
    again.LoadStateDict(opt.StateDict())                      # positional form
    assert torch.equal(again.v[3], opt.v[3])


def test_resume_reports_a_topology_mismatch_before_loading(tmp_path):
    """A checkpoint of a 2-way tensor-parallel run, resumed in a run without tensor parallelism, is
    refused by its recorded topology, not by a shape error half way through the weights."""
    from infinitrain_b200.checkpoint.checkpoint import Checkpoint, ResumeFromCheckpoint, TrainerState
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel
    from infinitrain_b200.parallel import global_env as genv

    genv.InitAllEnv(world_size=1, rank=0)
    cfg = TransformerConfig.GPT2(n_layer=1, n_embd=32, n_head=4, n_kv_head=4, vocab_size=64, original_vocab_size=64, block_size=16)
    m = TransformerModel(cfg)
    for r in (0, 1):
        d = tmp_path / "ck" / f"rank_{r:06d}"
        d.mkdir(parents=True)
        Checkpoint.SaveTrainerState(str(d / "trainer_state.json"),
                                    TrainerState(2, 2, 1e-4, 1, 4, 4, 32, 64, ddp_size=1, tp_size=2, sp_size=1, pp_size=1))
    with pytest.raises(ValueError, match="TP_SIZE mismatch: checkpoint has 2, but current run has 1"):
        ResumeFromCheckpoint(str(tmp_path / "ck"), m, None, cfg)


def test_newest_complete_checkpoint_skips_what_a_failure_left_half_written(tmp_path):
    """A step directory counts for a rank only when its trainer_state.json (written last, through a
    rename) is there, parses and names that step."""
    from infinitrain_b200.checkpoint import Checkpoint, NewestCompleteCheckpoint, TrainerState
    from infinitrain_b200.parallel import global_env as genv

    genv.InitAllEnv(world_size=1, rank=0)
    assert NewestCompleteCheckpoint(str(tmp_path / "absent")) == 0
    for step in (2, 4, 6):
        d = tmp_path / f"checkpoint_step_{step:06d}"
        d.mkdir()
        if step != 6:                                      # step 6: model written, the job died before the state file
            Checkpoint.SaveTrainerState(str(d / "trainer_state.json"), TrainerState(global_step=step))
        (d / "model.ckpt").write_bytes(b"x")
    (tmp_path / "checkpoint_step_notanumber").mkdir()
    assert NewestCompleteCheckpoint(str(tmp_path)) == 4
    (tmp_path / "checkpoint_step_000004" / "trainer_state.json").write_text("{ \"global_step\": 3 }")   # another step's file
    assert NewestCompleteCheckpoint(str(tmp_path)) == 2
    assert not (tmp_path / "checkpoint_step_000002" / "trainer_state.json.tmp").exists()
    # ranks of a larger job look into their own directories
    genv.InitAllEnv(world_size=2, rank=1)
    try:
        assert NewestCompleteCheckpoint(str(tmp_path)) == 0
        (tmp_path / "checkpoint_step_000002" / "rank_000001").mkdir()
        Checkpoint.SaveTrainerState(str(tmp_path / "checkpoint_step_000002" / "rank_000001" / "trainer_state.json"),
                                    TrainerState(global_step=2))
        assert NewestCompleteCheckpoint(str(tmp_path)) == 2
    finally:
        genv.InitAllEnv(world_size=1, rank=0)
