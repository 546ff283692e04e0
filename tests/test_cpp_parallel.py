"""The C++ frontend's parallel stack (itb/parallel_env.h, process_group.h, tensor_parallel.h, ddp.h,
pipeline.h) end to end: the C++ trainer started as several CPU ranks by the C++ launcher must follow the
loss trajectory of one rank on the same weight and token files, whatever mix of tensor / sequence /
pipeline / data parallelism and ZeRO stage splits the work (reference: the per-strategy runs of
scripts/test_config.json, compared by scripts/compare_loss.py)."""
import os
import re
import socket
import subprocess

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV = {**os.environ, "OMP_NUM_THREADS": "1"}


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _losses(text):
    return [float(m.group(1)) for m in re.finditer(r"step\s+\d+/\d+\s+\|\s+train loss\s+([\d.]+)", text)]


@pytest.fixture(scope="module")
def binaries():
    import importlib.util

    from infinitrain_b200 import _ext

    spec = importlib.util.spec_from_file_location("itb_cpp_build", os.path.join(ROOT, "examples", "cpp", "build.py"))
    cpp_build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(cpp_build)
    launcher = _ext.launcher_path()
    if not launcher.exists():
        _ext.build_launcher()
    return str(launcher), str(cpp_build.build(cuda=False))


@pytest.fixture(scope="module")
def files(tmp_path_factory):
    from infinitrain_b200.data import write_token_file
    from infinitrain_b200.models import llmc
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel
    from infinitrain_b200.parallel import global_env as genv

    d = tmp_path_factory.mktemp("cpppar")
    genv.InitAllEnv(world_size=1, rank=0)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, 256, (4 * 64 * 40 + 1,), generator=g).tolist()
    write_token_file(str(d / "tokens16.bin"), toks)
    write_token_file(str(d / "tokens32.bin"), toks, llama3=True)
    torch.manual_seed(42)
    gcfg = TransformerConfig.GPT2(n_layer=4, n_embd=96, n_head=12, n_kv_head=12, vocab_size=256, original_vocab_size=256,
                                  block_size=64)
    lcfg = TransformerConfig.LLaMA3(n_layer=4, n_embd=64, n_head=4, n_kv_head=2, vocab_size=256, original_vocab_size=256,
                                    block_size=64, multiple_of=16, ffn_dim_multiplier=1.5)
    for cfg, name, write in ((gcfg, "gpt2.bin", llmc.write_gpt2_llmc), (lcfg, "llama3.bin", llmc.write_llama3_llmc)):
        m = TransformerModel(cfg)
        with torch.no_grad():
            for p in m.parameters():   # biases and norm weights away from 0 / 1, so that a lost gradient shows
                p.normal_(0, 0.1) if p.dim() > 1 else p.add_(torch.randn_like(p) * 0.1)
        write(str(d / name), cfg, llmc.full_state_dict(m))
    return d


def _train(binaries, files, family, ranks, *extra, iters=4):
    launcher, trainer = binaries
    tokens = "tokens16.bin" if family == "gpt2" else "tokens32.bin"
    cmd = [trainer, "--family", family, "--device", "cpu", "--llmc_filepath", f"{family}.bin", "--input_bin", tokens,
           "--batch_size", "2", "--sequence_length", "64", "--total_batch_size", "1024", "--num_iteration", str(iters),
           "--dtype", "float32", *extra]
    if ranks > 1:
        cmd = [launcher, f"--nproc_per_node={ranks}", f"--rdzv_endpoint=127.0.0.1:{_free_port()}", "--", *cmd]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=files, env=ENV)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    losses = _losses(r.stdout + r.stderr)
    assert len(losses) == iters, (r.stdout + r.stderr)[-3000:]
    return losses, r.stdout + r.stderr


LLAMA = ("--learning_rate", "0.01", "--optimizer", "adam")
GPT2 = ("--learning_rate", "0.05", "--optimizer", "sgd")


@pytest.fixture(scope="module")
def single(binaries, files):
    return {"llama3": _train(binaries, files, "llama3", 1, *LLAMA)[0], "gpt2": _train(binaries, files, "gpt2", 1, *GPT2)[0]}


@pytest.mark.parametrize("family,ranks,flags", [
    ("gpt2", 2, ("--tensor_parallel", "2")),
    ("gpt2", 2, ("--tensor_parallel", "2", "--sequence_parallel")),
    ("llama3", 2, ("--tensor_parallel", "2", "--sequence_parallel")),
    ("llama3", 2, ("--pipeline_parallel", "2", "--pipeline_schedule", "gpipe")),
    ("llama3", 2, ("--pipeline_parallel", "2", "--virtual_pipeline_parallel", "2")),
    ("llama3", 2, ("--zero_stage", "1")),
    ("llama3", 2, ("--zero_stage", "2", "--no_overlap_grad_reduce")),
    ("llama3", 4, ("--pipeline_parallel", "2", "--zero_stage", "1")),
    ("llama3", 8, ("--tensor_parallel", "2", "--sequence_parallel", "--pipeline_parallel", "2", "--virtual_pipeline_parallel", "2",
                   "--zero_stage", "1")),
], ids=lambda v: "_".join(s.strip("-") for s in v) if isinstance(v, tuple) else str(v))
def test_parallel_run_follows_the_single_rank_trajectory(binaries, files, single, family, ranks, flags):
    losses, log = _train(binaries, files, family, ranks, *(LLAMA if family == "llama3" else GPT2), *flags)
    want = single[family]
    assert max(abs(a - b) for a, b in zip(losses, want)) <= 2e-5, list(zip(losses, want))
    tp = int(flags[flags.index("--tensor_parallel") + 1]) if "--tensor_parallel" in flags else 1
    pp = int(flags[flags.index("--pipeline_parallel") + 1]) if "--pipeline_parallel" in flags else 1
    assert f"DP={ranks // (tp * pp)}, TP={tp}, SP={tp if '--sequence_parallel' in flags else 1}, PP={pp}" in log


def test_gpt2_pipeline_unties_the_embedding_like_the_reference_does(binaries, files, single):
    """Two stages cannot share one tensor between the lookup and the output projection: the first loss is
    the single-rank one (same weights), later ones drift by the missing tie only."""
    losses, log = _train(binaries, files, "gpt2", 2, *GPT2, "--pipeline_parallel", "2")
    assert abs(losses[0] - single["gpt2"][0]) <= 2e-6
    assert max(abs(a - b) for a, b in zip(losses, single["gpt2"])) <= 5e-3
    assert "pipeline schedule (1f1b)" in log and "F0.0" in log


def test_model_parallel_checkpoint_resumes_per_rank(binaries, files, tmp_path):
    """Every rank of a tensor-parallel job saves and reloads its own slice; the resumed run continues the
    uninterrupted one."""
    flags = (*LLAMA, "--tensor_parallel", "2")
    full, _ = _train(binaries, files, "llama3", 2, *flags, iters=4)
    _train(binaries, files, "llama3", 2, *flags, "--save", str(tmp_path), "--save_interval", "2", iters=2)
    ckpt = tmp_path / "checkpoint_step_000002"
    assert sorted(p.name for p in ckpt.iterdir()) == ["rank_000000", "rank_000001"]
    assert (ckpt / "rank_000001" / "model.ckpt").exists() and (ckpt / "rank_000001" / "trainer_state.json").exists()
    launcher, trainer = binaries
    cmd = [launcher, "--nproc_per_node=2", f"--rdzv_endpoint=127.0.0.1:{_free_port()}", "--", trainer, "--family", "llama3",
           "--device", "cpu", "--llmc_filepath", "llama3.bin", "--input_bin", "tokens32.bin", "--batch_size", "2",
           "--sequence_length", "64", "--total_batch_size", "1024", "--num_iteration", "4", "--dtype", "float32", *flags,
           "--load", str(ckpt)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=files, env=ENV)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    resumed = _losses(r.stdout + r.stderr)
    assert len(resumed) == 2 and max(abs(a - b) for a, b in zip(resumed, full[2:])) <= 2e-5, (resumed, full)


def test_profile_flag_writes_per_rank_reports_with_ops_and_collectives(binaries, files, tmp_path):
    """--profile: every rank writes <family>.report.rank<r>, <family>.records.log.rank<r> and a Chrome
    trace; the records are tagged by step and hold the ops, the optimizer step and the process-group
    collectives."""
    import shutil

    work = tmp_path / "run"
    work.mkdir()
    for name in ("llama3.bin", "tokens32.bin"):
        shutil.copy(files / name, work / name)
    launcher, trainer = binaries
    cmd = [launcher, "--nproc_per_node=2", f"--rdzv_endpoint=127.0.0.1:{_free_port()}", "--", trainer, "--family", "llama3",
           "--device", "cpu", "--llmc_filepath", "llama3.bin", "--input_bin", "tokens32.bin", "--batch_size", "2",
           "--sequence_length", "64", "--total_batch_size", "256", "--num_iteration", "2", "--dtype", "float32", *LLAMA,
           "--tensor_parallel", "2", "--profile"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=work, env=ENV)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    for rank in (0, 1):
        report = (work / f"llama3.report.rank{rank}").read_text()
        records = (work / f"llama3.records.log.rank{rank}").read_text()
        assert "Tag: Step_1" in report and "Tag: Step_2" in report and "Device Avg(us)" in report
        for name in ("linear", "rmsnorm", "attention_packed", "adam.Step", "pg.AllReduce(TP0)"):
            assert name in report, (name, report[:2000])
        first = records.splitlines()[0].split("\t")
        assert first[0] == "Step_1" and first[1] == str(rank) and first[3] == "cpu"
        # the same records as a Chrome trace: one complete event per record, the rank as the process id
        import json

        trace = json.loads((work / f"llama3.trace.rank{rank}.json").read_text())
        events = trace["traceEvents"]
        assert len(events) == len(records.splitlines()) and all(e["ph"] == "X" and e["pid"] == rank for e in events)
        assert {"linear", "pg.AllReduce(TP0)"} <= {e["name"] for e in events} and events[-1]["args"]["tag"] == "Step_2"


@pytest.mark.parametrize("flags", [("--tensor_parallel", "2"), ("--tensor_parallel", "2", "--sequence_parallel"),
                                   ("--tensor_parallel", "2", "--sequence_parallel", "--zero_stage", "1")],
                         ids=["tp2", "tp2_sp", "dp2_tp2_sp_zero1"])
def test_lora_on_tensor_parallel_linears_follows_the_single_rank_adapters(binaries, files, flags):
    """LoRA around column- and row-parallel linears (A or B split like the base weight, the replicated
    factor's partial gradients summed over the group): same loss trajectory as LoRA on one rank, whose
    adapters start from the same draws."""
    lora = (*LLAMA, "--lora_rank", "4", "--lora_alpha", "8", "--lora_target_modules", "c_attn,c_proj,c_fc,c_fc2",
            "--learning_rate", "0.02")
    one, log1 = _train(binaries, files, "llama3", 1, *lora, iters=5)
    ranks = 4 if "--zero_stage" in flags else 2
    got, log = _train(binaries, files, "llama3", ranks, *lora, *flags, iters=5)
    frozen, _ = _train(binaries, files, "llama3", 1, *lora[:-1], "0.0", iters=5)
    assert max(abs(a - b) for a, b in zip(one, frozen)) > 1e-3, (one, frozen)   # the adapters do move the loss
    assert max(abs(a - b) for a, b in zip(got, one)) <= 3e-5, list(zip(got, one))
    assert "LoRA" in log


def test_checkpoint_rotation_keeps_the_newest_steps(binaries, files, tmp_path):
    """--max_checkpoint_keep 2 with a checkpoint every step: after three steps the directories of steps 2
    and 3 are left; --save_optimizer_state=false leaves the optimizer state out.  Two data-parallel ranks:
    only rank 0 writes, both take part in the barrier before the rotation."""
    _train(binaries, files, "llama3", 2, *LLAMA, "--save", str(tmp_path), "--save_interval", "1", "--max_checkpoint_keep", "2",
           "--save_optimizer_state=false", iters=3)
    assert sorted(p.name for p in tmp_path.iterdir()) == ["checkpoint_step_000002", "checkpoint_step_000003"]
    assert sorted(p.name for p in (tmp_path / "checkpoint_step_000003").iterdir()) == ["model.ckpt", "trainer_state.json"]


def test_gpt2_padded_vocabulary_under_tensor_parallelism(binaries, tmp_path):
    """An llm.c GPT-2 file whose vocabulary (250) is padded to 256 rows: one rank uses the 250 real rows,
    two tensor-parallel ranks split the 256 padded rows and must keep the padding out of the softmax."""
    from infinitrain_b200.data import write_token_file
    from infinitrain_b200.models import llmc
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel
    from infinitrain_b200.parallel import global_env as genv

    genv.InitAllEnv(world_size=1, rank=0)
    g = torch.Generator().manual_seed(3)
    write_token_file(str(tmp_path / "tokens16.bin"), torch.randint(0, 250, (2 * 64 * 40 + 1,), generator=g).tolist())
    torch.manual_seed(7)
    cfg = TransformerConfig.GPT2(n_layer=2, n_embd=96, n_head=12, n_kv_head=12, vocab_size=250, original_vocab_size=250, block_size=64)
    m = TransformerModel(cfg)
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.1) if p.dim() > 1 else p.add_(torch.randn_like(p) * 0.1)
    llmc.write_gpt2_llmc(str(tmp_path / "gpt2.bin"), cfg, llmc.full_state_dict(m), padded_vocab_size=256)
    one, _ = _train(binaries, tmp_path, "gpt2", 1, *GPT2)
    two, _ = _train(binaries, tmp_path, "gpt2", 2, *GPT2, "--tensor_parallel", "2", "--sequence_parallel")
    assert max(abs(a - b) for a, b in zip(one, two)) <= 2e-5, list(zip(one, two))


def test_gpt2_tensor_and_sequence_parallel_inside_pipeline_stages(binaries, files):
    """GPT-2 (learned positions, biases, LayerNorm) on TP2+SP x PP2 against PP2 alone: both run the untied
    two-stage model, so the trajectories must agree; the position table and the row-parallel biases are
    the parameters whose sequence-parallel gradient sum this exercises."""
    pp, _ = _train(binaries, files, "gpt2", 2, *GPT2, "--pipeline_parallel", "2")
    both, _ = _train(binaries, files, "gpt2", 4, *GPT2, "--pipeline_parallel", "2", "--tensor_parallel", "2", "--sequence_parallel")
    assert max(abs(a - b) for a, b in zip(pp, both)) <= 2e-5, list(zip(pp, both))


def test_ranks_meet_through_a_shared_file_instead_of_a_tcp_store(binaries, files, single, tmp_path):
    """ITB_RDZV_FILE: the job's store is a file every rank can reach (the reference's ranks exchange their
    communicator ids through files too); the endpoint the launcher exports is never contacted."""
    launcher, trainer = binaries
    cmd = [launcher, "--nproc_per_node=2", "--rdzv_endpoint=127.0.0.1:1", "--", trainer, "--family", "llama3", "--device", "cpu",
           "--llmc_filepath", "llama3.bin", "--input_bin", "tokens32.bin", "--batch_size", "2", "--sequence_length", "64",
           "--total_batch_size", "1024", "--num_iteration", "4", "--dtype", "float32", *LLAMA, "--tensor_parallel", "2"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=files,
                       env={**ENV, "ITB_RDZV_FILE": str(tmp_path / "rendezvous")})
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    losses = _losses(r.stdout + r.stderr)
    assert len(losses) == 4 and max(abs(a - b) for a, b in zip(losses, single["llama3"])) <= 2e-5


def _start_ranks(trainer, files, world, extra, env_extra, iters=6):
    """The rank processes started directly (no launcher that would end the survivors itself)."""
    port = _free_port()
    procs = []
    for rank in range(world):
        env = {**ENV, "RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world), "MASTER_ADDR": "127.0.0.1",
               "MASTER_PORT": str(port), **env_extra}
        cmd = [trainer, "--family", "llama3", "--device", "cpu", "--llmc_filepath", "llama3.bin", "--input_bin", "tokens32.bin",
               "--batch_size", "2", "--sequence_length", "64", "--total_batch_size", "1024", "--num_iteration", str(iters),
               "--dtype", "float32", *LLAMA, *extra]
        procs.append(subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=files, env=env))
    return procs


@pytest.mark.parametrize("kind,flags", [("exit", ("--tensor_parallel", "2")), ("mute", ("--zero_stage", "1")),
                                        ("stall:60", ("--pipeline_parallel", "2"))], ids=["exit_tp", "mute_zero1", "stall_pp"])
def test_survivors_of_a_failed_rank_stop_with_a_report_instead_of_waiting(binaries, files, kind, flags):
    """--heartbeat_timeout: rank 1 leaves, falls silent or stalls at step 3 (host-side injection, between
    steps).  Rank 0 sits in a collective that will never complete; its watchdog sees the stale heartbeat,
    aborts the process groups and the rank ends with exit code 75 and a report, within seconds."""
    import time

    _, trainer = binaries
    t0 = time.time()
    # the muted rank goes on training: the run must outlast the watchdog's patience
    procs = _start_ranks(trainer, files, 2, (*flags, "--heartbeat_timeout", "2"), {"ITB_FAULT": f"1:3:{kind}"},
                         iters=200 if kind == "mute" else 6)
    try:
        out0, _ = procs[0].communicate(timeout=120)
    finally:
        for p in procs:                        # the stalled rank is still asleep: end exactly the processes started here
            if p.poll() is None:
                p.kill()
        out1, _ = procs[1].communicate(timeout=30)
    elapsed = time.time() - t0
    if kind == "mute":
        # the muted rank keeps training; the watchdog of rank 0 cannot tell it from a dead one and stops the job
        assert procs[0].returncode == 75 and "stale_heartbeat" in out0, out0[-2000:]
    else:
        assert procs[0].returncode == 75, (procs[0].returncode, out0[-2000:])
        # a rank that waits inside a collective does not beat either: the stalled rank's own watchdog may be the
        # first to call the abort, and rank 0 then reports that request
        want = "rank 0 stops: rank 1: stale_heartbeat" if kind == "exit" else "rank 0 stops: rank 1: "
        assert want in out0, out0[-2000:]
    assert len(_losses(out0 + out1)) >= 2          # steps 1 and 2 were trained before the fault
    if kind == "exit":
        assert procs[1].returncode == 17
    assert elapsed < 60, elapsed


def test_heartbeats_cost_nothing_visible_and_an_unarmed_injector_does_nothing(binaries, files, single):
    losses, _ = _train(binaries, files, "llama3", 2, *LLAMA, "--tensor_parallel", "2", "--heartbeat_timeout", "30")
    assert max(abs(a - b) for a, b in zip(losses, single["llama3"])) <= 2e-5


@pytest.mark.parametrize("old_ranks,new_ranks,flags", [(4, 2, ("--zero_stage", "1")), (2, 4, ("--zero_stage", "2")),
                                                       (4, 8, ("--zero_stage", "1", "--tensor_parallel", "2"))],
                         ids=["zero1_4_to_2", "zero2_2_to_4", "tp2_zero1_dp2_to_dp4"])
def test_elastic_resume_recuts_the_zero_state_for_another_data_parallel_size(binaries, files, tmp_path, old_ranks, new_ranks, flags):
    """--elastic_resume: a ZeRO checkpoint of one data-parallel size continues on another.  The global batch
    of a step is the same token range for both sizes, so the resumed run must follow the uninterrupted one."""
    launcher, trainer = binaries

    def run(ranks, iters, *extra):
        cmd = [launcher, f"--nproc_per_node={ranks}", f"--rdzv_endpoint=127.0.0.1:{_free_port()}", "--", trainer, "--family", "llama3",
               "--device", "cpu", "--llmc_filepath", "llama3.bin", "--input_bin", "tokens32.bin", "--batch_size", "2",
               "--sequence_length", "64", "--total_batch_size", "1024", "--num_iteration", str(iters), "--dtype", "float32", *LLAMA,
               *flags, *extra]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=files, env=ENV)
        return r.returncode, r.stdout + r.stderr

    rc, log = run(old_ranks, 5)
    assert rc == 0, log[-3000:]
    full = _losses(log)
    rc, log = run(old_ranks, 3, "--save", str(tmp_path), "--save_interval", "3")
    assert rc == 0, log[-3000:]
    ckpt = tmp_path / "checkpoint_step_000003"
    assert len(list(ckpt.iterdir())) == old_ranks
    rc, log = run(new_ranks, 5, "--load", str(ckpt))                       # without the flag: refused, with the reason
    assert rc != 0 and "--elastic_resume accepts another data-parallel size" in log, log[-2000:]
    rc, log = run(new_ranks, 5, "--load", str(ckpt), "--elastic_resume")
    assert rc == 0, log[-3000:]
    resumed = _losses(log)
    assert "elastic resume: ZeRO optimizer state" in log
    assert len(resumed) == 2 and max(abs(a - b) for a, b in zip(resumed, full[3:])) <= 2e-5, (resumed, full)


def _read_adapter(path):
    import struct

    import numpy as np

    raw = open(path, "rb").read()
    magic, version, count = struct.unpack_from("<III", raw, 0)
    assert magic == 0x4C4F5241 and version == 1
    at, out = 12, {}
    for _ in range(count):
        (n,) = struct.unpack_from("<I", raw, at)
        name = raw[at + 4:at + 4 + n].decode()
        at += 4 + n
        (ndim,) = struct.unpack_from("<I", raw, at)
        dims = struct.unpack_from(f"<{ndim}q", raw, at + 4)
        at += 4 + 8 * ndim
        size = int(np.prod(dims)) if ndim else 1
        out[name] = np.frombuffer(raw, dtype="<f4", count=size, offset=at).reshape(dims)
        at += 4 * size
    assert at == len(raw)
    return out


def test_one_adapter_file_whatever_the_layout_that_trained_it(binaries, files, tmp_path):
    """--lora_save_path under tensor + pipeline parallelism writes ONE ordinary adapter file (sharded factors
    joined, the fused QKV rows back in Q | K | V order, global layer numbers); it equals the file of the
    one-rank run, and either file loads on either layout and in the Python trainer."""
    import sys

    import numpy as np

    lora = (*LLAMA, "--lora_rank", "4", "--lora_alpha", "8", "--lora_target_modules", "c_attn,c_proj,c_fc,c_fc2")
    layout = ("--tensor_parallel", "2", "--sequence_parallel", "--pipeline_parallel", "2")
    one_file, four_file = str(tmp_path / "one.lora"), str(tmp_path / "four.lora")
    # plain SGD: Adam's normalised steps turn summation-order noise in near-zero gradients into visible differences
    # between layouts, which says nothing about the files
    sgd = ("--optimizer", "sgd", "--learning_rate", "0.5")
    _train(binaries, files, "llama3", 1, *lora, *sgd, "--lora_save_path", one_file, iters=4)
    _train(binaries, files, "llama3", 4, *lora, *layout, *sgd, "--lora_save_path", four_file, iters=4)
    assert not (tmp_path / "four.lora.rank0").exists()
    a, b = _read_adapter(one_file), _read_adapter(four_file)
    assert sorted(a) == sorted(b) and len(a) == 4 * 5 * 2          # 4 layers, 5 adapted linears, two factors each
    assert "transformer.h.3.attn.c_attn.lora_B" in a
    for name in a:
        assert a[name].shape == b[name].shape and np.abs(a[name] - b[name]).max() <= 2e-4, name
    assert max(np.abs(v).max() for k, v in a.items() if k.endswith("lora_B")) > 1e-3      # the adapters did train
    # either file on either layout: the frozen adapters give the same losses
    frozen = ("--learning_rate", "0.0")
    on_one, _ = _train(binaries, files, "llama3", 1, *lora, *frozen, "--lora_load_path", four_file, iters=2)
    on_four, _ = _train(binaries, files, "llama3", 4, *lora, *layout, *frozen, "--lora_load_path", one_file, iters=2)
    plain, _ = _train(binaries, files, "llama3", 1, *lora, *frozen, iters=2)
    assert max(abs(x - y) for x, y in zip(on_one, on_four)) <= 3e-5, (on_one, on_four)
    assert max(abs(x - y) for x, y in zip(on_one, plain)) > 1e-3                          # and they are not the untrained ones
    # the Python trainer reads the file the four C++ ranks wrote
    py = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "llama3", "main.py"), "--device", "cpu", "--llmc_filepath",
                         "llama3.bin", "--input_bin", "tokens32.bin", "--batch_size", "2", "--sequence_length", "64",
                         "--total_batch_size", "1024", "--num_iteration", "2", "--dtype", "float32", *lora, "--learning_rate", "0.0",
                         "--optimizer", "adam", "--lora_load_path", four_file], capture_output=True, text=True, timeout=600, cwd=files,
                        env=ENV)
    assert py.returncode == 0, (py.stdout + py.stderr)[-3000:]
    assert max(abs(x - y) for x, y in zip(_losses(py.stdout + py.stderr), on_one)) <= 3e-5


def test_two_launchers_play_two_nodes(binaries, files, single):
    """Multi-node start: one infini_run per node (--nnodes 2 --node_rank 0|1, two ranks each) against one
    rendezvous endpoint; the four ranks (TP2 x DP2, the tensor-parallel pairs inside a node) follow the
    one-rank trajectory."""
    launcher, trainer = binaries
    port = _free_port()
    cmd = [trainer, "--family", "llama3", "--device", "cpu", "--llmc_filepath", "llama3.bin", "--input_bin", "tokens32.bin",
           "--batch_size", "2", "--sequence_length", "64", "--total_batch_size", "1024", "--num_iteration", "4", "--dtype", "float32",
           *LLAMA, "--tensor_parallel", "2", "--zero_stage", "1"]
    nodes = [subprocess.Popen([launcher, "--nnodes=2", f"--node_rank={n}", "--nproc_per_node=2", f"--rdzv_endpoint=127.0.0.1:{port}",
                               "--", *cmd], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=files, env=ENV)
             for n in (0, 1)]
    outs = [p.communicate(timeout=600)[0] for p in nodes]
    assert all(p.returncode == 0 for p in nodes), outs[0][-2000:] + outs[1][-2000:]
    assert "world_size = 4" in outs[0] and not _losses(outs[0])          # the last rank logs: it lives on node 1
    losses = _losses(outs[1])
    assert len(losses) == 4 and max(abs(a - b) for a, b in zip(losses, single["llama3"])) <= 2e-5


def test_launcher_restarts_a_failed_job_from_its_newest_checkpoint(binaries, files, tmp_path):
    """infini_run --max_restarts: rank 1 leaves at step 4 of the first attempt; the launcher ends rank 0, starts
    both again with ITB_RESTART_COUNT=1, and the trainer goes on from the newest checkpoint every rank has
    (step 2): the job ends with exit code 0 and its last steps repeat the uninterrupted run's."""
    launcher, trainer = binaries
    cmd = [trainer, "--family", "llama3", "--device", "cpu", "--llmc_filepath", "llama3.bin", "--input_bin", "tokens32.bin",
           "--batch_size", "2", "--sequence_length", "64", "--total_batch_size", "1024", "--num_iteration", "6", "--dtype", "float32",
           *LLAMA, "--zero_stage", "1"]
    full, _ = _train(binaries, files, "llama3", 2, *LLAMA, "--zero_stage", "1", iters=6)
    # a fixed port below the range the system hands to outgoing connections: the second attempt listens on port + 1
    r = subprocess.run([launcher, "--nproc_per_node=2", "--max_restarts=1", "--rdzv_endpoint=127.0.0.1:29961", "--", *cmd,
                        "--save", str(tmp_path), "--save_interval", "2"], capture_output=True, text=True, timeout=600, cwd=files,
                       env={**ENV, "ITB_FAULT": "1:4:exit"})
    log = r.stdout + r.stderr
    assert r.returncode == 0, log[-3000:]
    assert "attempt 0 ended with exit code 17; restarting (1 of 1)" in log
    assert "restart 1: resuming from " in log and "checkpoint_step_000002" in log
    steps = [int(m.group(1)) for m in re.finditer(r"step\s+(\d+)/6", log)]
    assert steps == [1, 2, 3, 3, 4, 5, 6], steps
    losses = _losses(log)
    assert max(abs(a - b) for a, b in zip(losses[3:], full[2:])) <= 2e-5, (losses, full)
    # without restarts left the failure is the job's exit code
    r = subprocess.run([launcher, "--nproc_per_node=2", f"--rdzv_endpoint=127.0.0.1:{_free_port()}", "--", *cmd], capture_output=True,
                       text=True, timeout=600, cwd=files, env={**ENV, "ITB_FAULT": "1:2:exit:9"})
    assert r.returncode == 9


def test_data_parallel_ranks_of_a_model_parallel_job_resume_from_their_groups_first_rank(binaries, files, tmp_path):
    """TP2 x DP2 without ZeRO: only data-parallel rank 0 of every tensor-parallel slice saves; on resume the
    other data-parallel ranks read that slice too, and the run continues the uninterrupted one."""
    flags = (*LLAMA, "--tensor_parallel", "2")
    full, _ = _train(binaries, files, "llama3", 4, *flags, iters=4)
    _train(binaries, files, "llama3", 4, *flags, "--save", str(tmp_path), "--save_interval", "2", iters=2)
    ckpt = tmp_path / "checkpoint_step_000002"
    assert sorted(p.name for p in ckpt.iterdir()) == ["rank_000000", "rank_000001"]
    launcher, trainer = binaries
    r = subprocess.run([launcher, "--nproc_per_node=4", f"--rdzv_endpoint=127.0.0.1:{_free_port()}", "--", trainer, "--family", "llama3",
                        "--device", "cpu", "--llmc_filepath", "llama3.bin", "--input_bin", "tokens32.bin", "--batch_size", "2",
                        "--sequence_length", "64", "--total_batch_size", "1024", "--num_iteration", "4", "--dtype", "float32", *flags,
                        "--load", str(ckpt)], capture_output=True, text=True, timeout=600, cwd=files, env=ENV)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    resumed = _losses(r.stdout + r.stderr)
    assert len(resumed) == 2 and max(abs(a - b) for a, b in zip(resumed, full[2:])) <= 2e-5, (resumed, full)
