"""Example trainers end to end on CPU (tiny configs), the C++ launcher, and hybrid parallel runs."""
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(cmd, env=None, timeout=600):
    e = dict(os.environ)
    e.update(env or {})
    e["OMP_NUM_THREADS"] = "1"
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return r.stdout + r.stderr


def _losses(out):
    return [float(m.group(2)) for m in re.finditer(r"step\s+(\d+)/\d+\s+\|\s+train loss\s+([\d.]+)", out)]


def test_mnist_trains():
    out = _run([sys.executable, "examples/mnist/main.py", "--num_epoch", "1"])
    assert "final loss" in out


def test_gpt2_single_process_cpu(tmp_path):
    out = _run([sys.executable, "examples/gpt2/main.py", "--device", "cpu", "--n_layer", "2", "--n_embd", "64", "--n_head", "4", "--vocab_size", "512",
                "--batch_size", "2",
                "--sequence_length", "32", "--total_batch_size", "128", "--num_iteration", "3", "--optimizer", "adam",
                "--learning_rate", "1e-3", "--overfit_single_batch", "--save", str(tmp_path), "--save_interval", "3",
                "--metrics_jsonl", str(tmp_path / "metrics.jsonl")])
    l = _losses(out)
    assert len(l) == 3 and l[-1] < l[0]
    import json

    recs = [json.loads(line) for line in open(tmp_path / "metrics.jsonl")]
    assert [r["step"] for r in recs] == [1, 2, 3] and abs(recs[2]["loss"] - l[2]) < 1e-5 and recs[0]["tokens_per_s"] > 0
    assert os.path.exists(os.path.join(tmp_path, "checkpoint_step_000003", "model.ckpt"))


def _launcher():
    from infinitrain_b200 import _ext

    p = _ext.launcher_path()
    if not p.exists():
        _ext.build_launcher()
    return str(p)


@pytest.mark.parametrize("flags", [
    ["--tensor_parallel", "2", "--sequence_parallel"],
    ["--pipeline_parallel", "2", "--virtual_pipeline_parallel", "2"],
    ["--zero_stage", "1"],
])
def test_llama3_two_ranks_via_launcher(flags):
    port = 29600 + abs(hash(tuple(flags))) % 300
    out = _run([_launcher(), "--nproc_per_node=2", f"--rdzv_endpoint=127.0.0.1:{port}", "--", sys.executable,
                "examples/llama3/main.py", "--device", "cpu", "--n_layer", "4", "--n_embd", "64", "--n_head", "4",
                "--n_kv_head", "2", "--vocab_size", "512", "--batch_size", "2",
                "--sequence_length", "32", "--total_batch_size", "256", "--num_iteration", "2", "--model", "llama3-1b",
                "--overfit_single_batch", "--learning_rate", "1e-3", *flags], timeout=900)
    l = _losses(out)
    assert len(l) == 2 and l[1] < l[0] + 1e-3, out[-1500:]


def test_trainer_stops_when_a_peer_is_lost():
    """Two data-parallel CPU ranks; rank 1 stops making progress between steps (host-side injected
    stall, far longer than the heartbeat limit).  Rank 0's heartbeat check notices before the next
    collective and stops with exit code 75 instead of waiting inside it."""
    import time

    port = 29950
    cmd = [_launcher(), "--nproc_per_node=2", f"--rdzv_endpoint=127.0.0.1:{port}", "--", sys.executable,
           "examples/llama3/main.py", "--device", "cpu", "--n_layer", "2", "--n_embd", "64", "--n_head", "4",
           "--n_kv_head", "2", "--vocab_size", "512", "--batch_size", "2", "--sequence_length", "32",
           "--total_batch_size", "128", "--num_iteration", "6", "--model", "llama3-1b", "--overfit_single_batch",
           "--learning_rate", "1e-3", "--heartbeat_timeout", "3"]
    e = dict(os.environ)
    e.update(OMP_NUM_THREADS="1", ITB_FAULT="1:3:stall:120")
    t0 = time.time()
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=e, cwd=ROOT)
    out = r.stdout + r.stderr
    assert time.time() - t0 < 200
    assert r.returncode != 0
    assert "peer failure detected at step 3" in out, out[-2000:]
    assert len(_losses(out)) == 2          # two steps completed before the fault


def test_elastic_resume_on_fewer_ranks(tmp_path):
    """ZeRO-1 training saved by 4 data-parallel CPU ranks resumes on 2: weights are reloaded, the
    sharded Adam state is re-sharded, training continues from the saved step."""
    common = [sys.executable, "examples/llama3/main.py", "--device", "cpu", "--n_layer", "2", "--n_embd", "64",
              "--n_head", "4", "--n_kv_head", "2", "--vocab_size", "512", "--batch_size", "2", "--sequence_length", "32",
              "--model", "llama3-1b", "--overfit_single_batch", "--learning_rate", "1e-3", "--zero_stage", "1",
              "--save_optimizer_state"]
    out = _run([_launcher(), "--nproc_per_node=4", "--rdzv_endpoint=127.0.0.1:29921", "--", *common,
                "--total_batch_size", "256", "--num_iteration", "2", "--save", str(tmp_path), "--save_interval", "2"],
               timeout=900)
    first = _losses(out)
    ckpt = os.path.join(tmp_path, "checkpoint_step_000002")
    assert len(first) == 2 and sorted(os.listdir(ckpt)) == [f"rank_{r:06d}" for r in range(4)]
    out = _run([_launcher(), "--nproc_per_node=2", "--rdzv_endpoint=127.0.0.1:29922", "--", *common,
                "--total_batch_size", "128", "--num_iteration", "4", "--load", ckpt, "--elastic_resume"], timeout=900)
    resumed = _losses(out)
    assert len(resumed) == 2, out[-1500:]                      # steps 3 and 4 only
    assert all(v == v for v in resumed) and resumed[-1] < first[0]
    # without the flag the topology check refuses
    r = subprocess.run([_launcher(), "--nproc_per_node=2", "--rdzv_endpoint=127.0.0.1:29923", "--", *common,
                        "--total_batch_size", "128", "--num_iteration", "4", "--load", ckpt], capture_output=True,
                       text=True, timeout=900, cwd=ROOT, env={**os.environ, "OMP_NUM_THREADS": "1"})
    assert r.returncode != 0


def test_elastic_resume_under_tensor_parallelism_follows_the_uninterrupted_run(tmp_path):
    """TP2 x DP2 with ZeRO-1 saves after step 2; TP2 x DP4 resumes with --elastic_resume.  A step's global
    batch is the same token range under both sizes, so steps 3 and 4 must repeat the uninterrupted run's."""
    import torch

    from infinitrain_b200.data import write_token_file

    g = torch.Generator().manual_seed(3)
    write_token_file(str(tmp_path / "tokens.bin"), torch.randint(0, 512, (2 * 32 * 80 + 1,), generator=g).tolist(), llama3=True)
    common = [sys.executable, "examples/llama3/main.py", "--device", "cpu", "--n_layer", "2", "--n_embd", "64", "--n_head", "4",
              "--n_kv_head", "2", "--vocab_size", "512", "--batch_size", "2", "--sequence_length", "32", "--model", "llama3-1b",
              "--input_bin", str(tmp_path / "tokens.bin"), "--learning_rate", "1e-2", "--zero_stage", "1", "--tensor_parallel", "2",
              "--save_optimizer_state", "--total_batch_size", "512"]

    def run(ranks, port, *extra):
        return _losses(_run([_launcher(), f"--nproc_per_node={ranks}", f"--rdzv_endpoint=127.0.0.1:{port}", "--", *common, *extra],
                            timeout=900))

    full = run(4, 29931, "--num_iteration", "4")
    first = run(4, 29932, "--num_iteration", "2", "--save", str(tmp_path / "ck"), "--save_interval", "2")
    ckpt = os.path.join(tmp_path, "ck", "checkpoint_step_000002")
    assert first == full[:2] and len(os.listdir(ckpt)) == 4
    resumed = run(8, 29933, "--num_iteration", "4", "--load", ckpt, "--elastic_resume")
    assert len(resumed) == 2 and max(abs(a - b) for a, b in zip(resumed, full[2:])) <= 2e-5, (resumed, full)


def test_run_matrix_and_compare(tmp_path):
    """The configuration-matrix runner writes one log per run; comparing a matrix against itself
    passes (same seeds, deterministic CPU math)."""
    a, b = tmp_path / "a", tmp_path / "b"
    # timings of such tiny CPU runs are noise: only the losses are held to their tolerance here
    for out, extra in ((a, []), (b, ["--compare", str(a), "--tps-band", "100"])):
        _run([sys.executable, "examples/common/run_matrix.py", "examples/common/matrix_smoke.json", "--out", str(out),
              "--only", "1,1_bfloat16,zero1", "--port", "29760", *extra], timeout=900)
    assert sorted(os.listdir(a)) == ["gpt2_1.log", "gpt2_1_bfloat16.log", "llama3_zero1.log"]
    assert len(_losses(open(a / "llama3_zero1.log").read())) == 3


def test_run_matrix_through_the_cpp_trainer(tmp_path):
    """--frontend cpp: the same matrix file drives the C++ trainer (from-scratch model of the matrix's shape,
    synthetic tokens); its logs carry the step line the comparison tools read."""
    out = _run([sys.executable, "examples/common/run_matrix.py", "examples/common/matrix_smoke.json", "--out", str(tmp_path / "dry"),
                "--frontend", "cpp", "--dry-run"], timeout=900)
    lines = [ln for ln in out.splitlines() if "itb_train" in ln]
    assert len(lines) == 4 and all("--family" in ln for ln in lines) and sum("infini_run" in ln for ln in lines) == 2
    _run([sys.executable, "examples/common/run_matrix.py", "examples/common/matrix_smoke.json", "--out", str(tmp_path / "run"),
          "--frontend", "cpp", "--only", "1,zero1", "--port", "29790"], timeout=900)
    assert len(_losses(open(tmp_path / "run" / "gpt2_1.log").read())) == 3
    zero1 = _losses(open(tmp_path / "run" / "llama3_zero1.log").read())
    assert len(zero1) == 3 and zero1[-1] < zero1[0]


def test_validation_loss_is_logged(tmp_path):
    import torch

    from infinitrain_b200.data import write_token_file

    g = torch.Generator().manual_seed(3)
    val = str(tmp_path / "val.bin")
    write_token_file(val, torch.randint(0, 512, (2 * 32 * 6 + 1,), generator=g).tolist())
    out = _run([sys.executable, "examples/gpt2/main.py", "--device", "cpu", "--n_layer", "2", "--n_embd", "64", "--n_head", "4",
                "--vocab_size", "512", "--batch_size", "2", "--sequence_length", "32", "--total_batch_size", "64",
                "--num_iteration", "5", "--optimizer", "adam", "--learning_rate", "1e-3", "--input_val_bin", val,
                "--val_loss_every", "2", "--val_max_batches", "4"])
    vals = [(int(m.group(1)), float(m.group(2))) for m in re.finditer(r"step\s+(\d+)/5 \| val loss ([\d.]+) \(4 batches\)", out)]
    assert [s for s, _ in vals] == [2, 4, 5] and all(5.0 < v < 8.0 for _, v in vals)
    assert len(_losses(out)) == 5                     # the train-loss parser does not pick the validation lines up


def test_ddp_with_gradient_accumulation_equals_one_rank(tmp_path):
    """Two data-parallel ranks with two micro-batches each see the same four batches per step as one
    rank with four micro-batches: the loss trajectories must coincide (gradients of the micro-batches
    that ran under no_sync are part of the bucket that gets averaged)."""
    import torch

    from infinitrain_b200.data import write_token_file

    g = torch.Generator().manual_seed(4)
    data = str(tmp_path / "train.bin")
    write_token_file(data, torch.randint(0, 512, (2 * 32 * 24 + 1,), generator=g).tolist())
    common = ["examples/gpt2/main.py", "--device", "cpu", "--n_layer", "2", "--n_embd", "64", "--n_head", "4",
              "--vocab_size", "512", "--batch_size", "2", "--sequence_length", "32", "--total_batch_size", "256",
              "--num_iteration", "4", "--optimizer", "sgd", "--learning_rate", "0.5", "--input_bin", data, "--seed", "7"]
    one = _losses(_run([sys.executable, *common]))
    two = _losses(_run([_launcher(), "--nproc_per_node=2", "--rdzv_endpoint=127.0.0.1:29927", "--", sys.executable, *common]))
    assert len(one) == 4 and len(two) == 4
    assert max(abs(a - b) for a, b in zip(one, two)) <= 2e-5, list(zip(one, two))
    assert abs(one[0] - one[-1]) > 1e-3


@pytest.fixture(scope="module")
def llama_files(tmp_path_factory):
    import torch

    from infinitrain_b200.data import write_token_file
    from infinitrain_b200.models import llmc
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel
    from infinitrain_b200.parallel import global_env as genv

    d = tmp_path_factory.mktemp("hybrid")
    genv.InitAllEnv(world_size=1, rank=0)
    cfg = TransformerConfig.LLaMA3(n_layer=4, n_embd=64, n_head=4, n_kv_head=2, vocab_size=256, original_vocab_size=256,
                                   block_size=64, multiple_of=16, ffn_dim_multiplier=1.5)
    torch.manual_seed(42)
    m = TransformerModel(cfg)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() > 1:
                p.normal_(0, 0.1)
    llmc.write_llama3_llmc(str(d / "l4.bin"), cfg, llmc.full_state_dict(m))
    g = torch.Generator().manual_seed(1)
    write_token_file(str(d / "tok.bin"), torch.randint(0, 256, (4 * 64 * 30 + 1,), generator=g).tolist(), llama3=True)
    common = ["examples/llama3/main.py", "--device", "cpu", "--llmc_filepath", str(d / "l4.bin"), "--input_bin", str(d / "tok.bin"),
              "--batch_size", "2", "--sequence_length", "64", "--total_batch_size", "512", "--num_iteration", "3",
              "--dtype", "float32", "--learning_rate", "0.05", "--optimizer", "sgd"]
    return common, _losses(_run([sys.executable, *common]))


@pytest.mark.parametrize("ranks,flags", [
    (4, ["--tensor_parallel", "2", "--sequence_parallel", "--zero_stage", "2"]),
    (4, ["--tensor_parallel", "2", "--sequence_parallel", "--pipeline_parallel", "2"]),
    (8, ["--tensor_parallel", "2", "--sequence_parallel", "--pipeline_parallel", "2", "--virtual_pipeline_parallel", "2",
         "--zero_stage", "2"]),
])
def test_hybrid_parallel_runs_follow_the_one_rank_trajectory(llama_files, ranks, flags):
    """DP x TP+SP x PP (x vPP, ZeRO) on CPU ranks against ONE rank on the same weights and the same
    global batch: the same losses step by step.  Catches gradients that a parallel mode loses or
    counts twice (sequence-parallel-replicated parameters under ZeRO-2 or inside a pipeline stage)."""
    common, one = llama_files
    port = 29940 + ranks + len(flags)
    out = _run([_launcher(), f"--nproc_per_node={ranks}", f"--rdzv_endpoint=127.0.0.1:{port}", "--", sys.executable, *common,
                *flags], timeout=900)
    got = _losses(out)
    assert len(one) == 3 and len(got) == 3
    assert max(abs(a - b) for a, b in zip(one, got)) <= 2e-5, list(zip(one, got))
    assert abs(one[0] - one[1]) > 1e-2


def test_launcher_restarts_a_failed_job_from_its_newest_checkpoint(llama_files, tmp_path):
    """infini_run --max_restarts with the Python trainer: rank 1 leaves at step 4 of the first attempt; both ranks
    are started again with ITB_RESTART_COUNT=1 and go on from the newest checkpoint every rank has (step 2): the
    job ends with exit code 0 and its last steps repeat the uninterrupted run's."""
    common, _ = llama_files
    six = list(common)
    six[six.index("--num_iteration") + 1] = "6"
    flags = ["--zero_stage", "1", "--optimizer", "adam", "--learning_rate", "0.01", "--save_optimizer_state"]
    full = _losses(_run([_launcher(), "--nproc_per_node=2", "--rdzv_endpoint=127.0.0.1:29941", "--", sys.executable, *six, *flags],
                        timeout=900))
    # a fixed port below the range the system hands to outgoing connections: the second attempt listens on port + 1
    out = _run([_launcher(), "--nproc_per_node=2", "--max_restarts=1", "--rdzv_endpoint=127.0.0.1:29945", "--", sys.executable, *six,
                *flags, "--save", str(tmp_path), "--save_interval", "2"], env={"ITB_FAULT": "1:4:exit"}, timeout=900)
    assert "attempt 0 ended with exit code 17; restarting (1 of 1)" in out
    assert "restart 1: resuming from " in out and "checkpoint_step_000002" in out
    steps = [int(m.group(1)) for m in re.finditer(r"step\s+(\d+)/6", out)]
    assert steps == [1, 2, 3, 3, 4, 5, 6], steps
    got = _losses(out)
    assert max(abs(a - b) for a, b in zip(got[3:], full[2:])) <= 2e-5, (got, full)


def test_two_launchers_play_two_nodes(llama_files):
    """One infini_run per node (--nnodes 2 --node_rank 0|1, two ranks each) against one rendezvous endpoint:
    the four gloo ranks (TP2 x DP2 with ZeRO-1) follow the one-rank trajectory."""
    import socket

    common, one = llama_files
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    env = {**os.environ, "OMP_NUM_THREADS": "1"}
    nodes = [subprocess.Popen([_launcher(), "--nnodes=2", f"--node_rank={n}", "--nproc_per_node=2",
                               f"--rdzv_endpoint=127.0.0.1:{port}", "--", sys.executable, *common, "--tensor_parallel", "2",
                               "--zero_stage", "1"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=ROOT, env=env)
             for n in (0, 1)]
    outs = [p.communicate(timeout=900)[0] for p in nodes]
    assert all(p.returncode == 0 for p in nodes), outs[0][-2000:] + outs[1][-2000:]
    got = _losses(outs[1])                                   # the last rank logs: it lives on node 1
    assert len(got) == 3 and not _losses(outs[0])
    assert max(abs(a - b) for a, b in zip(got, one)) <= 2e-5, list(zip(got, one))


@pytest.mark.parametrize("ranks,flags", [
    (2, ["--tensor_parallel", "2"]),
    (8, ["--tensor_parallel", "2", "--sequence_parallel", "--pipeline_parallel", "2", "--virtual_pipeline_parallel", "2",
         "--zero_stage", "2"]),
])
def test_lora_in_any_layout_follows_the_one_rank_run_and_writes_the_same_adapter(llama_files, tmp_path, ranks, flags):
    """One whole-model adapter file goes into a one-rank run and into a model-parallel run: the same
    losses, and the adapter gathered from the parallel ranks equals the one-rank result (sharded LoRA
    factors re-assembled, the replicated ones' partial gradients summed over the tensor-parallel group,
    a stage's local layer numbers made global)."""
    import torch

    from infinitrain_b200.nn.lora.lora_utils import _read_lora_file

    common, _ = llama_files
    lora_flags = ["--lora_rank", "4", "--lora_alpha", "8", "--lora_target_modules", "c_attn,c_proj,c_fc,c_fc2"]
    start, one_out, par_out = (str(tmp_path / n) for n in ("start.bin", "one.bin", "par.bin"))
    two_steps = list(common)
    two_steps[two_steps.index("--num_iteration") + 1] = "2"
    _run([sys.executable, *two_steps, *lora_flags, "--lora_save_path", start])      # B leaves zero after a step
    one = _losses(_run([sys.executable, *common, *lora_flags, "--lora_load_path", start, "--lora_save_path", one_out]))
    out = _run([_launcher(), f"--nproc_per_node={ranks}", f"--rdzv_endpoint=127.0.0.1:{29970 + ranks}", "--",
                sys.executable, *common, *lora_flags, *flags, "--lora_load_path", start, "--lora_save_path", par_out,
                "--lora_merge_check"], timeout=900)
    par = _losses(out)
    if "--pipeline_parallel" not in flags:           # merged == unmerged == unmerged again, on sharded factors too
        assert re.search(r"lora merge check: .* ok", out) and "MISMATCH" not in out
    assert len(one) == 3 and max(abs(a - b) for a, b in zip(one, par)) <= 2e-6, list(zip(one, par))
    a, b, c = _read_lora_file(one_out), _read_lora_file(par_out), _read_lora_file(start)
    assert sorted(a) == sorted(b) and len(a) == 4 * 5 * 2
    assert max(float((a[k] - b[k]).abs().max()) for k in a) < 1e-6
    assert max(float((a[k] - c[k]).abs().max()) for k in a) > 1e-4        # and training moved them


def test_fresh_adapters_do_not_depend_on_the_layout(llama_files, tmp_path):
    """No adapter file to start from: every adapter draws its A factor from a generator keyed by its
    whole-model path (row-parallel factors at their unsharded shape), so one rank and TP2+SP x PP2 start from
    the same adapters, follow the same losses and write the same adapter file."""
    from infinitrain_b200.nn.lora.lora_utils import _read_lora_file

    common, _ = llama_files
    lora_flags = ["--lora_rank", "4", "--lora_alpha", "8", "--lora_target_modules", "c_attn,c_proj,c_fc,c_fc2", "--learning_rate", "0.5"]
    one_out, par_out = str(tmp_path / "one.bin"), str(tmp_path / "par.bin")
    one = _losses(_run([sys.executable, *common, *lora_flags, "--lora_save_path", one_out]))
    par = _losses(_run([_launcher(), "--nproc_per_node=4", "--rdzv_endpoint=127.0.0.1:29981", "--", sys.executable, *common,
                        *lora_flags, "--tensor_parallel", "2", "--sequence_parallel", "--pipeline_parallel", "2", "--lora_save_path",
                        par_out], timeout=900))
    assert len(one) == 3 and max(abs(a - b) for a, b in zip(one, par)) <= 2e-5, list(zip(one, par))
    a, b = _read_lora_file(one_out), _read_lora_file(par_out)
    assert sorted(a) == sorted(b) and len(a) == 4 * 5 * 2
    assert max(float((a[k] - b[k]).abs().max()) for k in a) < 2e-4
    assert max(float(a[k].abs().max()) for k in a if k.endswith("lora_B")) > 1e-3          # B left zero: they trained


def test_gpu_regression_matrix_expands_to_the_references_runs(tmp_path):
    """examples/common/matrix_gpu.json is the reference's scripts/test_config.json (groups basic, zero,
    lora) for both model families and both dtypes; --dry-run prints the command of every run, --profile
    adds the second pass with the profiler on."""
    import json
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = json.load(open(os.path.join(root, "examples", "common", "matrix_gpu.json")))
    ids = {r["id"] for r in spec["runs"]}
    for want in ("1", "2_bfloat16", "3", "4", "5_bfloat16", "6", "7", "8", "3_zero1", "3_zero2", "8_zero2", "lora_3", "lora_5"):
        assert want in ids, want
    eight = next(r for r in spec["runs"] if r["id"] == "8" and r["family"] == "llama3")
    assert eight["nproc"] == 8 and eight["args"]["tensor_parallel"] == 2 and eight["args"]["virtual_pipeline_parallel"] == 2
    r = subprocess.run([sys.executable, os.path.join(root, "examples", "common", "run_matrix.py"),
                        os.path.join(root, "examples", "common", "matrix_gpu.json"), "--out", str(tmp_path), "--dry-run", "--profile"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 2 * len(spec["runs"])
    assert sum("--profile" in ln for ln in lines) == len(spec["runs"])
    assert any("--nproc_per_node=8" in ln and "--pipeline_parallel 8" in ln for ln in lines)
