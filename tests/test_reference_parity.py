"""Parity with the UNMODIFIED reference, both sides on CPU in fp32.

The reference's stock GPT-2 trainer (its ``USE_CUDA=OFF`` build, ``baseline/build_reference.py
--cpu-only``) and this framework's trainer read the same llm.c weight file and the same token file
and take the same SGD steps; per-step losses must agree within the reference's own fp32 tolerance
of 1e-5 (its scripts/compare_loss.py:20,56-57).  The same pair of programs exchanges LoRA adapter
files and checkpoints."""
import os
import re
import shutil
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "baseline", "_ref", "bin", "gpt2_cpu")
# the reference checkout: ITB_REFERENCE_SRC, else a directory named "reference" beside this repository
SRC = os.environ.get("ITB_REFERENCE_SRC") or os.path.join(os.path.dirname(ROOT), "reference")
OURS = [sys.executable, os.path.join(ROOT, "examples", "gpt2", "main.py")]


def _losses(text):
    return [float(m.group(1)) for m in re.finditer(r"step\s+\d+/\d+\s+\|\s+train loss\s+([\d.]+)", text)]


def _run(cmd, cwd):
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=cwd)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return _losses(r.stdout + r.stderr)


def _close(a, b, n):
    assert len(a) == n and len(b) == n, (a, b)
    assert max(abs(x - y) for x, y in zip(a, b)) <= 1e-5, list(zip(a, b))


@pytest.fixture(scope="module")
def world(tmp_path_factory):
    """Reference binary, a 2-layer GPT-2 llm.c file and a token file, shared by the tests below."""
    if not os.path.exists(BIN):
        if not os.path.isdir(os.path.join(SRC, "infini_train")):
            pytest.skip("no reference checkout to build the CPU-only trainer from")
        r = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "build_reference.py"), "--cpu-only", "--src", SRC],
                           capture_output=True, text=True, timeout=1500)
        assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    from infinitrain_b200.data import write_token_file
    from infinitrain_b200.models import llmc
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel
    from infinitrain_b200.parallel import global_env as genv

    d = tmp_path_factory.mktemp("parity")
    genv.InitAllEnv(world_size=1, rank=0)
    # 12 heads: the reference's llm.c loader keeps n_kv_head = 12 whatever the file says
    # (example/gpt2/checkpoint_loader.cc:81-89) and its config check wants n_kv_head == n_head.
    cfg = TransformerConfig.GPT2(n_layer=2, n_embd=96, n_head=12, n_kv_head=12, vocab_size=256, original_vocab_size=256,
                                 block_size=64)
    torch.manual_seed(42)
    m = TransformerModel(cfg)
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.1)
    llmc.write_gpt2_llmc(str(d / "model.bin"), cfg, llmc.full_state_dict(m))
    g = torch.Generator().manual_seed(1)
    write_token_file(str(d / "tokens.bin"), torch.randint(0, 256, (4 * 64 * 16 + 1,), generator=g).tolist())
    common = ["--device", "cpu", "--llmc_filepath", "model.bin", "--input_bin", "tokens.bin", "--batch_size", "4",
              "--sequence_length", "64", "--dtype", "float32", "--learning_rate", "0.05"]
    return d, common


def test_gpt2_sgd_trajectory_equals_the_reference(world):
    d, common = world
    args = [*common, "--total_batch_size", "256", "--num_iteration", "10"]
    a = _run([BIN, *args, "--overfit_single_batch=false"], d)
    b = _run([*OURS, *args, "--optimizer", "sgd"], d)
    _close(a, b, 10)
    assert abs(a[0] - a[-1]) > 1e-3


def test_gradient_accumulation_trajectory_equals_the_reference(world):
    d, common = world
    args = [*common, "--total_batch_size", "512", "--num_iteration", "6"]          # two micro-batches per step
    _close(_run([BIN, *args, "--overfit_single_batch=false"], d), _run([*OURS, *args, "--optimizer", "sgd"], d), 6)


def test_lora_adapter_file_and_training_match_the_reference(world):
    """An adapter file written here is read by the reference; both train the adapters (base frozen)
    along the same trajectory and write adapter files with the same tensors."""
    from infinitrain_b200.models import llmc
    from infinitrain_b200.nn import lora

    d, common = world
    lcfg = lora.LoRAConfig(rank=4, alpha=8.0, target_modules=lora.ParseLoRATargetModules("c_attn,c_proj"))

    def adapters(path=None):
        m = lora.GetLoRAModel(llmc.GPT2FromLLMC(str(d / "model.bin")), lcfg)
        if path:
            lora.LoadLoRAWeights(m, str(d / path))
        return m

    m = adapters()
    torch.manual_seed(7)
    with torch.no_grad():
        for p in lora.GetLoRAParameters(m):
            p.normal_(0, 0.3)              # B starts at zero by default; give both factors weight
    lora.SaveLoRAWeights(m, str(d / "adapter.bin"))
    args = [*common, "--total_batch_size", "256", "--num_iteration", "6", "--lora_rank", "4", "--lora_alpha", "8",
            "--lora_load_path", "adapter.bin"]
    a = _run([BIN, *args, "--overfit_single_batch=false", "--lora_save_path", "ref_adapter.bin"], d)
    b = _run([*OURS, *args, "--optimizer", "sgd", "--lora_save_path", "our_adapter.bin"], d)
    _close(a, b, 6)
    ra, oa, ia = ({k: v.detach() for k, v in lora.LoRAStateDict(adapters(p)).items()} for p in ("ref_adapter.bin", "our_adapter.bin", "adapter.bin"))
    assert max(float((ra[k] - oa[k]).abs().max()) for k in ra) < 1e-6
    assert max(float((ra[k] - ia[k]).abs().max()) for k in ra) > 1e-5        # and they did train


def test_resume_from_a_checkpoint_written_by_the_reference(world):
    from infinitrain_b200.checkpoint.checkpoint import Checkpoint

    d, common = world
    args = [*common, "--total_batch_size", "256", "--num_iteration", "8"]
    a = _run([BIN, *args, "--overfit_single_batch=false", "--save", "ref_ckpt", "--save_interval", "4"], d)
    ck = d / "ref_ckpt" / "checkpoint_step_000004"
    st = Checkpoint.LoadTrainerState(str(ck / "trainer_state.json"))       # the file lacks a comma after vocab_size
    assert (st.global_step, st.consumed_batches) == (4, 4)
    # The stock trainer records its DEFAULT model shape (12 layers, 768 wide) when the weights came
    # from an llm.c file (example/gpt2/main.cc:213-216,365-375); put the file's real shape there.
    assert st.n_layer == 12
    text = (ck / "trainer_state.json").read_text()
    text = text.replace('"n_layer": 12', '"n_layer": 2').replace('"n_embd": 768', '"n_embd": 96')
    (ck / "trainer_state.json").write_text(text.replace('"vocab_size": 50304', '"vocab_size": 256'))
    b = _run([*OURS, *args, "--optimizer", "sgd", "--load", str(ck)], d)
    _close(a[4:], b, 4)
    shutil.rmtree(d / "ref_ckpt")


def test_per_module_dumps_line_up_with_the_reference(world):
    """With the precision checker on, both trainers log one record per module call under the same
    names and dump the same .npy files; every forward output and every backward gradient agrees
    within the reference's own comparison rule (allclose, atol 1e-5, rtol 1e-3)."""
    import glob
    import importlib.util

    d, common = world
    args = [*common, "--total_batch_size", "512", "--num_iteration", "2"]
    _run([BIN, *args, "--overfit_single_batch=false", "--precision_check",
          "level=1,format=simple,path=pc_ref,save_tensors=true"], d)
    _run([*OURS, *args, "--optimizer", "sgd", "--precision_check", "level=1,format=simple,path=pc_ours,save_tensors=true"], d)
    (ref_dir,), (our_dir,) = glob.glob(str(d / "pc_ref" / "*")), glob.glob(str(d / "pc_ours" / "*"))

    def names(run):
        return [ln.split()[2] for ln in open(os.path.join(run, "precision_check_rank_0.log"))]

    a, b = names(ref_dir), names(our_dir)
    assert len(a) == len(b) > 200
    assert sorted(a) == sorted(b)                        # same records; only the two embedding tables' backward order differs
    assert [n for n in a if n.endswith("_forward")] == [n for n in b if n.endswith("_forward")]
    assert sorted(os.listdir(os.path.join(ref_dir, "rank_0"))) == sorted(os.listdir(os.path.join(our_dir, "rank_0")))
    spec = importlib.util.spec_from_file_location("compare_precision",
                                                  os.path.join(ROOT, "examples", "common", "compare_precision.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.main([ref_dir, our_dir]) == 0
    theirs = os.path.join(SRC, "scripts", "precision_check", "precision_compare.py")
    if os.path.exists(theirs):          # and the reference's own comparison tool says the same
        r = subprocess.run([sys.executable, theirs, "--dir1", ref_dir, "--dir2", our_dir], capture_output=True, text=True,
                           timeout=300)
        assert r.returncode == 0 and " 0 failed, 0 errors" in r.stdout, r.stdout[-1500:]
        assert "Missing: 0 in dir1 only, 0 in dir2 only" in r.stdout


def test_reference_regression_script_accepts_our_log(world, tmp_path):
    """The reference's own scripts/compare_loss.py, given a log directory written by its trainer and
    one written by ours (same file names, same step-line format), finds no loss mismatch."""
    script = os.path.join(SRC, "scripts", "compare_loss.py")
    if not os.path.exists(script):
        pytest.skip("no reference checkout with scripts/compare_loss.py")
    d, common = world
    args = [*common, "--total_batch_size", "256", "--num_iteration", "6"]
    for name, cmd in (("ref", [BIN, *args, "--overfit_single_batch=false"]), ("ours", [*OURS, *args, "--optimizer", "sgd"])):
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=d)
        assert r.returncode == 0, r.stderr[-2000:]
        (tmp_path / name).mkdir()
        (tmp_path / name / "gpt2_1.log").write_text(r.stdout + r.stderr)
    r = subprocess.run([sys.executable, script, str(tmp_path / "ref"), str(tmp_path / "ours")], capture_output=True,
                       text=True, timeout=120, cwd=os.path.dirname(script))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "gpt2_1" in r.stdout or "1/1" in r.stdout or "passed" in r.stdout.lower(), r.stdout


def test_reference_resumes_from_a_checkpoint_written_here(world):
    """The other direction: a checkpoint written here with --save_reference_buffers (the causal-mask
    buffers the reference's strict loader wants) is resumed by the reference's trainer, which then
    follows its own uninterrupted trajectory."""
    d, common = world
    args = [*common, "--total_batch_size", "256", "--num_iteration", "8"]
    whole = _run([BIN, *args, "--overfit_single_batch=false"], d)
    first = [*common, "--total_batch_size", "256", "--num_iteration", "4"]
    _run([*OURS, *first, "--optimizer", "sgd", "--save", "our_ckpt", "--save_interval", "4", "--save_reference_buffers"], d)
    ck = d / "our_ckpt" / "checkpoint_step_000004"
    # The stock trainer validates against its DEFAULT model shape when the weights come from an llm.c
    # file (example/gpt2/main.cc:213-216 keeps model_config at GPT2Config()): record that shape.
    text = (ck / "trainer_state.json").read_text()
    text = text.replace('"n_layer": 2', '"n_layer": 12').replace('"n_embd": 96', '"n_embd": 768')
    (ck / "trainer_state.json").write_text(text.replace('"vocab_size": 256', '"vocab_size": 50304'))
    resumed = _run([BIN, *args, "--overfit_single_batch=false", "--load", str(ck)], d)
    _close(whole[4:], resumed, 4)
    shutil.rmtree(d / "our_ckpt")
