"""Loss-trajectory parity with the UNMODIFIED reference, both on CPU in fp32.

The reference's stock GPT-2 trainer (its ``USE_CUDA=OFF`` build, ``baseline/build_reference.py
--cpu-only``) and this framework's trainer read the same llm.c weight file and the same token file
and take the same SGD steps; the per-step losses must agree within the reference's own fp32
tolerance of 1e-5 (its scripts/compare_loss.py:20,56-57)."""
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "baseline", "_ref", "bin", "gpt2_cpu")
SRC = os.environ.get("ITB_REFERENCE_SRC", os.path.join(os.sep, "root", "reference"))


def _reference_binary():
    if not os.path.exists(BIN):
        if not os.path.isdir(os.path.join(SRC, "infini_train")):
            pytest.skip("no reference checkout to build the CPU-only trainer from")
        r = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "build_reference.py"), "--cpu-only", "--src", SRC],
                           capture_output=True, text=True, timeout=1500)
        assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return BIN


def _losses(text):
    return [float(m.group(1)) for m in re.finditer(r"step\s+\d+/\d+\s+\|\s+train loss\s+([\d.]+)", text)]


def test_gpt2_sgd_trajectory_equals_the_reference(tmp_path):
    from infinitrain_b200.data import write_token_file
    from infinitrain_b200.models import llmc
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel
    from infinitrain_b200.parallel import global_env as genv

    exe = _reference_binary()
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
    model_bin, tokens_bin = str(tmp_path / "model.bin"), str(tmp_path / "tokens.bin")
    llmc.write_gpt2_llmc(model_bin, cfg, llmc.full_state_dict(m))
    g = torch.Generator().manual_seed(1)
    write_token_file(tokens_bin, torch.randint(0, 256, (4 * 64 * 12 + 1,), generator=g).tolist())
    common = ["--device", "cpu", "--llmc_filepath", model_bin, "--input_bin", tokens_bin, "--batch_size", "4",
              "--sequence_length", "64", "--total_batch_size", "256", "--num_iteration", "10", "--dtype", "float32",
              "--learning_rate", "0.05"]
    ref = subprocess.run([exe, *common, "--overfit_single_batch=false"], capture_output=True, text=True, timeout=600,
                         cwd=tmp_path)
    assert ref.returncode == 0, ref.stderr[-2000:]
    ours = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "gpt2", "main.py"), *common, "--optimizer", "sgd"],
                          capture_output=True, text=True, timeout=600, cwd=tmp_path)
    assert ours.returncode == 0, ours.stderr[-2000:]
    a, b = _losses(ref.stdout + ref.stderr), _losses(ours.stdout + ours.stderr)
    assert len(a) == 10 and len(b) == 10
    assert max(abs(x - y) for x, y in zip(a, b)) <= 1e-5, list(zip(a, b))
    assert abs(a[0] - a[-1]) > 1e-3            # the weights moved: this is a trajectory, not ten forward passes
