"""bf16 loss-trajectory parity on a GPU against the UNMODIFIED reference's CUDA build.

The reference's acceptance rule for bf16 runs is a per-step absolute loss difference of at most 1e-2
on the step line its trainers print (scripts/compare_loss.py:56-57, example/gpt2/main.cc:489-497).
Here the reference's stock ``example/gpt2`` trainer (``baseline/_ref/bin/gpt2``, cuBLAS GEMMs, SIMT
kernels, materialised attention) and this framework's trainer (tcgen05 GEMMs, flash attention, fused
norms) read the same llm.c weight file and token file and take the same ten SGD steps under bf16
autocast; the test holds both residual-stream dtypes of this framework to that rule.

The reference trains GPT-2 with ``wte`` and ``lm_head`` untied on CUDA (its ``Module::To`` re-creates
every parameter, which breaks the aliasing: src/nn/modules/module.cc:269-285), so this side runs with
``--untie_weights``.
"""
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "baseline", "_ref", "bin", "gpt2")
OURS = [sys.executable, os.path.join(ROOT, "examples", "gpt2", "main.py")]
kBf16Tolerance = 1e-2       # scripts/compare_loss.py:57
kSteps = 10

pytestmark = pytest.mark.gpu


def _losses(text):
    return [float(m.group(1)) for m in re.finditer(r"step\s+\d+/\d+\s+\|\s+train loss\s+([\d.]+)", text)]


def _run(cmd, cwd, env=None):
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=cwd, env=env)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return _losses(r.stdout + r.stderr), r.stdout + r.stderr


@pytest.fixture(scope="module")
def world(tmp_path_factory):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    if not os.path.exists(BIN):
        pytest.skip("the reference's CUDA trainer is not built (python baseline/build_reference.py --src <checkout>)")
    from infinitrain_b200.data import write_token_file
    from infinitrain_b200.models import llmc
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel
    from infinitrain_b200.parallel import global_env as genv

    d = tmp_path_factory.mktemp("parity_gpu")
    genv.InitAllEnv(world_size=1, rank=0)
    # GPT-2 width and head size at a quarter of the depth, a small vocabulary: seconds per run
    cfg = TransformerConfig.GPT2(n_layer=3, n_embd=768, n_head=12, n_kv_head=12, vocab_size=8192,
                                 original_vocab_size=8192, block_size=1024)
    torch.manual_seed(42)
    m = TransformerModel(cfg)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if p.dim() >= 2:
                p.normal_(0, 0.02)
    llmc.write_gpt2_llmc(str(d / "model.bin"), cfg, llmc.full_state_dict(m))
    g = torch.Generator().manual_seed(1)
    B, T = 4, 256
    # a skewed unigram distribution (most of the mass on a few dozen ids): something SGD learns within ten
    # steps, so that the trajectories being compared actually move
    n_tok = B * T * (kSteps + 3) + 1
    ids = torch.multinomial(1.0 / torch.arange(1, 8193, dtype=torch.float64) ** 1.5, n_tok, replacement=True, generator=g)
    write_token_file(str(d / "tokens.bin"), ids.tolist())
    common = ["--llmc_filepath", "model.bin", "--input_bin", "tokens.bin", "--batch_size", str(B), "--sequence_length",
              str(T), "--total_batch_size", str(B * T), "--num_iteration", str(kSteps), "--dtype", "bfloat16",
              "--learning_rate", "0.003"]
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "OMP_NUM_THREADS")}
    ref, log = _run([BIN, *common, "--model", "gpt2", "--device", "cuda", "--nthread_per_process", "1",
                     "--overfit_single_batch=false", "--freq_generate_txt", "1000000"], d, env)
    assert len(ref) == kSteps, log[-2000:]
    (d / "reference_bf16.log").write_text(log)
    return d, common, ref


@pytest.mark.parametrize("residual", ["float32", "bfloat16"])
def test_bf16_sgd_trajectory_is_within_the_reference_tolerance(world, residual):
    d, common, ref = world
    ours, log = _run([*OURS, *common, "--optimizer", "sgd", "--device", "cuda", "--untie_weights", "--residual_dtype",
                      residual], d)
    (d / f"ours_bf16_residual_{residual}.log").write_text(log)
    assert len(ours) == kSteps, log[-2000:]
    diffs = [abs(a - b) for a, b in zip(ref, ours)]
    out = os.environ.get("ITB_TEST_ARTIFACTS", "")
    if out and os.path.isdir(out):       # keep the per-step figures when the caller names a folder for them
        with open(os.path.join(out, f"parity_bf16_residual_{residual}.txt"), "w") as f:
            f.write("step reference ours abs_diff\n")
            for i, (a, b) in enumerate(zip(ref, ours)):
                f.write(f"{i + 1} {a:.6f} {b:.6f} {abs(a - b):.6f}\n")
            f.write(f"max_abs_diff {max(diffs):.6f}\n")
    assert max(diffs) <= kBf16Tolerance, list(zip(ref, ours))
    assert abs(ref[0] - ref[-1]) > 2 * kBf16Tolerance, "the run must move the loss by more than the tolerance"
