"""Multi-GPU tests (run as child processes, one per GPU): the NVLink kernels against NCCL, and DDP /
ZeRO training with the fused kernels against the single-GPU run of the same global batch."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _torchrun(script, n, *args, timeout=600):
    env = dict(os.environ)
    env.setdefault("ITB_NO_REBUILD", "1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(HERE, script), *args]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + "\n" + r.stderr[-3000:]
    return r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("nvls", ["1", "0"])
def test_nvlink_collectives_match_nccl(nvls):
    os.environ["ITB_NVLS"] = nvls
    out = _torchrun("mgpu_worker.py", min(_ngpu(), 8), "collectives")
    assert "COLLECTIVES OK" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode", ["zero0", "zero1", "zero2", "zero0_nccl", "zero2_nccl"])
def test_ddp_training_matches_single_gpu(mode):
    os.environ["ITB_NVLS"] = "1"
    out = _torchrun("mgpu_worker.py", 2, "ddp", mode)
    assert "DDP OK" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("nvls", ["1", "0"])
def test_fused_tensor_parallel_linears_match_nccl(nvls):
    os.environ["ITB_NVLS"] = nvls
    out = _torchrun("mgpu_worker.py", 2, "tp_fused")
    assert "TP FUSED OK" in out


@pytest.mark.skipif(_ngpu() < 8, reason="needs 8 GPUs")
def test_fused_tensor_parallel_linears_match_nccl_8_ranks():
    os.environ["ITB_NVLS"] = "1"
    out = _torchrun("mgpu_worker.py", 8, "tp_fused")
    assert "TP FUSED OK" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_vocab_parallel_cross_entropy_merge_kernel():
    os.environ["ITB_NVLS"] = "1"
    out = _torchrun("mgpu_worker.py", 2, "vocab_ce")
    assert "VOCAB CE OK" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("nvls", ["1", "0"])
def test_fused_gemm_all_reduce_matches_nccl(nvls):
    os.environ["ITB_NVLS"] = nvls
    out = _torchrun("mgpu_worker.py", 2, "tp_fused_nosp")
    assert "TP NOSP OK" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_tp_sp_model_training_fused_matches_nccl():
    os.environ["ITB_NVLS"] = "1"
    out = _torchrun("mgpu_worker.py", 2, "tp_model")
    assert "TP MODEL OK" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_pipeline_parallel_on_gpus():
    out = _torchrun("mgpu_worker.py", 2, "pp_gpu")
    assert "PP GPU OK" in out


@pytest.mark.gpu
@pytest.mark.skipif(_ngpu() < 4, reason="needs 4 GPUs")
@pytest.mark.parametrize("flags", [
    ["--tensor_parallel", "2", "--sequence_parallel", "--zero_stage", "2"],
    ["--tensor_parallel", "2", "--sequence_parallel", "--pipeline_parallel", "2"],
])
def test_hybrid_training_follows_the_single_gpu_trajectory(tmp_path, flags):
    """DP x TP+SP with ZeRO-2, and TP+SP x PP, on 4 GPUs against ONE GPU on the same llm.c weights and
    the same global batch, in fp32: the same losses step by step (the GPU counterpart of
    tests/test_examples_cpu.py::test_hybrid_parallel_runs_follow_the_one_rank_trajectory; no rank leaves
    early and NVLS is off for the collectives)."""
    import re
    import subprocess
    import sys

    from infinitrain_b200 import _ext
    from infinitrain_b200.data import write_token_file
    from infinitrain_b200.models import llmc
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel
    from infinitrain_b200.parallel import global_env as genv

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    genv.InitAllEnv(world_size=1, rank=0)
    cfg = TransformerConfig.LLaMA3(n_layer=4, n_embd=256, n_head=4, n_kv_head=2, vocab_size=1024, original_vocab_size=1024,
                                   block_size=512, multiple_of=64, ffn_dim_multiplier=1.5)
    torch.manual_seed(42)
    m = TransformerModel(cfg)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() > 1:
                p.normal_(0, 0.05)
    llmc.write_llama3_llmc(str(tmp_path / "w.bin"), cfg, llmc.full_state_dict(m))
    g = torch.Generator().manual_seed(1)
    write_token_file(str(tmp_path / "t.bin"), torch.randint(0, 1024, (2 * 512 * 20 + 1,), generator=g).tolist(), llama3=True)
    common = [os.path.join(root, "examples", "llama3", "main.py"), "--device", "cuda", "--llmc_filepath", str(tmp_path / "w.bin"),
              "--input_bin", str(tmp_path / "t.bin"), "--batch_size", "2", "--sequence_length", "512", "--total_batch_size",
              "4096", "--num_iteration", "3", "--dtype", "float32", "--learning_rate", "0.05", "--optimizer", "sgd"]
    env = {**os.environ, "NCCL_NVLS_ENABLE": "0", "ITB_NO_REBUILD": "1"}

    def losses(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=root)
        assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
        return [float(x.group(1)) for x in re.finditer(r"step\s+\d+/\d+\s+\|\s+train loss\s+([\d.]+)", r.stdout + r.stderr)]

    one = losses([sys.executable, *common])
    launcher = _ext.launcher_path()
    if not launcher.exists():
        _ext.build_launcher()
    four = losses([str(launcher), "--nproc_per_node=4", "--rdzv_endpoint=127.0.0.1:29990", "--", sys.executable, *common, *flags])
    assert len(one) == 3 and len(four) == 3
    assert max(abs(a - b) for a, b in zip(one, four)) <= 1e-4, list(zip(one, four))
