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
