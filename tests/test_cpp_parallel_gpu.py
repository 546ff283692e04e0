"""The C++ trainer on GPUs: NCCL process groups (own communication stream, events), bucketed data
parallelism overlapped with backward, ZeRO-1 and tensor + sequence parallelism must follow the
single-GPU trajectory of the same binary, in fp32 (libtorch formulation) and under bf16 autocast (the
fused sm_100a kernels)."""
import os
import subprocess

import pytest
import torch

from test_cpp_parallel import ENV, LLAMA, ROOT, _free_port, _losses, files  # noqa: F401  (files is a fixture)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda_binaries():
    import importlib.util

    from infinitrain_b200 import _ext

    _ext.load(required=True)
    spec = importlib.util.spec_from_file_location("itb_cpp_build", os.path.join(ROOT, "examples", "cpp", "build.py"))
    cpp_build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(cpp_build)
    launcher = _ext.launcher_path()
    if not launcher.exists():
        _ext.build_launcher()
    return str(launcher), str(cpp_build.build(cuda=True))


def _train(cuda_binaries, files, ranks, dtype, *extra, iters=4):
    launcher, trainer = cuda_binaries
    cmd = [trainer, "--family", "llama3", "--device", "cuda", "--llmc_filepath", "llama3.bin", "--input_bin", "tokens32.bin",
           "--batch_size", "2", "--sequence_length", "64", "--total_batch_size", "1024", "--num_iteration", str(iters),
           "--dtype", dtype, *LLAMA, *extra]
    if ranks > 1:
        cmd = [launcher, f"--nproc_per_node={ranks}", f"--rdzv_endpoint=127.0.0.1:{_free_port()}", "--", *cmd]
    env = {**ENV, "NCCL_NVLS_ENABLE": "0"}
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=files, env=env)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    losses = _losses(r.stdout + r.stderr)
    assert len(losses) == iters, (r.stdout + r.stderr)[-3000:]
    return losses


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-4), ("bfloat16", 3e-2)])
def test_cpp_trainer_on_two_gpus_follows_one_gpu(cuda_binaries, files, dtype, tol):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    one = _train(cuda_binaries, files, 1, dtype)
    for flags in ((), ("--zero_stage", "1"), ("--tensor_parallel", "2", "--sequence_parallel"),
                  ("--pipeline_parallel", "2", "--virtual_pipeline_parallel", "2")):
        got = _train(cuda_binaries, files, 2, dtype, *flags)
        assert max(abs(a - b) for a, b in zip(got, one)) <= tol, (flags, list(zip(got, one)))
