"""The C++ frontend (infinitrain_b200/csrc/frontend/itb) on CPU: its API checks, and its trainer
against the Python trainer and the unmodified reference on the same weight and token files."""
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref", "bin", "gpt2_cpu")
ENV = {**os.environ, "OMP_NUM_THREADS": "2"}


def _losses(text):
    return [float(m.group(1)) for m in re.finditer(r"step\s+\d+/\d+\s+\|\s+train loss\s+([\d.]+)", text)]


def _free_port() -> int:
    import socket

    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _run(cmd, cwd):
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True, timeout=900, cwd=cwd, env=ENV)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return _losses(r.stdout + r.stderr)


@pytest.fixture(scope="module")
def trainer():
    import importlib.util

    spec = importlib.util.spec_from_file_location("itb_cpp_build", os.path.join(ROOT, "examples", "cpp", "build.py"))
    cpp_build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(cpp_build)
    return str(cpp_build.build(cuda=False))


@pytest.fixture(scope="module")
def files(tmp_path_factory):
    from infinitrain_b200.data import write_token_file
    from infinitrain_b200.models import llmc
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel
    from infinitrain_b200.parallel import global_env as genv

    d = tmp_path_factory.mktemp("cppfe")
    genv.InitAllEnv(world_size=1, rank=0)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, 256, (4 * 64 * 20 + 1,), generator=g).tolist()
    write_token_file(str(d / "tokens16.bin"), toks)
    write_token_file(str(d / "tokens32.bin"), toks, llama3=True)
    torch.manual_seed(42)
    gcfg = TransformerConfig.GPT2(n_layer=2, n_embd=96, n_head=12, n_kv_head=12, vocab_size=256, original_vocab_size=256,
                                  block_size=64)
    lcfg = TransformerConfig.LLaMA3(n_layer=2, n_embd=64, n_head=4, n_kv_head=2, vocab_size=256, original_vocab_size=256,
                                    block_size=64, multiple_of=16, ffn_dim_multiplier=1.5)
    for cfg, name, write in ((gcfg, "gpt2.bin", llmc.write_gpt2_llmc), (lcfg, "llama3.bin", llmc.write_llama3_llmc)):
        m = TransformerModel(cfg)
        with torch.no_grad():
            for p in m.parameters():
                if p.dim() > 1:
                    p.normal_(0, 0.1)
        write(str(d / name), cfg, llmc.full_state_dict(m))
    return d


def test_api_checks(tmp_path):
    from torch.utils import cpp_extension as ce

    exe = tmp_path / "frontend_api"
    lib = ce.library_paths()[0]
    cmd = ["g++", "-std=c++17", "-O1", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *[f"-I{p}" for p in ce.include_paths()], f"-I{os.path.join(ROOT, 'infinitrain_b200', 'csrc', 'frontend')}",
           os.path.join(ROOT, "tests", "native", "frontend_api.cc"), "-o", str(exe), f"-L{lib}", f"-Wl,-rpath,{lib}",
           "-ltorch", "-ltorch_cpu", "-lc10", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([str(exe), str(tmp_path)], capture_output=True, text=True, timeout=300, env=ENV)
    assert r.returncode == 0 and r.stdout.startswith("ok "), r.stdout + r.stderr


def test_gpt2_trajectory_matches_python_trainer_and_reference(trainer, files):
    common = ["--device", "cpu", "--llmc_filepath", "gpt2.bin", "--input_bin", "tokens16.bin", "--batch_size", "4",
              "--sequence_length", "64", "--total_batch_size", "256", "--num_iteration", "8", "--dtype", "float32",
              "--learning_rate", "0.05"]
    cpp = _run([trainer, "--family", "gpt2", *common, "--optimizer", "sgd"], files)
    py = _run([sys.executable, os.path.join(ROOT, "examples", "gpt2", "main.py"), *common, "--optimizer", "sgd"], files)
    assert len(cpp) == 8 and max(abs(a - b) for a, b in zip(cpp, py)) <= 2e-6, list(zip(cpp, py))
    if os.path.exists(REF):
        ref = _run([REF, *common, "--overfit_single_batch=false"], files)
        assert max(abs(a - b) for a, b in zip(cpp, ref)) <= 1e-5, list(zip(cpp, ref))


def test_llama3_adam_with_accumulation_matches_python_trainer(trainer, files):
    common = ["--device", "cpu", "--llmc_filepath", "llama3.bin", "--input_bin", "tokens32.bin", "--batch_size", "4",
              "--sequence_length", "64", "--total_batch_size", "512", "--num_iteration", "6", "--dtype", "float32",
              "--learning_rate", "1e-3", "--optimizer", "adam"]
    cpp = _run([trainer, "--family", "llama3", *common], files)
    py = _run([sys.executable, os.path.join(ROOT, "examples", "llama3", "main.py"), *common], files)
    assert len(cpp) == 6 and max(abs(a - b) for a, b in zip(cpp, py)) <= 2e-6, list(zip(cpp, py))
    assert cpp[-1] < cpp[0]                               # and the loss goes down


def test_checkpoint_written_by_cpp_resumes_in_cpp_and_in_python(trainer, files):
    common = ["--device", "cpu", "--llmc_filepath", "llama3.bin", "--input_bin", "tokens32.bin", "--batch_size", "4",
              "--sequence_length", "64", "--total_batch_size", "256", "--num_iteration", "8", "--dtype", "float32",
              "--learning_rate", "1e-3", "--optimizer", "adam"]
    full = _run([trainer, "--family", "llama3", *common, "--save", "ck", "--save_interval", "4"], files)
    ck = os.path.join("ck", "checkpoint_step_000004")
    assert sorted(os.listdir(files / ck)) == ["model.ckpt", "optimizer.ckpt", "trainer_state.json"]
    again = _run([trainer, "--family", "llama3", *common, "--load", ck], files)
    assert len(again) == 4 and max(abs(a - b) for a, b in zip(full[4:], again)) <= 1e-6
    py = _run([sys.executable, os.path.join(ROOT, "examples", "llama3", "main.py"), *common, "--load", ck,
               "--save_optimizer_state"], files)
    assert len(py) == 4 and max(abs(a - b) for a, b in zip(full[4:], py)) <= 2e-6, list(zip(full[4:], py))


def test_lora_training_matches_python_trainer_and_reference(trainer, files):
    """All three trainers load one adapter file, train the adapters on the frozen base along the same
    trajectory and write adapter files with the same tensors."""
    from infinitrain_b200.models import llmc
    from infinitrain_b200.nn import lora

    lcfg = lora.LoRAConfig(rank=4, alpha=8.0, target_modules=lora.ParseLoRATargetModules("c_attn,c_proj"))

    def adapters(path=None):
        m = lora.GetLoRAModel(llmc.GPT2FromLLMC(str(files / "gpt2.bin")), lcfg)
        if path:
            lora.LoadLoRAWeights(m, str(files / path))
        return m

    m = adapters()
    torch.manual_seed(7)
    with torch.no_grad():
        for p in lora.GetLoRAParameters(m):
            p.normal_(0, 0.3)
    lora.SaveLoRAWeights(m, str(files / "adapter.bin"))
    common = ["--device", "cpu", "--llmc_filepath", "gpt2.bin", "--input_bin", "tokens16.bin", "--batch_size", "4",
              "--sequence_length", "64", "--total_batch_size", "256", "--num_iteration", "5", "--dtype", "float32",
              "--learning_rate", "0.05", "--lora_rank", "4", "--lora_alpha", "8", "--lora_load_path", "adapter.bin"]
    cpp = _run([trainer, "--family", "gpt2", *common, "--optimizer", "sgd", "--lora_save_path", "cpp_adapter.bin"], files)
    py = _run([sys.executable, os.path.join(ROOT, "examples", "gpt2", "main.py"), *common, "--optimizer", "sgd",
               "--lora_save_path", "py_adapter.bin"], files)
    assert len(cpp) == 5 and max(abs(a - b) for a, b in zip(cpp, py)) <= 1e-5, list(zip(cpp, py))
    a, b = ({k: v.detach() for k, v in lora.LoRAStateDict(adapters(p)).items()} for p in ("cpp_adapter.bin", "py_adapter.bin"))
    assert max(float((a[k] - b[k]).abs().max()) for k in a) < 1e-5
    if os.path.exists(REF):
        ref = _run([REF, *common, "--overfit_single_batch=false"], files)
        assert max(abs(x - y) for x, y in zip(cpp, ref)) <= 1e-5, list(zip(cpp, ref))


def test_text_generation_matches_python_sampler(trainer, tmp_path):
    """Same weights, same tokenizer file, same xorshift* stream: the C++ trainer and the Python
    Tokenizer.GenerateText sample the same continuation of the reference's prompt."""
    from infinitrain_b200.data import Tokenizer, write_token_file
    from infinitrain_b200.data.tokenizer import write_tokenizer_file
    from infinitrain_b200.models import llmc
    from infinitrain_b200.nn.transformer import TransformerConfig, TransformerModel
    from infinitrain_b200.parallel import global_env as genv

    genv.InitAllEnv(world_size=1, rank=0)
    V = 4096                                                 # the prompt's GPT-2 token ids go up to 3616
    cfg = TransformerConfig.GPT2(n_layer=1, n_embd=48, n_head=12, n_kv_head=12, vocab_size=V, original_vocab_size=V,
                                 block_size=32)
    torch.manual_seed(5)
    m = TransformerModel(cfg)
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.3)
    llmc.write_gpt2_llmc(str(tmp_path / "m.bin"), cfg, llmc.full_state_dict(m))
    write_tokenizer_file(str(tmp_path / "tok.bin"), [f"<{i}>".encode() for i in range(V)], eot=V - 1)
    write_token_file(str(tmp_path / "t.bin"), torch.randint(0, V, (2 * 32 * 4 + 1,)).tolist())
    want = Tokenizer(str(tmp_path / "tok.bin")).GenerateText(m, 2, 32, 16, torch.device("cpu"), print_fn=None)
    r = subprocess.run([trainer, "--family", "gpt2", "--device", "cpu", "--llmc_filepath", "m.bin", "--input_bin", "t.bin",
                        "--tokenizer_bin", "tok.bin", "--batch_size", "2", "--sequence_length", "32", "--total_batch_size",
                        "64", "--num_iteration", "1", "--learning_rate", "0", "--freq_generate_txt", "1", "--text_length", "16"],
                       capture_output=True, text=True, timeout=300, cwd=tmp_path, env=ENV)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [ln for ln in r.stdout.splitlines() if ln.startswith("The meaning of life is")]
    assert got == [want] and want.count("<") == 11, (got, want)


def test_two_rank_data_parallel_matches_python_ddp(trainer, files):
    """Two CPU ranks started by the C++ launcher: the C++ trainer (gradient buckets averaged through its
    store transport) and the Python trainer (gloo DDP) follow the same loss trajectory."""
    from infinitrain_b200 import _ext

    launcher = _ext.launcher_path()
    if not launcher.exists():
        _ext.build_launcher()
    common = ["--device", "cpu", "--llmc_filepath", "gpt2.bin", "--input_bin", "tokens16.bin", "--batch_size", "2",
              "--sequence_length", "64", "--total_batch_size", "512", "--num_iteration", "5", "--dtype", "float32",
              "--learning_rate", "0.05", "--optimizer", "sgd"]
    cpp = _run([launcher, "--nproc_per_node=2", f"--rdzv_endpoint=127.0.0.1:{_free_port()}", "--", trainer, "--family", "gpt2", *common],
               files)
    py = _run([launcher, "--nproc_per_node=2", f"--rdzv_endpoint=127.0.0.1:{_free_port()}", "--", sys.executable,
               os.path.join(ROOT, "examples", "gpt2", "main.py"), *common], files)
    assert len(cpp) == 5 and len(py) == 5, (cpp, py)
    assert max(abs(a - b) for a, b in zip(cpp, py)) <= 1e-5, list(zip(cpp, py))


def test_per_module_records_line_up_with_the_reference(trainer, files):
    """With --precision_check the C++ trainer writes the reference's record lines and dump files for
    every module it has (the reference adds its three pipeline-stage wrappers); all tensors both sides
    dump agree within allclose(atol 1e-5, rtol 1e-3)."""
    import glob

    import numpy as np

    if not os.path.exists(REF):
        pytest.skip("the reference's CPU build is not there")
    common = ["--device", "cpu", "--llmc_filepath", "gpt2.bin", "--input_bin", "tokens16.bin", "--batch_size", "4",
              "--sequence_length", "64", "--total_batch_size", "512", "--num_iteration", "2", "--dtype", "float32",
              "--learning_rate", "0.05"]
    _run([REF, *common, "--overfit_single_batch=false", "--precision_check", "level=1,format=simple,path=pc_ref,save_tensors=true"],
         files)
    _run([trainer, "--family", "gpt2", *common, "--optimizer", "sgd", "--precision_check",
          "level=1,format=simple,path=pc_cpp,save_tensors=true"], files)
    (ref_dir,), (cpp_dir,) = glob.glob(str(files / "pc_ref" / "*")), glob.glob(str(files / "pc_cpp" / "*"))
    ref_files = set(os.listdir(os.path.join(ref_dir, "rank_0")))
    cpp_files = set(os.listdir(os.path.join(cpp_dir, "rank_0")))
    assert cpp_files <= ref_files and len(cpp_files) >= 100
    assert all(f.startswith(("TransformerFirstStage", "TransformerChunk", "TransformerLastStage")) for f in ref_files - cpp_files)
    for f in sorted(cpp_files):
        a, b = np.load(os.path.join(ref_dir, "rank_0", f)), np.load(os.path.join(cpp_dir, "rank_0", f))
        assert a.shape == b.shape and np.allclose(a, b, atol=1e-5, rtol=1e-3), f
    ref_names = {ln.split()[2] for ln in open(os.path.join(ref_dir, "precision_check_rank_0.log"))}
    cpp_lines = open(os.path.join(cpp_dir, "precision_check_rank_0.log")).read().splitlines()
    assert {ln.split()[2] for ln in cpp_lines} <= ref_names
    assert re.match(r"\[GAS-0\] \[L-0\] transformer\.wte_forward tensor\[0\]: dtype=float32 shape=\(4,64,96\) min=\S+ max=\S+ "
                    r"mean=\S+ \[.*, \.\.\.\] \[NaN:0 Inf:0\]$", cpp_lines[0])


def test_md5_records_and_function_level_of_the_cpp_precision_checker(trainer, files):
    """format=md5 writes the digest of every recorded tensor's fp32 bytes (rounded to multiples of
    md5_tolerance first, the reference's quantisation); level=2 adds one record per op input, output and
    output gradient.  The digests are checked against hashlib over the dumped tensors, and against the
    Python checker's own digest function."""
    import glob
    import hashlib

    import numpy as np

    from infinitrain_b200.utils.precision_checker import ComputeMD5

    common = ["--family", "gpt2", "--device", "cpu", "--llmc_filepath", "gpt2.bin", "--input_bin", "tokens16.bin", "--batch_size", "2",
              "--sequence_length", "64", "--total_batch_size", "128", "--num_iteration", "1", "--dtype", "float32",
              "--learning_rate", "0.05", "--optimizer", "sgd"]
    for tag, tol in (("plain", 0.0), ("quantised", 1e-3)):
        cfg = f"level=2,format=md5,path=pc_md5_{tag},save_tensors=true" + (f",md5_tolerance={tol}" if tol else "")
        _run([trainer, *common, "--precision_check", cfg], files)
        (out,) = glob.glob(str(files / f"pc_md5_{tag}" / "*"))
        lines = open(os.path.join(out, "precision_check_rank_0.log")).read().splitlines()
        recs = [re.match(r"\[GAS-0\] \[L-0\] (\S+) tensor\[(\d+)\]: dtype=float32 shape=\(([\d,]*)\) md5=([0-9a-f]{32})$", ln) for ln in lines]
        assert all(recs) and len(recs) > 100, [ln for ln, m in zip(lines, recs) if not m][:3]
        names = [m.group(1) for m in recs]
        # modules and functions, forward and backward
        assert "transformer.h.0.attn.c_attn_forward" in names and "transformer.h.0.attn.c_attn_backward" in names
        for fn in ("Linear", "LayerNorm", "Attention", "Embedding", "CrossEntropy"):
            assert f"{fn}Function_forward" in names and any(n.startswith(f"{fn}Function") and n.endswith("_backward") for n in names), fn
        checked = 0
        for m in recs:
            path = os.path.join(out, "rank_0", m.group(1) + ".npy")
            if m.group(2) != "0" or names.count(m.group(1)) != 1:
                continue                                   # several tensors of one record share a dump file name
            a = np.load(path)
            assert ",".join(str(d) for d in a.shape) == m.group(3)
            import torch as _t
            assert ComputeMD5(_t.from_numpy(a), tol) == m.group(4), m.group(1)
            if not tol:
                assert hashlib.md5(a.astype(np.float32).tobytes()).hexdigest() == m.group(4)
            checked += 1
        assert checked > 40


def test_validation_loss_and_single_batch_overfit_match_python_trainer(trainer, files):
    """--input_val_bin / --val_loss_every / --val_max_batches and --overfit_single_batch: the C++ and the
    Python trainer log the same validation losses and the same single-batch trajectory."""
    common = ["--device", "cpu", "--llmc_filepath", "gpt2.bin", "--input_bin", "tokens16.bin", "--batch_size", "4",
              "--sequence_length", "64", "--total_batch_size", "512", "--num_iteration", "5", "--dtype", "float32",
              "--learning_rate", "0.05", "--optimizer", "sgd", "--input_val_bin", "tokens16.bin", "--val_loss_every", "2",
              "--val_max_batches", "3", "--overfit_single_batch"]

    def run(cmd):
        r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True, timeout=900, cwd=files, env=ENV)
        assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
        text = r.stdout + r.stderr
        val = [(int(m.group(1)), float(m.group(2)), int(m.group(3)))
               for m in re.finditer(r"step\s+(\d+)/\d+ \| val loss ([\d.]+) \((\d+) batches\)", text)]
        return _losses(text), val

    cpp, cpp_val = run([trainer, "--family", "gpt2", *common])
    py, py_val = run([sys.executable, os.path.join(ROOT, "examples", "gpt2", "main.py"), *common])
    assert len(cpp) == 5 and max(abs(a - b) for a, b in zip(cpp, py)) <= 2e-6, list(zip(cpp, py))
    assert all(b < a for a, b in zip(cpp, cpp[1:]))              # one batch, seen ten times: the loss only falls
    assert [v[0] for v in cpp_val] == [2, 4, 5] and all(v[2] == 3 for v in cpp_val)
    assert len(py_val) == 3 and max(abs(a[1] - b[1]) for a, b in zip(cpp_val, py_val)) <= 2e-6, (cpp_val, py_val)


def _write_idx(path, array):
    import struct

    with open(path, "wb") as f:
        f.write(struct.pack(">HBB", 0, 0x08, array.ndim) + struct.pack(">" + "I" * array.ndim, *array.shape))
        f.write(array.tobytes())


def test_mnist_trainer_learns_and_data_parallel_replicas_change_nothing(tmp_path):
    """examples/cpp/mnist.cc on IDX files: the loss falls, the test set is classified, and running the
    network through the single-process DataParallel module (three replicas in threads) prints the same
    numbers as the one module."""
    import importlib.util

    import numpy as np

    spec = importlib.util.spec_from_file_location("itb_cpp_build", os.path.join(ROOT, "examples", "cpp", "build.py"))
    cpp_build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(cpp_build)
    exe = cpp_build.build(src=os.path.join(ROOT, "examples", "cpp", "mnist.cc"), out=str(tmp_path / "itb_mnist"))
    g = np.random.default_rng(0)
    centers = g.uniform(0, 255, (10, 784))
    for prefix, n in (("train", 640), ("t10k", 128)):
        labels = g.integers(0, 10, n).astype(np.uint8)
        images = np.clip(centers[labels] + g.normal(0, 30, (n, 784)), 0, 255).astype(np.uint8).reshape(n, 28, 28)
        _write_idx(tmp_path / f"{prefix}-images-idx3-ubyte", images)
        _write_idx(tmp_path / f"{prefix}-labels-idx1-ubyte", labels)

    def run(*extra):
        r = subprocess.run([str(exe), "--dataset", str(tmp_path), "--bs", "64", "--num_epoch", "3", "--lr", "0.5", *extra],
                           capture_output=True, text=True, timeout=600, env=ENV)
        assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
        text = r.stdout + r.stderr
        epochs = [float(m.group(1)) for m in re.finditer(r"train loss ([\d.]+)", text)]
        final = re.search(r"Total: (\d+), Correct: (\d+), Accuracy: ([\d.]+), AverageLoss: ([\d.]+)", text)
        assert len(epochs) == 3 and final, text[-2000:]
        return epochs, [float(x) for x in final.groups()], [l for l in text.splitlines() if "loss" in l.lower() and "ms" not in l]

    epochs, final, lines = run()
    assert epochs[2] < 0.5 * epochs[0]
    assert final[0] == 128 and final[2] > 0.9
    epochs_dp, final_dp, lines_dp = run("--data_parallel", "3")
    assert lines_dp == lines and final_dp == final
    r = subprocess.run([str(exe), "--dataset", str(tmp_path / "absent")], capture_output=True, text=True, timeout=60, env=ENV)
    assert r.returncode != 0 and "cannot open IDX file" in r.stdout + r.stderr
