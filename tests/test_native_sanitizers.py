"""The framework-free C++ runtime (planners, token file, batch ring) built with ThreadSanitizer and
with AddressSanitizer + UBSan and run on the host."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUNTIME = os.path.join(ROOT, "infinitrain_b200", "csrc", "runtime")


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
@pytest.mark.parametrize("sanitizer", ["thread", "address,undefined"])
def test_runtime_under_sanitizers(tmp_path, sanitizer):
    exe = tmp_path / "runtime_checks"
    cmd = ["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer", f"-I{RUNTIME}",
           os.path.join(ROOT, "tests", "native", "runtime_sanitizers.cc"), os.path.join(RUNTIME, "planners.cpp"),
           "-o", str(exe), "-pthread"]
    b = subprocess.run(cmd, capture_output=True, text=True)
    if b.returncode != 0 and "sanitize" in b.stderr and "cannot find" in b.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert b.returncode == 0, b.stderr[-3000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1", ASAN_OPTIONS="detect_leaks=1",
               UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout + r.stderr[-3000:]
    assert "runtime checks ok" in r.stdout
    assert "Sanitizer" not in r.stderr and "runtime error" not in r.stderr, r.stderr[-3000:]


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_tp_protocol_model_and_its_negative_control(tmp_path):
    """Host-threads model of the fused tensor-parallel launches' flag protocol: with the rule the
    kernels use no reader ever sees a newer epoch in a workspace slot (also race-free under
    ThreadSanitizer); waiting for one launch less is caught."""
    src = os.path.join(ROOT, "tests", "native", "tp_protocol_model.cc")
    good, bad = tmp_path / "model_tsan", tmp_path / "model_relaxed"
    b = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", src, "-o", str(good), "-pthread"],
                       capture_output=True, text=True)
    if b.returncode != 0 and "sanitize" in b.stderr and "cannot find" in b.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert b.returncode == 0, b.stderr[-2000:]
    r = subprocess.run([str(good)], capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, TSAN_OPTIONS="halt_on_error=1"))
    assert r.returncode == 0 and "protocol model ok" in r.stdout, r.stdout + r.stderr[-2000:]
    assert "ThreadSanitizer" not in r.stderr
    subprocess.run(["g++", "-std=c++17", "-O1", "-DITB_MODEL_SLACK=1", src, "-o", str(bad), "-pthread"], check=True)
    r = subprocess.run([str(bad)], capture_output=True, text=True, timeout=300)
    assert r.returncode != 0 and "protocol violations" in r.stderr


@pytest.mark.skipif(shutil.which("cmake") is None, reason="needs cmake")
def test_parallel_stack_under_thread_sanitizer(tmp_path):
    """The C++ frontend's process groups, DDP reducer, ZeRO optimizer and pipeline executor, with the
    ranks played by threads (tests/native/test_parallel.cc), built with -fsanitize=thread through the
    CMake project's ITB_SANITIZE option: no data race may be reported."""
    build = tmp_path / "tsan"
    gen = ["-G", "Ninja"] if shutil.which("ninja") else []
    cxx = ["-DCMAKE_CXX_COMPILER=/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []
    cfg = subprocess.run(["cmake", "-S", ROOT, "-B", str(build), *gen, *cxx, "-DITB_WITH_CUDA=OFF", "-DITB_SANITIZE=thread"],
                         capture_output=True, text=True, timeout=600)
    assert cfg.returncode == 0, cfg.stdout[-3000:] + cfg.stderr[-3000:]
    b = subprocess.run(["cmake", "--build", str(build), "--target", "test_parallel_cpu"], capture_output=True, text=True,
                       timeout=3000)
    if b.returncode != 0 and "cannot find" in (b.stdout + b.stderr) and "tsan" in (b.stdout + b.stderr):
        pytest.skip("sanitizer runtime not installed")
    assert b.returncode == 0, b.stdout[-4000:] + b.stderr[-3000:]
    r = subprocess.run([str(build / "test_parallel_cpu"), "--device", "cpu"], capture_output=True, text=True, timeout=900)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "0 failed" in out, out[-4000:]
    assert "ThreadSanitizer" not in out, out[-6000:]
