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
