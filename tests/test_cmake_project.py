"""The native CMake project: configures without CUDA, builds the launcher, the C++ trainer and the
native test suites, and runs them through ctest (label ``cpu``), the compile-fail test included.
Counterpart of the reference's ``BUILD_TEST`` configuration (CMakeLists.txt:218-234,
cmake/test_macros.cmake:50-156); the ``cuda`` label needs a B200 and is run there."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("cmake") is None or shutil.which("g++") is None, reason="needs cmake and g++")
def test_cmake_project_builds_and_its_cpu_suites_pass(tmp_path):
    build = tmp_path / "build"
    gen = ["-G", "Ninja"] if shutil.which("ninja") else []
    cfg = subprocess.run(["cmake", "-S", ROOT, "-B", str(build), *gen, "-DITB_WITH_CUDA=OFF"], capture_output=True,
                         text=True, timeout=600)
    assert cfg.returncode == 0, cfg.stdout[-3000:] + cfg.stderr[-3000:]
    b = subprocess.run(["cmake", "--build", str(build), "-j", str(os.cpu_count() or 4)], capture_output=True, text=True,
                       timeout=3000)
    assert b.returncode == 0, b.stdout[-4000:] + b.stderr[-3000:]
    t = subprocess.run(["ctest", "--test-dir", str(build), "-L", "cpu", "--output-on-failure"], capture_output=True,
                       text=True, timeout=1800)
    assert t.returncode == 0, t.stdout[-6000:] + t.stderr[-2000:]
    assert "100% tests passed" in t.stdout
    # the suites are registered per device, and the negative compile test is among them
    listing = subprocess.run(["ctest", "--test-dir", str(build), "-N"], capture_output=True, text=True, timeout=120).stdout
    for name in ("test_runtime_cpu", "test_ops_cpu", "frontend_api", "compile_fail_dtype", "compile_ok_dtype"):
        assert name in listing, listing
    # the harness filters by device and lists its cases
    cases = subprocess.run([str(build / "test_ops_cpu"), "--list"], capture_output=True, text=True, timeout=60).stdout
    assert "Ops.LinearForwardBackward/cpu" in cases and "Ops.CausalAttentionWithGroupedHeads/cpu" in cases
    skipped = subprocess.run([str(build / "test_ops_cpu"), "--device", "cuda"], capture_output=True, text=True, timeout=60)
    assert skipped.returncode in (0, 77)          # 77 without a GPU: ctest's "skipped"
