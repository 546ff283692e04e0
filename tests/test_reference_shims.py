"""The header-only stand-ins that let the unmodified reference build without its submodules
(glog / gflags / Eigen subset): compiled into a small program and exercised on the host."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIMS = os.path.join(ROOT, "baseline", "shims")

PROGRAM = r'''
#include "Eigen/Dense"
#include "gflags/gflags.h"
#include "glog/logging.h"
#include <cstdio>
DEFINE_string(model, "d12", "model name");
DEFINE_uint32(batch_size, 4, "batch");
DEFINE_bool(overfit_single_batch, true, "");
DEFINE_double(learning_rate, 1e-4, "");
DEFINE_int32(zero_stage, 0, "");
DEFINE_validator(zero_stage, [](const char*, int32_t v) { return v >= 0 && v <= 3; });
using M = Eigen::Map<Eigen::Matrix<float, Eigen::Dynamic, Eigen::Dynamic, Eigen::RowMajor>>;
using V = Eigen::Map<Eigen::Matrix<float, 1, Eigen::Dynamic, Eigen::RowMajor>>;
int main(int argc, char** argv) {
    google::InitGoogleLogging(argv[0]);
    gflags::ParseCommandLineFlags(&argc, &argv, true);
    float a[6] = {1, 2, 3, 4, 5, 6}, w[6] = {1, 0, 1, 0, 1, 0}, o[4], b[2] = {10, 20}, gb[2];
    M A(a, 2, 3), W(w, 2, 3), O(o, 2, 2);
    V B(b, 1, 2), GB(gb, 1, 2);
    O = A * W.transpose();
    O.rowwise() += B;
    GB = O.colwise().sum();
    CHECK_EQ(static_cast<int>(o[0]), 14) << "product";
    int* p = CHECK_NOTNULL(&argc);
    LOG(INFO) << "model " << FLAGS_model << " batch " << FLAGS_batch_size << " overfit " << FLAGS_overfit_single_batch
              << " lr " << FLAGS_learning_rate << " zero " << FLAGS_zero_stage << " argc " << *p;
    std::printf("%g %g %g %g | %g %g\n", o[0], o[1], o[2], o[3], gb[0], gb[1]);
    if (FLAGS_batch_size == 99) LOG(FATAL) << "fatal path";
    return 0;
}
'''


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_shims_compile_and_behave(tmp_path):
    src = tmp_path / "prog.cc"
    src.write_text(PROGRAM)
    exe = tmp_path / "prog"
    subprocess.run(["g++", "-std=c++20", f"-I{SHIMS}", str(src), "-o", str(exe)], check=True)
    r = subprocess.run([str(exe), "--model=gpt2", "--batch_size", "16", "--overfit_single_batch=false",
                        "--learning_rate", "3e-4", "--zero_stage=2", "positional"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert r.stdout.strip() == "14 22 20 25 | 34 47"
    assert "model gpt2 batch 16 overfit 0 lr 0.0003 zero 2 argc 2" in r.stderr
    bad = subprocess.run([str(exe), "--zero_stage=7"], capture_output=True, text=True)
    assert bad.returncode != 0 and "validation" in bad.stderr
    unknown = subprocess.run([str(exe), "--no_such_flag=1"], capture_output=True, text=True)
    assert unknown.returncode != 0 and "unknown command line flag" in unknown.stderr
    fatal = subprocess.run([str(exe), "--batch_size=99"], capture_output=True, text=True)
    assert fatal.returncode != 0 and "fatal path" in fatal.stderr
