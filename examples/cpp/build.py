"""Builds the C++ frontend trainer ``infinitrain_b200/bin/itb_train`` from ``examples/cpp/train.cc``
against libtorch (the one inside the installed torch package).

    python examples/cpp/build.py            # CPU / libtorch-composite build
    python examples/cpp/build.py --cuda     # + the sm_100a kernels: -DITB_WITH_CUDA, links infinitrain_b200/_C.so
    python examples/cpp/build.py --cuda --src examples/cpp/check_fused.cc --out infinitrain_b200/bin/itb_check_fused
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]


def build(cuda: bool = False, out: str | None = None, src: str | None = None) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    dst = Path(out) if out else ROOT / "infinitrain_b200" / "bin" / ("itb_train_cuda" if cuda else "itb_train")
    dst.parent.mkdir(parents=True, exist_ok=True)
    srcs = [Path(src).resolve() if src else ROOT / "examples" / "cpp" / "train.cc"]
    csrc = ROOT / "infinitrain_b200" / "csrc"
    # every header the trainer sees: the frontend, the C launch interface of the kernels, the planners
    hdrs = sorted((csrc / "frontend" / "itb").glob("*.h")) + sorted((csrc / "kernels").glob("*.h")) + \
        sorted((csrc / "comm").glob("*.h")) + sorted((csrc / "runtime").glob("*.h")) + [csrc / "runtime" / "planners.cpp"]
    if dst.exists() and all(dst.stat().st_mtime > p.stat().st_mtime for p in srcs + hdrs):
        return dst
    inc = [f"-I{p}" for p in ce.include_paths(device_type="cuda" if cuda else "cpu")]
    inc.append(f"-I{ROOT / 'infinitrain_b200' / 'csrc' / 'frontend'}")
    libdir = ce.library_paths()[0]
    cmd = ["g++", "-std=c++17", "-O2", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", *inc,
           *map(str, srcs), "-o", str(dst), f"-L{libdir}", f"-Wl,-rpath,{libdir}", "-ltorch", "-ltorch_cpu", "-lc10",
           "-lpthread"]
    if cuda:
        import sysconfig

        pkg = ROOT / "infinitrain_b200"
        pylib = sysconfig.get_config_var("LIBDIR")
        # libtorch_cuda resolves NCCL, cuBLAS, ... from the wheels beside torch: a standalone binary needs
        # their directories on its run path (python gets them preloaded by `import torch`)
        nv = Path(torch.__file__).resolve().parents[1] / "nvidia"
        nvdirs = sorted(str(d) for d in nv.glob("*/lib")) if nv.is_dir() else []
        for d in nvdirs:
            cmd += [f"-L{d}", f"-Wl,-rpath,{d}"]
        if (nv / "nccl" / "include").is_dir():         # the NCCL that libtorch_cuda itself loads
            cmd += [f"-I{nv / 'nccl' / 'include'}", "-l:libnccl.so.2"]
        else:
            cmd += ["-lnccl"]
        cmd += ["-Wl,--allow-shlib-undefined"]
        cmd += ["-DITB_WITH_CUDA", f"-I{os.environ.get('CUDA_HOME', '/usr/local/cuda')}/include", "-Wl,--no-as-needed",
                "-ltorch_cuda", "-lc10_cuda", f"-L{os.environ.get('CUDA_HOME', '/usr/local/cuda')}/lib64", "-lcudart",
                # _C.so carries the kernels behind the C launch interface (and the Python bindings, hence libpython)
                str(pkg / "_C.so"), "-Wl,-rpath,$ORIGIN/..", f"-Wl,-rpath,{pkg}", "-ltorch_python", f"-L{pylib}", f"-Wl,-rpath,{pylib}",
                f"-lpython{sysconfig.get_python_version()}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + (r.stdout + r.stderr)[-6000:])
    return dst


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--cuda", action="store_true")
    ap.add_argument("--out", default=None)
    ap.add_argument("--src", default=None, help="another program on the frontend (default: examples/cpp/train.cc)")
    a = ap.parse_args()
    print(build(a.cuda, a.out, a.src))
    sys.exit(0)
