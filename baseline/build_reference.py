"""Builds the UNMODIFIED reference project (InfiniTensor/InfiniTrain) into ``baseline/_ref`` without its
third-party submodules: the sources are copied as they are, and glog / gflags / Eigen are replaced by
the small header-only stand-ins of ``baseline/shims`` (logging macros, flag parsing, the handful of
Eigen expressions the CPU kernels use).  Everything else -- the framework, its CUDA kernels, cuBLAS and
NCCL calls, the stock ``example/gpt2`` and ``example/llama3`` trainers -- is compiled from the
reference's own files with the flags of its CMakeLists.txt (C++20, ``--expt-extended-lambda
--expt-relaxed-constexpr``, USE_CUDA / USE_NCCL / USE_OMP), for sm_100 instead of its 75/80/90 list.

    python baseline/build_reference.py [--src <reference checkout>] [--jobs 8] [--cpu-only]

Outputs ``baseline/_ref/bin/{gpt2,llama3}``; needs nvcc but no GPU.  ``--cpu-only`` is the reference's
``USE_CUDA=OFF`` configuration (its CMakeLists.txt:64-73: no ``.cu`` file, no ``runtime/cuda`` or
``ccl/cuda`` sources): ``baseline/_ref/bin/{gpt2,llama3}_cpu`` run on a machine without a CUDA driver
and give the reference's own fp32 loss trajectory for parity checks.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CUDA = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))


def run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)) + "\n" + (r.stdout + r.stderr)[-6000:])


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=os.environ.get("ITB_REFERENCE_SRC")
                    or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"),
                    help="the reference checkout (default: ITB_REFERENCE_SRC, else a directory named 'reference' "
                         "beside this repository)")
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    ap.add_argument("--arch", default="100")
    ap.add_argument("--cpu-only", action="store_true")
    args = ap.parse_args()
    src = Path(args.src)
    out = HERE / "_ref"
    ref = out / "reference"
    build = out / "build"
    if ref.exists() and not args.cpu_only:
        shutil.rmtree(ref)
    if not ref.exists():
        shutil.copytree(src, ref, ignore=shutil.ignore_patterns(".git", "third_party", "docs"))
    build.mkdir(parents=True, exist_ok=True)
    (out / "bin").mkdir(parents=True, exist_ok=True)

    lib_cc = sorted((ref / "infini_train" / "src").rglob("*.cc"))
    lib_cu = sorted((ref / "infini_train" / "src").rglob("*.cu"))
    common = [ref / "example/common/tiny_shakespeare_dataset.cc", ref / "example/common/utils.cc",
              ref / "example/common/tokenizer.cc"]
    exes = {"gpt2": [ref / "example/gpt2/main.cc", ref / "example/gpt2/checkpoint_loader.cc"] + common,
            "llama3": [ref / "example/llama3/main.cc", ref / "example/llama3/checkpoint_loader.cc"] + common}
    defs = ["-DUSE_CUDA=1", "-DUSE_NCCL=1", "-DUSE_OMP=1"]
    inc = [f"-I{ref}", f"-I{HERE / 'shims'}", f"-I{CUDA / 'include'}"]
    suffix, tag = "", ""
    if args.cpu_only:
        lib_cc = [p for p in lib_cc if "runtime/cuda/" not in str(p) and "ccl/cuda/" not in str(p)]
        lib_cu = []
        defs = ["-DUSE_OMP=1"]
        inc = inc[:2]
        suffix, tag = "_cpu", "cpu__"
    cxx = ["g++", "-std=c++20", "-O2", "-fopenmp", "-fPIC", "-w", *defs, *inc]
    nvcc = [str(CUDA / "bin" / "nvcc"), "-std=c++20", "-O2", "--expt-extended-lambda", "--expt-relaxed-constexpr",
            "-gencode", f"arch=compute_{args.arch},code=sm_{args.arch}", "-Xcompiler", "-fopenmp,-fPIC,-w", "-w",
            *defs, *inc]

    def obj_of(p: Path) -> Path:
        return build / (tag + str(p.relative_to(ref)).replace("/", "__") + ".o")

    jobs = []
    all_src = lib_cc + lib_cu + sorted({p for v in exes.values() for p in v})
    for p in all_src:
        o = obj_of(p)
        if o.exists() and o.stat().st_mtime > p.stat().st_mtime:
            continue
        jobs.append((nvcc if p.suffix == ".cu" else cxx) + ["-c", str(p), "-o", str(o)])
    print(f"[reference] compiling {len(jobs)} of {len(all_src)} files with {args.jobs} jobs", flush=True)
    failed = []

    def work(cmd):
        try:
            run(cmd)
        except RuntimeError as e:
            failed.append(str(e))

    with ThreadPoolExecutor(args.jobs) as ex:
        list(ex.map(work, jobs))
    if failed:
        print(f"[reference] {len(failed)} files failed; first error:\n{failed[0]}", file=sys.stderr)
        return 1
    lib_objs = [str(obj_of(p)) for p in lib_cc + lib_cu]
    libs = [f"-L{CUDA / 'lib64'}", f"-L{CUDA / 'lib64' / 'stubs'}", "-lcudart", "-lcublas", "-lcuda", "-lnccl",
            "-fopenmp", "-lpthread", "-ldl"]
    if args.cpu_only:
        libs = ["-fopenmp", "-lpthread", "-ldl"]
    for name, files in exes.items():
        run(["g++", "-o", str(out / "bin" / (name + suffix)), *[str(obj_of(p)) for p in files], *lib_objs, *libs])
        print(f"[reference] linked {out / 'bin' / (name + suffix)}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
