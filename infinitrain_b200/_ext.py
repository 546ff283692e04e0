"""Build and load the native extension ``infinitrain_b200._C``.

The extension is built IN-TREE (``infinitrain_b200/_C.so``) for sm_100a only, with
``-gencode arch=compute_100a,code=sm_100a``.  A hash of the sources is stored beside the ``.so``; the
library is rebuilt only when the sources changed, so a machine that receives a prebuilt ``.so``
imports it directly and never runs the compiler.

On a machine with a GPU a missing or unloadable extension is an error (the CUDA path must never
fall back silently to PyTorch eager ops); on a CPU-only machine ``load()`` returns ``None`` when the
library cannot be loaded and the ops use their PyTorch reference implementations.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_CSRC = _PKG / "csrc"
_SO = _PKG / "_C.so"
_HASH = _PKG / "_C.hash"
_BUILD = _PKG / "csrc" / "build"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

_module = None
_load_error: Exception | None = None


def sources() -> list[Path]:
    out = []
    for pat in ("*.cpp", "kernels/*.cu", "comm/*.cu", "comm/*.cpp", "runtime/*.cpp", "runtime/*.cu"):
        out += sorted(_CSRC.glob(pat))
    return out


def _headers() -> list[Path]:
    out = []
    for pat in ("common/*.cuh", "common/*.h", "kernels/*.h", "kernels/*.cuh", "comm/*.h", "comm/*.cuh",
                "runtime/*.h", "launcher/*.cc"):
        out += sorted(_CSRC.glob(pat))
    return out


def source_hash() -> str:
    h = hashlib.sha256()
    for p in sources() + _headers():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def is_built() -> bool:
    return _SO.exists() and _HASH.exists() and _HASH.read_text().strip() == source_hash()


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile every source for sm_100a and link ``_C.so`` in-tree.  Needs nvcc, no GPU."""
    if is_built() and not force:
        return _SO
    import torch
    from torch.utils import cpp_extension as ce

    _BUILD.mkdir(parents=True, exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    inc = [f"-I{p}" for p in ce.include_paths(device_type="cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    common = ["-O3", "-std=c++17", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H", abi]
    objs, jobs = [], []
    for src in sources():
        obj = _BUILD / (src.stem + ".o")
        stamp = _BUILD / (src.stem + ".hash")
        h = hashlib.sha256(src.read_bytes() + b"".join(p.read_bytes() for p in _headers())).hexdigest()
        objs.append(str(obj))
        if obj.exists() and stamp.exists() and stamp.read_text() == h and not force:
            continue
        if src.suffix == ".cu":
            cmd = [nvcc, *NVCC_ARCH, "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
                   *common, *inc, "-c", str(src), "-o", str(obj)]
        else:
            cmd = ["g++", "-fPIC", "-Wno-unused-variable", *common, *inc, "-c", str(src), "-o", str(obj)]
        jobs.append((cmd, stamp, h))
    if verbose:
        print(f"[infinitrain_b200] compiling {len(jobs)} of {len(objs)} native sources", file=sys.stderr)

    def work(job):
        cmd, stamp, h = job
        _run(cmd)
        stamp.write_text(h)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(work, jobs))
    libdirs = ce.library_paths(device_type="cuda")
    link = ["g++", "-shared", *objs, "-o", str(_SO)]
    for d in libdirs:
        link += [f"-L{d}", f"-Wl,-rpath,{d}"]
    link += ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart"]
    _run(link)
    build_launcher()
    _HASH.write_text(source_hash())
    return _SO


def launcher_path() -> Path:
    return _PKG / "bin" / "infini_run"


def build_launcher() -> Path:
    """Compile the standalone C++ launcher (one process per local rank, rendezvous environment)."""
    out = launcher_path()
    out.parent.mkdir(parents=True, exist_ok=True)
    _run(["g++", "-O2", "-std=c++17", str(_CSRC / "launcher" / "infini_run.cc"), "-o", str(out)])
    return out


def load(required: bool | None = None):
    """Import ``_C``; build it first when nvcc is available and the library is stale or missing.

    ``required`` defaults to "a CUDA device is visible": then any failure raises.
    """
    global _module, _load_error
    if _module is not None:
        return _module
    import torch

    if required is None:
        required = torch.cuda.is_available()
    try:
        if not is_built():
            if _SO.exists() and os.environ.get("ITB_NO_REBUILD") == "1":
                pass  # use the shipped library as is
            else:
                build()
        spec = importlib.util.spec_from_file_location("infinitrain_b200._C", str(_SO))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _module = mod
        return mod
    except Exception as e:  # noqa: BLE001
        _load_error = e
        if required:
            raise RuntimeError(
                "infinitrain_b200: the native extension (_C.so) is required on a GPU machine and "
                f"could not be built or loaded: {e}") from e
        return None


def available() -> bool:
    return load(required=False) is not None
