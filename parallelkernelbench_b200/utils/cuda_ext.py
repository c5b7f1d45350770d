"""Compile a candidate's own CUDA source for sm_100a and load it with ctypes.

A solution file evaluated with ``launch eval --solution`` may bring its own kernel: it passes the source text to
:func:`compile_cuda_module`, gets a ``ctypes.CDLL`` back and calls its ``extern "C"`` entry points with raw pointers
(``tensor.data_ptr()``) and the current stream. The device headers of this package (``pkb/ptx.cuh``: mbarrier, TMA,
tcgen05, bounded waits; ``pkb/symm.cuh``: the symmetric-heap view and the cross-GPU barriers) are on the include path, so a
candidate builds on the same primitives as the built-in kernels.

The object is cached by a hash of source and flags; concurrent ranks serialise on a file lock, so the first rank compiles
and the others load the result - the "rank 0 compiles, then barrier" idiom of the reference's examples without needing a
barrier (reference: utils/cuda_helpers.py:14-47, kernelgen/solution_new_add_cuda.py:98-100, scripts/worker.py:49-55).
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
from pathlib import Path

_PKG = Path(__file__).resolve().parent.parent
INCLUDE_DIR = _PKG / "csrc" / "include"
BASE_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
              "-shared", "-Xcompiler", "-fPIC")
_loaded: dict[str, ctypes.CDLL] = {}


def cache_dir() -> Path:
    d = Path(os.environ.get("PKB_EXT_DIR") or (Path.home() / ".cache" / "parallelkernelbench_b200" / "ext"))
    d.mkdir(parents=True, exist_ok=True)
    return d


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def compile_cuda_module(source: str, name: str = "candidate", extra_flags: tuple[str, ...] = (), link_cuda: bool = True) -> ctypes.CDLL:
    """Build ``source`` (CUDA C++ with ``extern "C"`` entry points) into a shared object for sm_100a and load it.

    Compilation errors raise ``RuntimeError`` with nvcc's output. ``extra_flags`` are appended to the nvcc command
    (for example ``("-Xptxas", "-v")``); ``-gencode arch=compute_100a,code=sm_100a`` is always used. Source that names a
    cluster-multicast bulk/tensor load, a batched memcpy entry point or a device trap is refused with
    ``ForbiddenSourceError`` (see ``utils/source_screen.py``)."""
    from .source_screen import require_clean

    require_clean(source, f"CUDA source '{name}'")      # before nvcc: nothing forbidden is ever built, let alone launched
    flags = (*BASE_FLAGS, *extra_flags)
    key = hashlib.sha256(("\0".join(flags) + "\0" + source).encode()).hexdigest()[:24]
    if key in _loaded:
        return _loaded[key]
    d = cache_dir() / f"{name}_{key}"
    d.mkdir(parents=True, exist_ok=True)
    so, cu, lock = d / f"{name}.so", d / f"{name}.cu", d / ".lock"
    with open(lock, "w") as lf:
        fcntl.flock(lf, fcntl.LOCK_EX)                  # one rank compiles, the others wait here and then load
        try:
            if not so.exists():
                cu.write_text(source)
                tmp = d / f"{name}.so.tmp{os.getpid()}"
                cmd = [_nvcc(), *flags, f"-I{INCLUDE_DIR}", str(cu), "-o", str(tmp)]
                if link_cuda:
                    cmd += ["-lcudart_static", "-ldl", "-lrt", "-lpthread"]
                res = subprocess.run(cmd, capture_output=True, text=True)
                if res.returncode != 0:
                    tmp.unlink(missing_ok=True)
                    raise RuntimeError(f"nvcc failed ({res.returncode}) for {cu}:\n{res.stdout}\n{res.stderr}")
                (d / "nvcc.log").write_text(res.stdout + res.stderr)
                os.replace(tmp, so)                     # a loader never sees a half-written object
        finally:
            fcntl.flock(lf, fcntl.LOCK_UN)
    lib = ctypes.CDLL(str(so))
    _loaded[key] = lib
    return lib
