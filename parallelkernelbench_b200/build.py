"""Ahead-of-time build of the native libraries, in-tree.

Two shared objects are produced under ``parallelkernelbench_b200/_lib/``:

* ``libpkb200_cuda.so``  - every ``csrc/kernels/*.cu`` and ``csrc/runtime/*.cu`` compiled by nvcc for
  sm_100a only (``-gencode arch=compute_100a,code=sm_100a -lineinfo``). nvcc cross-compiles, so this
  works on a machine without a GPU.
* ``libpkb200_host.so``  - ``csrc/runtime/*.cpp`` compiled by g++: the CPU twin of the symmetric
  heap and its collectives (shared-memory ranks, ``std::atomic`` flags), usable with no CUDA at all.

There is no JIT at run time: ranks load the prebuilt objects with ctypes, which replaces the
reference's per-rank ``load_inline`` cache juggling (reference: utils/cuda_helpers.py:14-47,
scripts/worker.py:49-55).

Usage: ``python -m parallelkernelbench_b200.build [--force] [--verbose] [--ptxas-info] [--jitter] [--debug-bounds]``
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = CSRC / "include"
OUT_DIR = PKG / "_lib"
OBJ_DIR = PKG.parent / "build" / "obj"

CUDA_LIB = OUT_DIR / "libpkb200_cuda.so"
# debug variants of the CUDA library: same sources, one extra define, selected at load time by an environment variable
#   jitter: -DPKB_JITTER        random pauses around system-scope signals and waits      (PKB_JITTER=1)
#   bounds: -DPKB_DEBUG_BOUNDS  checked bases of symmetric-heap accesses, recorded not trapped (PKB_DEBUG_BOUNDS=1)
VARIANTS = {"jitter": "PKB_JITTER", "bounds": "PKB_DEBUG_BOUNDS"}
CUDA_LIB_JITTER = OUT_DIR / "libpkb200_cuda_jitter.so"
HOST_LIB = OUT_DIR / "libpkb200_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=default",
]
GXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-pthread", "-Wall"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def _headers_mtime() -> float:
    return max((p.stat().st_mtime for p in INCLUDE.rglob("*") if p.is_file()), default=0.0)


def cuda_sources() -> list[Path]:
    return sorted(list((CSRC / "kernels").glob("*.cu")) + list((CSRC / "runtime").glob("*.cu")))


def host_sources() -> list[Path]:
    return sorted((CSRC / "runtime").glob("*.cpp"))


def _run(cmd: list[str], verbose: bool) -> str:
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"command failed ({res.returncode}): {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    return res.stdout + res.stderr


def _compile_one(src: Path, obj: Path, force: bool, verbose: bool, ptxas_info: bool, hdr_mtime: float,
                 defines: tuple[str, ...] = ()) -> str:
    if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_mtime):
        return ""
    if src.suffix == ".cu":
        cmd = [_nvcc(), *NVCC_FLAGS, *[f"-D{d}" for d in defines], f"-I{INCLUDE}", "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
    else:
        cmd = ["g++", *GXX_FLAGS, f"-I{INCLUDE}", "-c", str(src), "-o", str(obj)]
    return _run(cmd, verbose)


def build_all(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> dict[str, Path]:
    """Compile whatever is out of date and link both libraries. Returns their paths."""
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    hdr_mtime = _headers_mtime()
    cu = cuda_sources()
    cpp = host_sources()
    jobs = [(s, OBJ_DIR / (s.stem + ("_cu.o" if s.suffix == ".cu" else "_cpp.o"))) for s in cu + cpp]
    logs = []
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        futs = {ex.submit(_compile_one, s, o, force, verbose, ptxas_info, hdr_mtime): s for s, o in jobs}
        for f in cf.as_completed(futs):
            out = f.result()
            if out and (verbose or ptxas_info):
                logs.append(f"== {futs[f].name}\n{out}")
    if logs:
        print("\n".join(logs))
    cu_objs = [str(o) for s, o in jobs if s.suffix == ".cu"]
    cpp_objs = [str(o) for s, o in jobs if s.suffix == ".cpp"]
    if cu_objs:
        newest = max(Path(o).stat().st_mtime for o in cu_objs)
        if force or not CUDA_LIB.exists() or CUDA_LIB.stat().st_mtime < newest:
            _run([_nvcc(), "-shared", "-o", str(CUDA_LIB), *cu_objs, "-lcudart_static", "-ldl", "-lrt", "-lpthread"], verbose)
    if cpp_objs:
        newest = max(Path(o).stat().st_mtime for o in cpp_objs)
        if force or not HOST_LIB.exists() or HOST_LIB.stat().st_mtime < newest:
            _run(["g++", "-shared", "-o", str(HOST_LIB), *cpp_objs, "-pthread", "-lrt"], verbose)
    return {"cuda": CUDA_LIB, "host": HOST_LIB}


def build_variant(variant: str, force: bool = False, verbose: bool = False) -> Path:
    """A debug variant of the CUDA library (see ``VARIANTS``): ``_lib/libpkb200_cuda_<variant>.so``."""
    define = VARIANTS[variant]
    out = OUT_DIR / f"libpkb200_cuda_{variant}.so"
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = OBJ_DIR.parent / f"obj_{variant}"
    obj_dir.mkdir(parents=True, exist_ok=True)
    hdr_mtime = _headers_mtime()
    jobs = [(s, obj_dir / (s.stem + "_cu.o")) for s in cuda_sources()]
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for f in [ex.submit(_compile_one, s, o, force, verbose, False, hdr_mtime, (define,)) for s, o in jobs]:
            f.result()
    objs = [str(o) for _, o in jobs]
    newest = max(Path(o).stat().st_mtime for o in objs)
    if force or not out.exists() or out.stat().st_mtime < newest:
        _run([_nvcc(), "-shared", "-o", str(out), *objs, "-lcudart_static", "-ldl", "-lrt", "-lpthread"], verbose)
    return out


def build_jitter(force: bool = False, verbose: bool = False) -> Path:
    return build_variant("jitter", force, verbose)


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--jitter", action="store_true", help="also build libpkb200_cuda_jitter.so (random pauses around signals and waits)")
    ap.add_argument("--debug-bounds", action="store_true", help="also build libpkb200_cuda_bounds.so (checked symmetric-heap bases)")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / shared memory per kernel")
    args = ap.parse_args(argv)
    libs = build_all(force=args.force or args.ptxas_info, verbose=args.verbose, ptxas_info=args.ptxas_info)
    if args.jitter:
        libs["cuda_jitter"] = build_variant("jitter", force=args.force, verbose=args.verbose)
    if args.debug_bounds:
        libs["cuda_bounds"] = build_variant("bounds", force=args.force, verbose=args.verbose)
    for k, v in libs.items():
        print(f"{k}: {v} ({'ok' if v.exists() else 'missing'})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
