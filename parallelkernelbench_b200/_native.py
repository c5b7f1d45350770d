"""ctypes bindings to the two prebuilt native libraries.

``cuda_lib()`` returns ``libpkb200_cuda.so`` (hand-written sm_100a kernels + the CUDA runtime
pieces), ``host_lib()`` returns ``libpkb200_host.so`` (CPU twin of the symmetric heap). Both are
built in-tree by :mod:`parallelkernelbench_b200.build`; nothing is compiled at import or run time.

There is deliberately no PyTorch fallback for a missing CUDA library: an op whose kernel cannot be
loaded raises :class:`NativeLibraryError`, so a GPU run can never silently time eager PyTorch.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent / "_lib"
_lock = threading.Lock()
_cuda = None
_host = None


class NativeLibraryError(RuntimeError):
    pass


class KernelStatusError(RuntimeError):
    """A kernel recorded a non-zero status word (for example a bounded wait that ran out)."""

    def __init__(self, words):
        self.words = list(words)
        names = {1: "MBARRIER_TIMEOUT", 2: "PEER_TIMEOUT", 3: "BAD_ARGUMENT", 4: "BOUNDS_VIOLATION"}
        w = self.words
        super().__init__(
            f"device status {names.get(w[0], w[0])}: kernel_id={w[1]} rank={w[2]} who={w[3]} "
            f"site={w[4]} tile={w[5]} block={w[6]} count={w[7]}"
        )


def _load(path: Path, what: str):
    if not path.exists():
        raise NativeLibraryError(
            f"{what} not found at {path}. Build it with `python -m parallelkernelbench_b200.build` "
            f"(or `python -c 'import __graft_entry__ as g; g.build()'`)."
        )
    try:
        return ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
    except OSError as e:  # pragma: no cover - depends on the machine
        raise NativeLibraryError(f"cannot load {path}: {e}") from e


def cuda_lib():
    global _cuda
    with _lock:
        if _cuda is None:
            # debug variants: PKB_JITTER=1 -> random pauses around signals and waits; PKB_DEBUG_BOUNDS=1 -> checked
            # symmetric-heap bases (violations recorded in the status block, the access redirected to a scratch line)
            name = "libpkb200_cuda.so"
            if os.environ.get("PKB_JITTER") == "1":
                name = "libpkb200_cuda_jitter.so"
            elif os.environ.get("PKB_DEBUG_BOUNDS") == "1":
                name = "libpkb200_cuda_bounds.so"
            lib = _load(_LIB_DIR / name, "CUDA kernel library")
            lib.pkb_last_error.restype = ctypes.c_char_p
            _cuda = lib
        return _cuda


def host_lib():
    global _host
    with _lock:
        if _host is None:
            lib = _load(_LIB_DIR / "libpkb200_host.so", "host shared-memory library")
            lib.pkbh_last_error.restype = ctypes.c_char_p
            _host = lib
        return _host


def cuda_lib_available() -> bool:
    return (_LIB_DIR / "libpkb200_cuda.so").exists()


def host_lib_available() -> bool:
    return (_LIB_DIR / "libpkb200_host.so").exists()


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = cuda_lib().pkb_last_error()
        raise RuntimeError(f"{what or 'native call'} failed (code {rc}): {msg.decode() if msg else ''}")


# ---- small helpers used by every op wrapper ---------------------------------------------------

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float
c_u32 = ctypes.c_uint32
c_u64 = ctypes.c_uint64


def ptr(t) -> ctypes.c_void_p:
    """Raw device (or host) pointer of a tensor; ``None`` maps to NULL."""
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def current_stream() -> ctypes.c_void_p:
    import torch

    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def read_status() -> list[int]:
    buf = (ctypes.c_uint32 * 16)()
    check(cuda_lib().pkb_status_read(buf), "pkb_status_read")
    return list(buf)


def clear_status() -> None:
    check(cuda_lib().pkb_status_clear(), "pkb_status_clear")


def raise_on_status(sync: bool = True) -> None:
    """Synchronise (optionally) and raise :class:`KernelStatusError` if any kernel gave up a wait."""
    if sync:
        import torch

        torch.cuda.synchronize()
    w = read_status()
    if w[0] != 0:
        clear_status()
        raise KernelStatusError(w)


# Count of kernels launched through this module's wrappers (bench.py reports it).
_launches = 0


def count_launch(n: int = 1) -> None:
    global _launches
    _launches += n


def launches() -> int:
    return _launches


def debug_env(name: str, default: str = "") -> str:
    return os.environ.get(name, default)
