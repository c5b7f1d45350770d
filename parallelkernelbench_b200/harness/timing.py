"""Device timing of an op with the 500 warm-up / 100 timed protocol.

* Input rotation: every *large* tensor argument (not only the first) is cloned into ``G`` groups and
  call ``i`` uses group ``i % G``; ``G = 1`` if the rotated bytes are at least 3x L2, else
  ``3*L2/bytes + 1`` capped at 128, so consecutive calls do not find their inputs in L2
  (the reference rotates only the first tensor argument: reference: utils/performance.py:41-76,
  scripts/worker.py:57-102).
* ``iters + 1`` CUDA events, one before the first call and one after each call, no host
  synchronisation inside the loop; per-iteration samples and the mean over the whole window.
* The returned dict has the reference's keys (``wall_time_ms`` ... ``timed_tensor_bytes``,
  reference: utils/performance.py:101-112) so downstream tooling carries over.
* Optional CUDA-graph mode: capture one call per input group and replay the graphs, which removes
  host launch overhead from launch-bound ops.
On CPU (gloo runs) the same loop is timed with ``time.perf_counter``.
"""
from __future__ import annotations

import time
from typing import Any, Callable

import torch

DEFAULT_L2_BYTES = 50 * 1024 * 1024
MAX_GROUPS = 128


def l2_bytes(device: torch.device) -> int:
    if device.type != "cuda":
        return DEFAULT_L2_BYTES
    try:
        n = int(torch.cuda.get_device_properties(device).L2_cache_size)
    except Exception:
        return DEFAULT_L2_BYTES
    return n if n > 0 else DEFAULT_L2_BYTES


def num_groups(input_bytes: int, l2: int) -> int:
    if input_bytes <= 0:
        return 1
    if input_bytes >= 3 * l2:
        return 1
    return int(min(max(2, 3 * l2 // input_bytes + 1), MAX_GROUPS))


def _tensor_bytes(x: Any) -> int:
    if isinstance(x, torch.Tensor):
        return x.numel() * x.element_size()
    if isinstance(x, (list, tuple)):
        return sum(_tensor_bytes(v) for v in x)
    return 0


def _clone_args(args: tuple) -> tuple:
    def c(x):
        if isinstance(x, torch.Tensor):
            return x.clone()
        if isinstance(x, list):
            return [c(v) for v in x]
        if isinstance(x, tuple):
            return tuple(c(v) for v in x)
        return x
    return tuple(c(a) for a in args)


class _Stamps:
    """Two readings of the GPU's nanosecond timer taken by one-thread kernels on the current stream."""

    def __init__(self, lib, device):
        from .. import _native as nv

        self._lib, self._nv = lib, nv
        self._buf = torch.zeros(2, dtype=torch.int64, device=device)

    def __call__(self, slot: int) -> None:
        if self._buf is None:
            return
        rc = self._lib.pkb_stamp_globaltimer(self._nv.ptr(self._buf[slot:]), self._nv.current_stream())
        if rc != 0:
            self._buf = None

    def elapsed_ms(self):
        if self._buf is None:
            return None
        a, b = (int(v) for v in self._buf.tolist())
        return (b - a) * 1e-6 if a and b and b >= a else None


def _stamper(device):
    """The device-clock cross-check is optional: without the kernel library (or with an older one) timing still works."""
    try:
        from .. import _native as nv

        lib = nv.cuda_lib()
        if not hasattr(lib, "pkb_stamp_globaltimer"):
            return None
        return _Stamps(lib, device)
    except Exception:
        return None


def measure(fn: Callable[..., Any], args: tuple, warmup: int = 500, iters: int = 100, device: torch.device | None = None,
            use_graph: bool = False, max_rotation_bytes: int = 8 << 30) -> dict:
    device = device or next((a.device for a in args if isinstance(a, torch.Tensor)), torch.device("cpu"))
    l2 = l2_bytes(device)
    nbytes = _tensor_bytes(args)
    groups = num_groups(nbytes, l2)
    while groups > 1 and groups * nbytes > max_rotation_bytes:
        groups -= 1
    arg_groups = [args] + [_clone_args(args) for _ in range(groups - 1)]
    cuda = device.type == "cuda"

    def call(i):
        return fn(*arg_groups[i % groups])

    graphs = None
    if cuda and use_graph:
        torch.cuda.synchronize()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for i in range(3):
                call(i)
        torch.cuda.current_stream().wait_stream(s)
        graphs = []
        for gidx in range(groups):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                call(gidx)
            graphs.append(g)

        def call(i):  # noqa: F811
            graphs[i % groups].replay()

    if cuda:
        torch.cuda.synchronize()
    for i in range(warmup):
        call(i)
    device_clock_ms = None
    if cuda:
        torch.cuda.synchronize()
        stamps = _stamper(device)
        events = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
        if stamps is not None:
            stamps(0)
        events[0].record()
        for i in range(iters):
            call(i)
            events[i + 1].record()
        if stamps is not None:
            stamps(1)
        torch.cuda.synchronize()
        per_iter = [float(events[i].elapsed_time(events[i + 1])) for i in range(iters)]
        total = float(events[0].elapsed_time(events[iters]))
        if stamps is not None:
            device_clock_ms = stamps.elapsed_ms()
    else:
        per_iter = []
        t_start = time.perf_counter()
        for i in range(iters):
            t0 = time.perf_counter()
            call(i)
            per_iter.append((time.perf_counter() - t0) * 1e3)
        total = (time.perf_counter() - t_start) * 1e3
    mean = total / max(iters, 1)
    var = sum((t - mean) ** 2 for t in per_iter) / (len(per_iter) - 1) if len(per_iter) > 1 else 0.0
    return {
        "wall_time_ms": mean,
        "wall_time_total_ms": total,
        "wall_time_std_ms": var ** 0.5,
        "min_time_ms": min(per_iter) if per_iter else mean,
        "max_time_ms": max(per_iter) if per_iter else mean,
        "iterations": iters,
        "warmup_iterations": warmup,
        "num_input_groups": float(groups),
        "l2_cache_size_bytes": float(l2),
        "timed_tensor_bytes": float(nbytes),
        "cuda_graph": bool(graphs),
        # the same interval on the GPU's own nanosecond timer (two one-thread stamp kernels around the loop): a cross-check of
        # the event timing; the two agree to within the launch gaps of the stamps
        "device_clock_total_ms": device_clock_ms,
    }
