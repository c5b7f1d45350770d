"""Sample GPU clocks and throttle reasons while a timed region runs.

A background ``nvidia-smi`` process (query mode, read-only) writes one CSV line every 200 ms;
``summary()`` reduces it to the median SM clock under load and the set of throttle reasons seen.
Nothing here changes any GPU setting.
"""
from __future__ import annotations

import os
import shutil
import signal
import statistics
import subprocess
import tempfile
import time

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def gpu_selector(device=None, gpu_index: int = 0) -> str:
    """What to pass to ``nvidia-smi -i`` for a torch device: its UUID. ``nvidia-smi`` numbers physical GPUs, a process
    numbers the GPUs it can see, so under CUDA_VISIBLE_DEVICES an index would select somebody else's GPU."""
    if device is not None:
        try:
            import torch

            return "GPU-" + str(torch.cuda.get_device_properties(device).uuid)
        except Exception:
            pass
    vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    ids = [v.strip() for v in vis.split(",") if v.strip()]
    if ids and gpu_index < len(ids):
        return ids[gpu_index]                 # a physical index or a UUID: both are accepted by -i
    return str(gpu_index)


class ClockSampler:
    def __init__(self, gpu_index: int = 0, period_ms: int = 200, path: str | None = None, device=None):
        self.gpu_index = gpu_selector(device, gpu_index)
        self.period_ms = period_ms
        self.path = path or os.path.join(tempfile.gettempdir(), f"pkb_clocks_{os.getpid()}.csv")
        self.proc = None

    def start(self) -> "ClockSampler":
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return self
        self._fh = open(self.path, "w")
        self.proc = subprocess.Popen(
            [exe, f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index),
             "-lms", str(self.period_ms)], stdout=self._fh, stderr=subprocess.DEVNULL)
        return self

    def stop(self) -> None:
        if self.proc is not None:
            self.proc.send_signal(signal.SIGTERM)
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self._fh.close()
            self.proc = None

    def summary(self) -> dict:
        """``{"sm_mhz": median under load, "sm_max_mhz": .., "reasons": [...], "samples": n}``."""
        rows = parse_clock_csv(self.path) if os.path.exists(self.path) else []
        return summarize_clock_rows(rows)

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        time.sleep(self.period_ms / 1000.0)
        self.stop()


def parse_clock_csv(path: str) -> list[dict]:
    rows = []
    with open(path) as fh:
        for line in fh:
            parts = [p.strip() for p in line.strip().split(",")]
            if len(parts) < 9:
                continue
            try:
                rows.append({"sm": float(parts[1]), "sm_max": float(parts[2]), "power": float(parts[3]),
                             "active": parts[4], "hw_slowdown": parts[5], "hw_thermal": parts[6],
                             "sw_thermal": parts[7], "sw_power_cap": parts[8]})
            except ValueError:
                continue
    return rows


def summarize_clock_rows(rows: list[dict]) -> dict:
    if not rows:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    pmax = max(r["power"] for r in rows)
    loaded = [r for r in rows if r["power"] >= 0.5 * pmax] or rows
    reasons = set()
    for r in rows:
        for key, name in (("hw_slowdown", "hw_slowdown"), ("hw_thermal", "hw_thermal_slowdown"),
                          ("sw_thermal", "sw_thermal_slowdown"), ("sw_power_cap", "sw_power_cap")):
            if r[key].lower().startswith("active"):
                reasons.add(name)
    return {"sm_mhz": statistics.median(r["sm"] for r in loaded), "sm_max_mhz": max(r["sm_max"] for r in rows),
            "power_w_max": pmax, "reasons": sorted(reasons), "samples": len(rows)}
