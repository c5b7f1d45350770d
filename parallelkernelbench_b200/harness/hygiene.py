"""Pre/post-job hygiene of the launcher.

Between jobs the launcher removes what a crashed job of OURS may have left behind: shared-memory
segments of the CPU heap (``/dev/shm/pkb200_*``) and rendezvous leftovers, and it reaps the exact
process group it started. It never kills by pattern and never touches GPU settings. The reference's
queue worker brackets every job with a similar clean-up and a device health check
(reference: run_together/worker.py:62-188).
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess


def clean_shared_segments(prefix: str = "pkb200_") -> list[str]:
    removed = []
    for p in glob.glob(f"/dev/shm/{prefix}*"):
        try:
            os.unlink(p)
            removed.append(p)
        except OSError:
            pass
    return removed


def gpu_health() -> dict:
    """Read-only device listing (``nvidia-smi -L``); ``{"ok": False}`` when there is no driver."""
    exe = shutil.which("nvidia-smi")
    if exe is None:
        return {"ok": False, "gpus": 0, "detail": "nvidia-smi not found"}
    try:
        r = subprocess.run([exe, "-L"], capture_output=True, text=True, timeout=30)
    except (OSError, subprocess.TimeoutExpired) as e:
        return {"ok": False, "gpus": 0, "detail": str(e)}
    n = sum(1 for ln in r.stdout.splitlines() if ln.startswith("GPU "))
    return {"ok": r.returncode == 0 and n > 0, "gpus": n, "detail": r.stdout.strip()[:400]}


def between_jobs() -> dict:
    return {"removed_segments": clean_shared_segments()}
