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


def _owner_alive(path: str, prefix: str) -> bool:
    """Segments are named ``<prefix><pid of the creating rank>_<port>``: the owner is alive if that process exists."""
    try:
        pid = int(os.path.basename(path)[len(prefix):].split("_")[0])
    except ValueError:
        return False                      # not our naming scheme any more: a leftover of an older version
    try:
        os.kill(pid, 0)                   # signal 0: existence check only
    except ProcessLookupError:
        return False
    except PermissionError:
        return True
    return True


def clean_shared_segments(prefix: str = "pkb200_", directory: str = "/dev/shm") -> list[str]:
    """Remove shared-memory segments whose creating process is gone (a job that runs next to this one keeps its heap)."""
    removed = []
    for p in glob.glob(os.path.join(directory, f"{prefix}*")):
        if _owner_alive(p, prefix):
            continue
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
