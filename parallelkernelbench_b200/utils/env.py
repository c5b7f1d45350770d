"""Environment facts and debug toggles (read once, in one place).

Debug toggles are environment variables because they must reach every rank of a torchrun job:

``PKB_WAIT_BUDGET_MS``  budget of device-side waits (default 4000; tests of the time-out path use ~5)
``PKB_COOLDOWN_SEC``    pause between the reference job and the candidate job (default 0.5,
                        same purpose as reference: run_local.py:57)
``PKB_VERBOSE``         print the torchrun command lines
"""
from __future__ import annotations

import json
import os
from pathlib import Path

REPO_ROOT = Path(__file__).resolve().parents[2]


def wait_budget_ns() -> int:
    return int(float(os.environ.get("PKB_WAIT_BUDGET_MS", "4000")) * 1e6)


def cooldown_sec() -> float:
    return float(os.environ.get("PKB_COOLDOWN_SEC", "0.5"))


def verbose() -> bool:
    return os.environ.get("PKB_VERBOSE", "0") not in ("", "0")


_FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
# measured on this pool: peer copy per direction, 8-rank all-reduce bus bandwidth at 1 GiB
NVLINK_GBS_PER_DIR = 770.0
NVLINK_GBS_NOMINAL = 900.0
ALLREDUCE_BUS_GBS = 725.0


def measured_peaks() -> dict:
    """Roofline denominators: the driver-written measurement if present, else the stated fallback."""
    p = REPO_ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            d["source"] = "measured"
            return d
        except (OSError, ValueError):
            pass
    return dict(_FALLBACK_PEAKS)


def git_sha() -> str:
    head = REPO_ROOT / ".git" / "HEAD"
    try:
        ref = head.read_text().strip()
        if ref.startswith("ref:"):
            return (REPO_ROOT / ".git" / ref.split(" ", 1)[1]).read_text().strip()[:12]
        return ref[:12]
    except OSError:
        return "unknown"
