"""Algorithm selection tables: which collective algorithm to use for a message size and group size.

The thresholds live in a versioned JSON file next to this module (``collectives_b200.json``), written by the tuner
(``python -m parallelkernelbench_b200.tuning.tune`` under torchrun) from measured crossover points, so that a new machine
is re-tuned by running one command instead of editing constants. ``PKB_TUNING_FILE`` selects another file.
The reference has no counterpart: its collectives are NCCL calls (reference: reference/1_allreduce.py:10-14).
"""
from __future__ import annotations

import json
import os
from functools import lru_cache
from pathlib import Path

DEFAULT_FILE = Path(__file__).with_name("collectives_b200.json")
_FALLBACK = {"ll_max_bytes": 256 * 1024, "oneshot_max_bytes": 512 * 1024, "large": "nvls"}


@lru_cache(maxsize=4)
def load_table(path: str | None = None) -> dict:
    path = path or os.environ.get("PKB_TUNING_FILE") or str(DEFAULT_FILE)
    with open(path) as fh:
        table = json.load(fh)
    if table.get("version") != 1:
        raise ValueError(f"{path}: unsupported tuning table version {table.get('version')!r}")
    return table


def _row(section: str, world: int, table: dict | None = None) -> dict:
    sec = (table or load_table()).get(section, {})
    return {**_FALLBACK, **sec.get("default", {}), **sec.get(str(world), {})}


def all_reduce_algo(nbytes: int, world: int, *, ll_ok: bool, nvls_ok: bool, table: dict | None = None) -> str:
    """``"ll"`` (no-barrier exchange), ``"oneshot"``, ``"twoshot"`` or ``"nvls"`` for a message of ``nbytes`` on ``world``
    ranks. ``ll_ok`` / ``nvls_ok`` say whether the call qualifies for those algorithms at all (dtype, op, multicast)."""
    if world <= 1:
        return "oneshot"
    row = _row("all_reduce", world, table)
    if ll_ok and nbytes <= row["ll_max_bytes"]:
        return "ll"
    if nbytes <= row["oneshot_max_bytes"]:
        return "oneshot"
    return "nvls" if (row["large"] == "nvls" and nvls_ok) else "twoshot"


def all_gather_ll_max(world: int, table: dict | None = None) -> int:
    return int(_row("all_gather", world, table)["ll_max_bytes"])


_NVLS_OFF = 1 << 62


def all_gather_nvls_min(world: int, table: dict | None = None) -> int:
    """Shard size in bytes from which the all-gather stores through the multicast mapping instead of pulling from the peers
    (``nvls_min_bytes`` of the table's ``all_gather`` row; absent = never)."""
    return int(_row("all_gather", world, table).get("nvls_min_bytes", _NVLS_OFF))


def reduce_scatter_nvls_min(world: int, table: dict | None = None) -> int:
    """Slice size in bytes from which the reduce-scatter lets the switch add (``multimem.ld_reduce``) instead of reading the
    peers' slices one by one (``nvls_min_bytes`` of the table's ``reduce_scatter`` row; absent = never)."""
    return int(_row("reduce_scatter", world, table).get("nvls_min_bytes", _NVLS_OFF))


def broadcast_nvls_min(world: int, table: dict | None = None) -> int:
    """Message size in bytes from which a broadcast on the whole-job group is stored through the multicast mapping by its root
    (``nvls_min_bytes`` of the table's ``broadcast`` row; absent = never)."""
    return int(_row("broadcast", world, table).get("nvls_min_bytes", _NVLS_OFF))


def all_to_all_push_min(world: int, table: dict | None = None, direct: bool = False) -> int:
    """Chunk size in bytes (per destination) from which the all-to-all pushes with TMA bulk stores into the receivers instead of
    staging its input and letting the receivers pull: ``push_min_bytes`` of the table's ``all_to_all`` row, or
    ``push_direct_min_bytes`` when the result lives in the symmetric heap and needs no copy out (absent = never)."""
    row = _row("all_to_all", world, table)
    return int(row.get("push_direct_min_bytes" if direct else "push_min_bytes", _NVLS_OFF))


def thresholds_from_timings(timings: dict[str, dict[int, float]]) -> dict:
    """One table row from measured times: ``timings[algo][nbytes] = microseconds``.

    ``ll_max_bytes`` is the largest size up to which ``ll`` is the fastest algorithm without a gap, ``oneshot_max_bytes``
    the largest size (at or above it) up to which ``oneshot`` beats both large-message algorithms, and ``large`` whichever of
    ``nvls`` / ``twoshot`` is faster at the largest measured size."""
    sizes = sorted({s for t in timings.values() for s in t})
    best = {s: min((t[s], a) for a, t in timings.items() if s in t)[1] for s in sizes}
    ll_max = 0
    for s in sizes:
        if best[s] != "ll":
            break
        ll_max = s
    one_max = ll_max
    for s in sizes:
        if s <= ll_max:
            continue
        if "oneshot" not in timings or s not in timings["oneshot"]:
            break
        others = [timings[a][s] for a in ("twoshot", "nvls") if a in timings and s in timings[a]]
        if others and timings["oneshot"][s] > min(others):
            break
        one_max = s
    top = sizes[-1]
    large = "nvls" if ("nvls" in timings and top in timings["nvls"]
                       and timings["nvls"][top] <= timings.get("twoshot", {}).get(top, float("inf"))) else "twoshot"
    return {"ll_max_bytes": ll_max, "oneshot_max_bytes": max(one_max, ll_max), "large": large}
