"""Offline inspectors of stored results (``logs/op_<name>/w<world>/<impl>/trial_<k>/``).

``inspect``   prints, per rank, shapes / dtypes and the first differing elements of the reference and
              candidate dumps, then the comparison verdict.
``perf-diff`` aggregates ``rank_<r>_perf.json`` of both implementations (mean / std / min / max over
              ranks), prints speed-up = reference max / ours max and the improvement in per cent, and
              writes ``comparison_ours.json`` beside the results.
Same roles as reference: utils/compare_outputs.py:108-336, utils/compare_performance.py:31-165.
"""
from __future__ import annotations

import glob
import json
import os
import statistics

import torch

from . import compare
from .launch import LOGS_ROOT, final_dir


def _world_of(op: str, world: int | None) -> int | None:
    if world is not None:
        return world
    cands = sorted(glob.glob(os.path.join(LOGS_ROOT, f"op_{op}", "w*")))
    return int(os.path.basename(cands[-1])[1:]) if cands else None


def _describe(x, indent="  ") -> str:
    if isinstance(x, torch.Tensor):
        return f"{indent}Tensor{tuple(x.shape)} {x.dtype} mean={x.float().mean().item():.4g} absmax={x.float().abs().max().item() if x.numel() else 0:.4g}"
    if isinstance(x, dict):
        return "\n".join(f"{indent}{k}:\n{_describe(v, indent + '  ')}" for k, v in x.items())
    return f"{indent}{type(x).__name__}: {x!r}"


def main_compare(a) -> int:
    world = _world_of(a.op, a.world)
    if world is None:
        print(f"no stored results for op {a.op} under {LOGS_ROOT}")
        return 1
    rd, cd = final_dir(a.op, "reference", a.trial, world), final_dir(a.op, "ours", a.trial, world)
    for r, path in sorted(compare.rank_files(rd).items()):
        ref = torch.load(path, map_location="cpu", weights_only=False)
        cpath = compare.rank_files(cd).get(r)
        print(f"rank {r}: reference\n{_describe(ref)}")
        if cpath is None:
            print("  (no candidate file)")
            continue
        cand = torch.load(cpath, map_location="cpu", weights_only=False)
        res = compare.compare_objects(ref, cand, a.atol, a.rtol)
        colour = "\033[32m" if res["ok"] else "\033[31m"
        print(f"  {colour}{'match' if res['ok'] else 'MISMATCH'}\033[0m max_abs_diff={res.get('max_abs_diff')}")
        for e in res["errors"][:a.max_print]:
            print(f"    {e}")
    out = compare.compare_dirs(rd, cd, a.atol, a.rtol)
    print(f"verdict: {out['kind']}")
    return 0 if out["ok"] else 1


def _perf_stats(d: str) -> dict | None:
    vals = []
    for f in sorted(glob.glob(os.path.join(d, "rank_*_perf.json"))):
        with open(f) as fh:
            vals.append(float(json.load(fh)["wall_time_ms"]))
    if not vals:
        return None
    return {"mean": statistics.mean(vals), "std": statistics.pstdev(vals), "min": min(vals), "max": max(vals), "n_ranks": len(vals)}


def main_perf(a) -> int:
    world = _world_of(a.op, a.world)
    if world is None:
        print(f"no stored results for op {a.op}")
        return 1
    ref = _perf_stats(final_dir(a.op, "reference", a.trial, world))
    ours = _perf_stats(final_dir(a.op, "ours", a.trial, world))
    if not ref or not ours:
        print("perf files missing (run eval with --measure-perf)")
        return 1
    speedup = ref["max"] / ours["max"]
    out = {"op": a.op, "world": world, "reference": ref, "ours": ours, "speedup": speedup,
           "improvement_pct": 100.0 * (ref["max"] - ours["max"]) / ref["max"]}
    print(f"reference: max {ref['max']:.4f} ms (mean {ref['mean']:.4f} +- {ref['std']:.4f}, ranks={ref['n_ranks']})")
    print(f"ours     : max {ours['max']:.4f} ms (mean {ours['mean']:.4f} +- {ours['std']:.4f}, ranks={ours['n_ranks']})")
    print(f"speedup {speedup:.2f}x ({out['improvement_pct']:.1f}% less time)")
    path = os.path.join(LOGS_ROOT, f"op_{a.op}", f"w{world}", "comparison_ours.json")
    with open(path, "w") as fh:
        json.dump(out, fh, indent=1)
    return 0
