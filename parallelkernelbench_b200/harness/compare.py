"""Per-rank output comparison.

An op returns a Tensor, a tuple/list (saved as ``{'output_0': ..}``) or a dict; ``save_output`` moves
it to CPU and writes ``rank_<r>.pt``. ``compare_dirs`` loads the reference and candidate files of
every rank and walks them recursively: dict keys must agree, sequences must have equal length,
tensor leaves are upcast to fp32 (fp64 stays fp64) and compared with ``allclose(atol, rtol)`` plus a
shape check, other leaves with ``==``. The result carries ``ok``, a ``kind`` (``match``,
``tensor_mismatch``, ``path_mismatch``, ``load_error``, ``missing_artifacts``), the first errors and
per-file max / mean absolute differences - the same semantics and vocabulary as the reference's
comparison core (reference: utils/problem_id.py:113-275, utils/input_output_tensors.py:15-45).
"""
from __future__ import annotations

import os
import re
from typing import Any

import torch

from ..utils.ragged import Ragged

_RANK_FILE = re.compile(r"^rank_(\d+)\.pt$")


def normalize_output(y: Any) -> Any:
    """Tensor stays a tensor, a ``Ragged`` result is cut to its valid length, tuple/list becomes ``{'output_i': ...}``, dicts
    are walked; all on CPU."""
    if isinstance(y, torch.Tensor):
        return y.detach().to("cpu")
    if isinstance(y, Ragged):                        # device-side length: trimmed here, outside any timed region
        return y.trimmed().detach().to("cpu")
    if isinstance(y, (tuple, list)):
        return {f"output_{i}": normalize_output(v) for i, v in enumerate(y)}
    if isinstance(y, dict):
        return {str(k): normalize_output(v) for k, v in y.items()}
    if isinstance(y, torch.Size):
        return list(y)
    return y


def save_output(y: Any, logs_dir: str, rank: int) -> str:
    os.makedirs(logs_dir, exist_ok=True)
    path = os.path.join(logs_dir, f"rank_{rank}.pt")
    torch.save(normalize_output(y), path)
    return path


def rank_files(d: str) -> dict[int, str]:
    out = {}
    if os.path.isdir(d):
        for f in os.listdir(d):
            m = _RANK_FILE.match(f)
            if m:
                out[int(m.group(1))] = os.path.join(d, f)
    return out


def _compare_leaf(a: Any, b: Any, path: str, atol: float, rtol: float, errors: list, stats: dict) -> bool:
    if isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor):
        if a.shape != b.shape:
            errors.append(f"{path}: shape {tuple(a.shape)} vs {tuple(b.shape)}")
            return False
        if a.numel() == 0:
            return True
        if a.is_complex() or b.is_complex():
            a, b = torch.view_as_real(a.to(torch.complex128)), torch.view_as_real(b.to(torch.complex128))
        up = torch.float64 if (a.dtype == torch.float64 or b.dtype == torch.float64) else torch.float32
        af, bf = a.to(up), b.to(up)
        diff = (af - bf).abs()
        finite = torch.isfinite(diff)
        mx = float(diff[finite].max()) if finite.any() else 0.0
        stats["max_abs_diff"] = max(stats.get("max_abs_diff", 0.0), mx)
        stats["mean_abs_diff"] = max(stats.get("mean_abs_diff", 0.0), float(diff[finite].mean()) if finite.any() else 0.0)
        # NaN never matches, not even NaN (torch.allclose without equal_nan, as the reference's gate: run_local.py:523-525)
        if not torch.allclose(af, bf, atol=atol, rtol=rtol):
            bad = int((~torch.isclose(af, bf, atol=atol, rtol=rtol)).sum())
            errors.append(f"{path}: {bad}/{a.numel()} elements differ (max abs diff {mx:.4g}, atol {atol}, rtol {rtol})")
            return False
        return True
    if isinstance(a, dict) and isinstance(b, dict):
        if set(a.keys()) != set(b.keys()):
            errors.append(f"{path}: keys {sorted(a.keys())} vs {sorted(b.keys())}")
            return False
        ok = True
        for k in sorted(a.keys()):
            ok = _compare_leaf(a[k], b[k], f"{path}.{k}", atol, rtol, errors, stats) and ok
        return ok
    if isinstance(a, (list, tuple)) and isinstance(b, (list, tuple)):
        if len(a) != len(b):
            errors.append(f"{path}: length {len(a)} vs {len(b)}")
            return False
        ok = True
        for i, (x, y) in enumerate(zip(a, b)):
            ok = _compare_leaf(x, y, f"{path}[{i}]", atol, rtol, errors, stats) and ok
        return ok
    if type(a) is not type(b) and not (isinstance(a, (int, float)) and isinstance(b, (int, float))):
        errors.append(f"{path}: type {type(a).__name__} vs {type(b).__name__}")
        return False
    if a != b:
        errors.append(f"{path}: value {a!r} vs {b!r}")
        return False
    return True


def compare_objects(a: Any, b: Any, atol: float = 1e-2, rtol: float = 1e-2) -> dict:
    errors: list[str] = []
    stats: dict = {}
    ok = _compare_leaf(a, b, "out", atol, rtol, errors, stats)
    return {"ok": ok, "errors": errors[:16], **stats}


STRICT_ATOL = STRICT_RTOL = 1e-2        # the gate of the reference harness (reference: run_local.py:523-525)


def accuracy_gate(ref: Any, cand: Any, atol: float, rtol: float, oracle=None) -> dict:
    """One implementation's output against the reference's, for gates that may be looser than 1e-2 / 1e-2.

    ``strict``: the candidate is within 1e-2 / 1e-2 of the reference - the reference harness's own criterion.
    ``oracle``: it is not, but it is within the op's gate AND ``oracle()`` (the reference code on the same inputs widened
    to fp32; called only when needed) shows the candidate at most twice as far from the fp32 result as the low-precision
    reference is, in max and in mean absolute error. A candidate that merely fits the loose gate fails.
    ``op_override_unverified``: no fp32 run is possible for the op, the op gate alone decided.
    Returns the comparison dict plus ``gate`` (and ``oracle_err`` when the fp32 run was used)."""
    strict = compare_objects(ref, cand, STRICT_ATOL, STRICT_RTOL)
    if strict["ok"]:
        return dict(strict, gate="strict")
    if atol <= STRICT_ATOL and rtol <= STRICT_RTOL:
        return dict(compare_objects(ref, cand, atol, rtol), gate="op")
    res = dict(compare_objects(ref, cand, atol, rtol), gate="op_override_unverified")
    if not res["ok"] or oracle is None:
        return res
    try:
        exact = oracle()
    except Exception as e:          # the reference code cannot run in fp32 for this op
        return dict(res, oracle_err=f"unavailable: {type(e).__name__}: {e}"[:200])
    if exact is None:
        return res
    e_ref = compare_objects(exact, ref, float("inf"), 0.0)
    e_cand = compare_objects(exact, cand, float("inf"), 0.0)
    if not (e_ref["ok"] and e_cand["ok"]):
        return dict(res, oracle_err="unusable: " + "; ".join((e_ref["errors"] + e_cand["errors"])[:2]))
    errs = {"ref_max": e_ref.get("max_abs_diff", 0.0), "ours_max": e_cand.get("max_abs_diff", 0.0),
            "ref_mean": e_ref.get("mean_abs_diff", 0.0), "ours_mean": e_cand.get("mean_abs_diff", 0.0)}
    earned = errs["ours_max"] <= 2.0 * errs["ref_max"] + 1e-3 and errs["ours_mean"] <= 2.0 * errs["ref_mean"] + 1e-4
    res.update(gate="oracle", oracle_err=errs)
    if not earned:
        res["ok"] = False
        res["errors"] = [f"within the op gate but further from the fp32 result than twice the reference's own error: {errs}"] + res["errors"]
    return res


def compare_dirs(ref_dir: str, cand_dir: str, atol: float = 1e-2, rtol: float = 1e-2, expected_ranks: int | None = None) -> dict:
    """Compare ``rank_<r>.pt`` of two job directories. Never raises."""
    ref, cand = rank_files(ref_dir), rank_files(cand_dir)
    if not ref or not cand or (expected_ranks is not None and (len(ref) < expected_ranks or len(cand) < expected_ranks)):
        return {"ok": False, "kind": "missing_artifacts", "errors": [f"reference files: {sorted(ref)}, candidate files: {sorted(cand)}"],
                "per_file": []}
    if set(ref) != set(cand):
        return {"ok": False, "kind": "path_mismatch", "errors": [f"rank sets differ: {sorted(ref)} vs {sorted(cand)}"], "per_file": []}
    per_file, errors, all_ok, kind = [], [], True, "match"
    for r in sorted(ref):
        try:
            a = torch.load(ref[r], map_location="cpu", weights_only=False)
            b = torch.load(cand[r], map_location="cpu", weights_only=False)
        except Exception as e:  # corrupt or truncated artifact
            per_file.append({"file": f"rank_{r}.pt", "ok": False, "detail": f"load error: {e}"})
            errors.append(f"rank {r}: load error: {e}")
            all_ok, kind = False, "load_error"
            continue
        res = compare_objects(a, b, atol, rtol)
        per_file.append({"file": f"rank_{r}.pt", "ok": res["ok"], "max_abs_diff": res.get("max_abs_diff"),
                         "mean_abs_diff": res.get("mean_abs_diff"), "detail": "; ".join(res["errors"][:3])})
        if not res["ok"]:
            all_ok = False
            if kind == "match":
                kind = "tensor_mismatch"
            errors.extend(f"rank {r}: {e}" for e in res["errors"][:4])
    return {"ok": all_ok, "kind": kind if not all_ok else "match", "errors": errors[:16], "per_file": per_file}
