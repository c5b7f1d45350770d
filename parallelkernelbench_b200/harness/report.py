"""Result bookkeeping shared by the launcher verbs.

``summarize_perf`` reduces the per-rank ``rank_<r>_perf.json`` files of a job to the job time (the
MAX over ranks - the slowest rank decides) plus mean and count; ``classify_trial`` turns the
outcome of a reference job and a candidate job into one of ``match``, ``tensor_mismatch``,
``path_mismatch``, ``load_error``, ``missing_artifacts``, ``no_artifacts``, ``harness_environment``
or ``interrupted``; ``environment_hint`` separates infrastructure failures (port clashes, NCCL
bootstrap, out of memory, missing driver) from kernel failures by pattern matching the captured
output. Same roles as reference: utils/run_utils.py:181-429.
"""
from __future__ import annotations

import glob
import json
import os

_ENV_PATTERNS = [
    ("address already in use", "rendezvous port already in use: another job holds the master port"),
    ("errno: 98", "rendezvous port already in use"),
    ("nccl error", "NCCL failed to initialise or lost a peer"),
    ("ncclsystemerror", "NCCL system error (shared memory / peer access)"),
    ("ncclunhandledcudaerror", "NCCL saw a CUDA error from an earlier launch"),
    ("cuda out of memory", "the GPU ran out of memory"),
    ("outofmemoryerror", "the GPU ran out of memory"),
    ("no cuda gpus are available", "no GPU visible to the job"),
    ("cuda driver version is insufficient", "CUDA driver too old for this runtime"),
    ("no space left on device", "disk full while writing artifacts"),
    ("timed out waiting for rank 0 to create the segment", "a CPU rank never mapped the shared segment"),
    ("connection refused", "rendezvous store unreachable"),
    ("broken pipe", "a peer process died during rendezvous"),
    ("cannot load", "native library failed to load"),
    ("not found at", "native library has not been built"),
]


def environment_hint(text: str) -> str | None:
    low = (text or "").lower()
    for pat, hint in _ENV_PATTERNS:
        if pat in low:
            return hint
    return None


def bounded_output(stdout: str, stderr: str, head: int = 32 * 1024, tail: int = 8 * 1024) -> dict:
    def clip(s, h, t):
        s = s or ""
        if len(s) <= h + t:
            return s
        return s[:h] + f"\n... [{len(s) - h - t} bytes elided] ...\n" + s[-t:]
    return {"stdout": clip(stdout, 0, tail), "stderr": clip(stderr, head, tail)}


def summarize_perf(job_dir: str) -> dict | None:
    vals, extra = [], {}
    for f in sorted(glob.glob(os.path.join(job_dir, "rank_*_perf.json"))):
        try:
            with open(f) as fh:
                d = json.load(fh)
        except (OSError, ValueError):
            continue
        vals.append(float(d["wall_time_ms"]))
        for k in ("roofline_ms", "limiter", "compute_ms", "nvlink_ms", "hbm_ms", "num_input_groups", "cuda_graph"):
            if k in d:
                extra[k] = d[k]
    if not vals:
        return None
    out = {"wall_time_ms_max": max(vals), "wall_time_ms_mean": sum(vals) / len(vals), "n_ranks": len(vals), **extra}
    if "roofline_ms" in extra:
        out["pct_of_roofline"] = 100.0 * extra["roofline_ms"] / out["wall_time_ms_max"]
    return out


def classify_trial(ref_job: dict, cand_job: dict, cmp: dict | None) -> dict:
    """``*_job`` are dicts from ``launch.run_job``; ``cmp`` the result of ``compare.compare_dirs``."""
    if ref_job.get("interrupted") or cand_job.get("interrupted"):
        return {"result": "interrupted"}
    for job in (ref_job, cand_job):
        if job["returncode"] != 0:
            hint = environment_hint(job.get("stdout", "") + job.get("stderr", ""))
            if hint:
                return {"result": "harness_environment", "harness_hint": hint, "failed_impl": job["impl"]}
    if ref_job["artifact_count"] == 0 or cand_job["artifact_count"] == 0:
        failed = ref_job if ref_job["artifact_count"] == 0 else cand_job
        return {"result": "no_artifacts", "failed_impl": failed["impl"], "returncode": failed["returncode"]}
    # a job that saved its outputs and failed afterwards (guard band overwritten, non-deterministic repeat run, a device
    # wait that ran out while being timed, a crash in the timing loop) is a failure even if the saved outputs compare equal
    if ref_job["returncode"] != 0 or ref_job.get("timed_out"):
        return {"result": "reference_failed", "failed_impl": ref_job["impl"], "returncode": ref_job["returncode"]}
    if cand_job["returncode"] != 0 or cand_job.get("timed_out"):
        return {"result": "candidate_failed", "failed_impl": cand_job["impl"], "returncode": cand_job["returncode"]}
    if cmp is None:
        return {"result": "no_artifacts"}
    return {"result": "match" if cmp["ok"] else cmp["kind"]}


def trial_line(trial: int, verdict: dict, ref_perf: dict | None, cand_perf: dict | None, gate: dict | None = None) -> str:
    s = f"trial {trial}: {verdict['result']}"
    if gate and gate.get("gate"):
        s += f" [gate: {gate['gate']}"
        if isinstance(gate.get("oracle"), dict):
            o = gate["oracle"]
            s += f", max error vs fp32: reference {o['ref_max']:.3g}, ours {o['ours_max']:.3g}"
        s += "]"
    if ref_perf and cand_perf:
        r, c = ref_perf["wall_time_ms_max"], cand_perf["wall_time_ms_max"]
        s += f" | ref {r:.4f} ms | ours {c:.4f} ms | speedup {r / c:.2f}x"
        if "pct_of_roofline" in cand_perf:
            s += f" | {cand_perf['pct_of_roofline']:.1f}% of roofline ({cand_perf.get('limiter')})"
    if verdict.get("harness_hint"):
        s += f" | environment: {verdict['harness_hint']}"
    return s


def ledger_rows(path: str, latest_only: bool = True) -> list[dict]:
    """Cells of a sweep ledger (one JSON object per line). With ``latest_only`` a later line for the same
    (op, world, config) replaces an earlier one, so a re-run after a fix supersedes the failed cell."""
    import json

    rows: dict[tuple, dict] | list = {} if latest_only else []
    with open(path) as fh:
        for line in fh:
            line = line.strip()
            if not line:
                continue
            try:
                d = json.loads(line)
            except ValueError:
                continue
            if "op" not in d or "world" not in d:
                continue
            if latest_only:
                rows[(d["op"], d["world"], d.get("config", "default"))] = d
            else:
                rows.append(d)
    out = list(rows.values()) if latest_only else rows
    return sorted(out, key=lambda d: (d["op"], d.get("config", "default"), d["world"]))


_COLUMNS = (("op", "op"), ("config", "config"), ("world", "GPUs"), ("result", "result"), ("gate", "gate"), ("ref_ms", "reference ms"),
            ("ours_ms", "ours ms"), ("speedup", "speed-up"), ("pct_of_roofline", "% of roofline"), ("limiter", "limiter"),
            ("git_sha", "commit"))


def _cell(v) -> str:
    if v is None:
        return "-"
    if isinstance(v, float):
        return f"{v:.4g}"
    return str(v)


def ledger_table(rows: list[dict], fmt: str = "markdown") -> str:
    """The sweep ledger as a markdown table or CSV (the reference only writes a per-problem JSON:
    utils/compare_performance.py:151-163; a table over all problems and world sizes is what a results page needs)."""
    if fmt == "csv":
        import csv
        import io

        buf = io.StringIO()
        w = csv.writer(buf)
        w.writerow([k for k, _ in _COLUMNS])
        for d in rows:
            w.writerow(["" if d.get(k) is None else d.get(k) for k, _ in _COLUMNS])
        return buf.getvalue()
    if fmt != "markdown":
        raise ValueError("fmt must be 'markdown' or 'csv'")
    lines = ["| " + " | ".join(h for _, h in _COLUMNS) + " |", "|" + "---|" * len(_COLUMNS)]
    for d in rows:
        lines.append("| " + " | ".join(_cell(d.get(k, "default" if k == "config" else None)) for k, _ in _COLUMNS) + " |")
    ok = sum(1 for d in rows if d.get("all_ok"))
    sp = [d["speedup"] for d in rows if d.get("speedup")]
    tail = f"\n{ok} of {len(rows)} cells match"
    if sp:
        import math

        tail += f"; geometric-mean speed-up over {len(sp)} timed cells: {math.exp(sum(math.log(x) for x in sp) / len(sp)):.3g}x"
    return "\n".join(lines) + tail + "\n"
