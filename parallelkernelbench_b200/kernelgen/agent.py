"""generate -> evaluate -> feedback loop around the harness."""
from __future__ import annotations

import os
from typing import Callable

from .prompt import build_prompt


class ReplayProposer:
    """Stands in for a model: returns the candidate files of a directory in sorted order, one per call."""

    def __init__(self, directory: str):
        self.files = sorted(os.path.join(directory, f) for f in os.listdir(directory) if f.endswith(".py"))
        self.calls = 0

    def __call__(self, prompt: str, feedback: str | None) -> str:
        if self.calls >= len(self.files):
            raise StopIteration("no more recorded candidates")
        with open(self.files[self.calls]) as fh:
            src = fh.read()
        self.calls += 1
        return src


def _feedback(summary: dict) -> str:
    t = summary["trials"][-1] if summary.get("trials") else {}
    lines = [f"verdict: {t.get('result', 'no result')}"]
    cmp = t.get("compare") or {}
    lines += [f"mismatch: {e}" for e in (cmp.get("errors") or [])[:4]]
    job = t.get("ours_job") or {}
    if job.get("stderr"):
        lines.append("stderr tail:\n" + job["stderr"][-1500:])
    if t.get("speedup"):
        lines.append(f"speed-up over the reference: {t['speedup']:.2f}x")
    return "\n".join(lines)


def optimise(op: str, propose: Callable[[str, str | None], str], workdir: str, nproc: int = 2, max_iters: int = 4, trials: int = 1,
             target_speedup: float = 0.0, **eval_kw) -> dict:
    """Ask ``propose`` for a solution file, evaluate it against the reference, feed the verdict back, until every trial
    matches (and ``target_speedup`` is reached when timing is on) or ``max_iters`` attempts are used. Returns the history."""
    from ..harness.launch import eval_op

    os.makedirs(workdir, exist_ok=True)
    history, feedback = [], None
    for it in range(max_iters):
        try:
            source = propose(build_prompt(op, nproc=nproc, feedback=feedback), feedback)
        except StopIteration:
            break
        path = os.path.join(workdir, f"{op}_candidate_{it}.py")
        with open(path, "w") as fh:
            fh.write(source)
        summary = eval_op(op, nproc, trials=trials, solution=path, **eval_kw)
        feedback = _feedback(summary)
        sp = (summary["trials"][-1].get("speedup") or 0.0) if summary.get("trials") else 0.0
        history.append({"iteration": it, "path": path, "all_ok": summary["all_ok"], "speedup": sp, "feedback": feedback})
        if summary["all_ok"] and sp >= target_speedup:
            break
    return {"op": op, "solved": bool(history and history[-1]["all_ok"]), "attempts": history}
