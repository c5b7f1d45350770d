"""generate -> evaluate -> feedback loop around the harness."""
from __future__ import annotations

import json
import os
import re
import shlex
import subprocess
import time
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


def extract_code(text: str) -> str:
    """The first fenced ``python`` block of a model reply (any fenced block if none is tagged; the whole text if there is
    no fence at all) - the convention of the reference's generator (reference: kernelgen/generate_kernel.py:129-139)."""
    m = re.search(r"```python\s*\n(.*?)```", text, re.S) or re.search(r"```[a-zA-Z0-9_+-]*\s*\n(.*?)```", text, re.S)
    return (m.group(1) if m else text).strip() + "\n"


class CommandProposer:
    """Asks an operator-supplied command for the next candidate: the prompt goes to its standard input, its standard
    output is the reply (code, or prose with a fenced code block). Any local model runner or script fits; no client of a
    hosted model is bundled (reference: kernelgen/generate_kernel.py:369-488 talks to four hosted providers)."""

    def __init__(self, command: str | list[str], timeout_s: float = 600.0, log_dir: str | None = None):
        self.argv = shlex.split(command) if isinstance(command, str) else list(command)
        self.timeout_s, self.log_dir, self.calls = timeout_s, log_dir, 0

    def __call__(self, prompt: str, feedback: str | None) -> str:
        res = subprocess.run(self.argv, input=prompt, capture_output=True, text=True, timeout=self.timeout_s)
        if self.log_dir:
            os.makedirs(self.log_dir, exist_ok=True)
            with open(os.path.join(self.log_dir, f"exchange_{self.calls}.json"), "w") as fh:
                json.dump({"argv": self.argv, "returncode": res.returncode, "prompt": prompt, "reply": res.stdout,
                           "stderr": res.stderr[-4000:]}, fh)
        self.calls += 1
        if res.returncode != 0 or not res.stdout.strip():
            raise StopIteration(f"proposer command failed (rc={res.returncode}): {res.stderr[-500:]}")
        return extract_code(res.stdout)


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
    out = {"op": op, "solved": bool(history and history[-1]["all_ok"]), "attempts": history, "nproc": nproc,
           "finished_at": time.strftime("%Y-%m-%dT%H:%M:%S")}
    with open(os.path.join(workdir, f"{op}_run.json"), "w") as fh:      # run record next to the candidates
        json.dump(out, fh, indent=1)
    return out
