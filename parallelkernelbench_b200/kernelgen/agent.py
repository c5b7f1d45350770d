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


class HttpProposer:
    """Asks a chat-completions endpoint for the next candidate: ``POST <base_url>/chat/completions`` with the usual
    ``{"model", "messages", "max_tokens", "temperature"}`` body, the reply read from ``choices[0].message.content``. That is
    the wire format of the hosted providers the reference talks to through their SDKs (reference:
    kernelgen/generate_kernel.py:390-488) and of model servers one can run next to the GPUs, so no SDK is needed; the key,
    if the endpoint wants one, comes from the environment variable named by ``api_key_env``. Feedback from the previous
    attempt is already part of the prompt text."""

    SYSTEM = ("You write one Python file that defines solution(rc, *inputs) for the distributed GPU workload described by the "
              "user. Reply with a single fenced python block and nothing that needs to be executed outside it.")

    def __init__(self, base_url: str, model: str, api_key_env: str | None = "PKB_KERNELGEN_API_KEY", max_tokens: int = 16384,
                 temperature: float = 0.2, timeout_s: float = 900.0, log_dir: str | None = None):
        self.url = base_url.rstrip("/") + "/chat/completions"
        self.model, self.api_key_env, self.max_tokens, self.temperature = model, api_key_env, max_tokens, temperature
        self.timeout_s, self.log_dir, self.calls = timeout_s, log_dir, 0

    def __call__(self, prompt: str, feedback: str | None) -> str:
        import requests

        headers = {"Content-Type": "application/json"}
        key = os.environ.get(self.api_key_env or "", "")
        if key:
            headers["Authorization"] = f"Bearer {key}"
        body = {"model": self.model, "max_tokens": self.max_tokens, "temperature": self.temperature,
                "messages": [{"role": "system", "content": self.SYSTEM}, {"role": "user", "content": prompt}]}
        try:
            resp = requests.post(self.url, headers=headers, json=body, timeout=self.timeout_s)
            status, text = resp.status_code, resp.text
            reply = resp.json()["choices"][0]["message"]["content"] if status == 200 else ""
        except (requests.RequestException, ValueError, KeyError, IndexError, TypeError) as e:
            status, text, reply = -1, f"{type(e).__name__}: {e}", ""
        if self.log_dir:
            os.makedirs(self.log_dir, exist_ok=True)
            with open(os.path.join(self.log_dir, f"exchange_{self.calls}.json"), "w") as fh:     # the key is never written
                json.dump({"url": self.url, "model": self.model, "status": status, "prompt": prompt, "reply": reply or text[-4000:]}, fh)
        self.calls += 1
        if not (reply or "").strip():
            raise StopIteration(f"endpoint gave no usable reply (status {status}): {text[-300:]}")
        return extract_code(reply)


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


def _trajectory(workdir: str, op: str, record: dict) -> None:
    """One JSON line per event of a run (prompt sent, candidate received, screen verdict, evaluation) in ``<op>_trajectory.jsonl``:
    the step-by-step record of an optimisation run, appendable across resumed runs (the reference keeps the agent framework's
    message history for the same purpose, reference: kernelgen/agent.py:198-287)."""
    record = {"time": time.strftime("%Y-%m-%dT%H:%M:%S"), "op": op, **record}
    with open(os.path.join(workdir, f"{op}_trajectory.jsonl"), "a") as fh:
        fh.write(json.dumps(record) + "\n")


def optimise(op: str, propose: Callable[[str, str | None], str], workdir: str, nproc: int = 2, max_iters: int = 4, trials: int = 1,
             target_speedup: float = 0.0, resume: bool = False, templates: str | None = None, hardware: str = "b200_8", **eval_kw) -> dict:
    """Ask ``propose`` for a solution file, evaluate it against the reference, feed the verdict back, until every trial
    matches (and ``target_speedup`` is reached when timing is on) or ``max_iters`` attempts are used.

    Every candidate is screened before it is evaluated (``utils.source_screen``): a file that names a construct that must not
    run on the shared GPUs is not launched, the hits go back to the proposer as feedback and the attempt counts. The run leaves
    the candidates, ``<op>_trajectory.jsonl`` (one line per event) and ``<op>_run.json`` (history, the best matching
    candidate and its speed-up) in ``workdir``; with ``resume`` a previous ``<op>_run.json`` is continued from its last
    feedback instead of starting over. ``templates`` / ``hardware``: a TOML file laid over the packaged prompt templates and
    the hardware profile to quote from them. Returns the run record."""
    from ..harness.launch import eval_op
    from ..utils.source_screen import screen_source

    os.makedirs(workdir, exist_ok=True)
    run_path = os.path.join(workdir, f"{op}_run.json")
    history, feedback = [], None
    if resume and os.path.exists(run_path):
        with open(run_path) as fh:
            prev = json.load(fh)
        history = prev.get("attempts", [])
        feedback = history[-1]["feedback"] if history else None
        _trajectory(workdir, op, {"event": "resume", "attempts_so_far": len(history)})
    for it in range(len(history), len(history) + max_iters):
        prompt = build_prompt(op, hardware=hardware, nproc=nproc, feedback=feedback, templates=templates)
        _trajectory(workdir, op, {"event": "prompt", "iteration": it, "prompt_chars": len(prompt), "had_feedback": feedback is not None})
        try:
            source = propose(prompt, feedback)
        except StopIteration as e:
            _trajectory(workdir, op, {"event": "proposer_stopped", "iteration": it, "why": str(e)[:300]})
            break
        path = os.path.join(workdir, f"{op}_candidate_{it}.py")
        hits = screen_source(source)
        if hits:
            # never written as a runnable file, never launched: the proposer is told why and may try again
            with open(path + ".rejected.txt", "w") as fh:
                fh.write("\n".join(hits) + "\n")
            feedback = "verdict: rejected before evaluation - the file names constructs that must not run here:\n" + "\n".join(hits)
            history.append({"iteration": it, "path": None, "all_ok": False, "speedup": 0.0, "feedback": feedback, "screened_out": True})
            _trajectory(workdir, op, {"event": "screened_out", "iteration": it, "hits": hits[:8]})
            continue
        with open(path, "w") as fh:
            fh.write(source)
        _trajectory(workdir, op, {"event": "candidate", "iteration": it, "path": path, "lines": source.count("\n")})
        summary = eval_op(op, nproc, trials=trials, solution=path, **eval_kw)
        feedback = _feedback(summary)
        last = summary["trials"][-1] if summary.get("trials") else {}
        sp = last.get("speedup") or 0.0
        history.append({"iteration": it, "path": path, "all_ok": summary["all_ok"], "speedup": sp, "feedback": feedback,
                        "result": last.get("result"), "gate": (last.get("gate") or {}).get("gate")})
        _trajectory(workdir, op, {"event": "evaluated", "iteration": it, "all_ok": summary["all_ok"], "result": last.get("result"),
                                  "speedup": sp})
        if summary["all_ok"] and sp >= target_speedup:
            break
    ok = [h for h in history if h["all_ok"]]
    best = max(ok, key=lambda h: h["speedup"]) if ok else None
    out = {"op": op, "solved": bool(ok), "best": best, "attempts": history, "nproc": nproc,
           "finished_at": time.strftime("%Y-%m-%dT%H:%M:%S")}
    with open(run_path, "w") as fh:      # run record next to the candidates
        json.dump(out, fh, indent=1)
    return out
