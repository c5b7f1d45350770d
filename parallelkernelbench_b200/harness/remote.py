"""Run harness jobs on another machine.

The reference reaches its GPUs through two hosted services: a client submits one job per (implementation, trial) with the
candidate source inline, a worker on the GPU side runs it and uploads the per-rank files, and the client downloads them and
compares locally (reference: run_together.py:95-433, run_together/worker.py:7-402, run_modal.py:126-309). This module
keeps that division of labour without any provider: the queue is a spool directory,

    <spool>/incoming/<job>.json      payload written by a client (atomically: temporary name, then rename)
    <spool>/running/<job>.json       claimed by a worker (rename = claim; two workers cannot take the same job)
    <spool>/done/<job>/result.json   written last; artifacts/ next to it holds rank_<r>.pt, rank_<r>_perf.json, traces/

and the transport that reaches it is either the local file system (a shared mount, or tests) or SFTP over SSH.

    # on the GPU box
    python -m parallelkernelbench_b200.harness.launch remote-worker --spool /scratch/pkb_spool
    # anywhere that can reach the spool
    python -m parallelkernelbench_b200.harness.launch eval --op tp_mlp --nproc 8 --measure-perf --remote-spool /scratch/pkb_spool
    python -m parallelkernelbench_b200.harness.launch eval --op 13 --nproc 8 --remote-spool /scratch/pkb_spool --remote-ssh user@gpubox

``RemoteRunner.run_job`` has the signature and the result of ``launch.run_job``, so ``launch.eval_op(..., runner=...)`` -
trials, accuracy gate, fp32 yardstick run, classification, EVAL_JSON - is the same code for local and remote jobs.
"""
from __future__ import annotations

import json
import os
import posixpath
import secrets
import shutil
import socket
import stat
import tempfile
import threading
import time
import traceback

ARTIFACT_SUFFIXES = (".pt", ".json", ".txt")
_JOB_KEYS = ("op", "impl", "nproc", "trial", "config", "overrides", "dtype", "backend", "measure_perf", "warmup", "iters", "graph",
             "profile", "timeout_s", "pg_timeout_s", "extra_worker_args")


# ---------------------------------------------------------------------------------------------------------------------
# transports
# ---------------------------------------------------------------------------------------------------------------------
class LocalTransport:
    """The spool is a directory this process can reach (same machine, or a shared mount)."""

    def __init__(self, root: str):
        self.root = os.path.abspath(root)
        for d in ("incoming", "running", "done"):
            os.makedirs(os.path.join(self.root, d), exist_ok=True)

    def _p(self, rel: str) -> str:
        return os.path.join(self.root, *rel.split("/"))

    def put_text_atomic(self, rel: str, text: str) -> None:
        dst = self._p(rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        tmp = dst + f".tmp{secrets.token_hex(4)}"
        with open(tmp, "w", encoding="utf-8") as fh:
            fh.write(text)
        os.replace(tmp, dst)

    def get_text(self, rel: str) -> str | None:
        try:
            with open(self._p(rel), encoding="utf-8") as fh:
                return fh.read()
        except OSError:
            return None

    def fetch_tree(self, rel: str, dest: str) -> list[str]:
        src = self._p(rel)
        names = []
        if os.path.isdir(src):
            for base, _dirs, files in os.walk(src):
                for f in files:
                    s = os.path.join(base, f)
                    r = os.path.relpath(s, src)
                    os.makedirs(os.path.dirname(os.path.join(dest, r)) or dest, exist_ok=True)
                    shutil.copyfile(s, os.path.join(dest, r))
                    names.append(r)
        return sorted(names)

    def remove_tree(self, rel: str) -> None:
        shutil.rmtree(self._p(rel), ignore_errors=True)


class SshTransport:
    """The spool lives on another host, reached by SFTP (paramiko; key-based login as configured for ``ssh``). Only the four
    operations of ``LocalTransport`` are needed. The test-suite runs this class against a stand-in SFTP client; a real
    connection needs an SSH server."""

    def __init__(self, target: str, root: str, port: int = 22):
        import paramiko

        user, _, host = target.rpartition("@")
        self.root = root
        self._client = paramiko.SSHClient()
        self._client.load_system_host_keys()
        self._client.set_missing_host_key_policy(paramiko.RejectPolicy())
        self._client.connect(host, port=port, username=user or None)
        self._sftp = self._client.open_sftp()
        for d in ("incoming", "running", "done"):
            self._mkdirs(posixpath.join(root, d))

    def _mkdirs(self, path: str) -> None:
        parts, cur = path.strip("/").split("/"), "/" if path.startswith("/") else ""
        for part in parts:
            cur = posixpath.join(cur, part)
            try:
                self._sftp.stat(cur)
            except OSError:
                self._sftp.mkdir(cur)

    def put_text_atomic(self, rel: str, text: str) -> None:
        dst = posixpath.join(self.root, rel)
        self._mkdirs(posixpath.dirname(dst))
        tmp = dst + f".tmp{secrets.token_hex(4)}"
        with self._sftp.open(tmp, "w") as fh:
            fh.write(text)
        self._sftp.posix_rename(tmp, dst)

    def get_text(self, rel: str) -> str | None:
        try:
            with self._sftp.open(posixpath.join(self.root, rel), "r") as fh:
                return fh.read().decode("utf-8", errors="replace")
        except OSError:
            return None

    def fetch_tree(self, rel: str, dest: str) -> list[str]:
        names: list[str] = []

        def walk(rdir: str, ldir: str, prefix: str) -> None:
            try:
                entries = self._sftp.listdir_attr(rdir)
            except OSError:
                return
            os.makedirs(ldir, exist_ok=True)
            for e in entries:
                r, l_ = posixpath.join(rdir, e.filename), os.path.join(ldir, e.filename)
                if stat.S_ISDIR(e.st_mode or 0):
                    walk(r, l_, prefix + e.filename + "/")
                else:
                    self._sftp.get(r, l_)
                    names.append(prefix + e.filename)

        walk(posixpath.join(self.root, rel), dest, "")
        return sorted(names)

    def remove_tree(self, rel: str) -> None:
        def rm(path: str) -> None:
            try:
                for e in self._sftp.listdir_attr(path):
                    p = posixpath.join(path, e.filename)
                    rm(p) if stat.S_ISDIR(e.st_mode or 0) else self._sftp.remove(p)
                self._sftp.rmdir(path)
            except OSError:
                pass

        rm(posixpath.join(self.root, rel))


# ---------------------------------------------------------------------------------------------------------------------
# worker side
# ---------------------------------------------------------------------------------------------------------------------
def _claim(spool: str) -> tuple[str, dict] | None:
    inc, run = os.path.join(spool, "incoming"), os.path.join(spool, "running")
    try:
        names = sorted(n for n in os.listdir(inc) if n.endswith(".json"))
    except OSError:
        return None
    for n in names:
        src, dst = os.path.join(inc, n), os.path.join(run, n)
        try:
            os.replace(src, dst)                       # the rename is the claim
        except OSError:
            continue                                   # another worker was faster
        try:
            with open(dst + ".owner", "w", encoding="utf-8") as fh:
                fh.write(f"{socket.gethostname()} {os.getpid()}")
        except OSError:
            pass
        try:
            with open(dst, encoding="utf-8") as fh:
                return n[:-5], json.load(fh)
        except (OSError, ValueError) as e:
            return n[:-5], {"_bad_payload": f"{type(e).__name__}: {e}"}
    return None


def _serve_one(spool: str, job_id: str, payload: dict) -> dict:
    """Run one claimed job and publish its result. Never raises."""
    from . import launch

    out_dir = os.path.join(spool, "done", job_id)
    art_dir = os.path.join(out_dir, "artifacts")
    os.makedirs(art_dir, exist_ok=True)
    result: dict
    tmp_solution = None
    try:
        if "_bad_payload" in payload:
            raise ValueError(payload["_bad_payload"])
        kw = {k: payload[k] for k in _JOB_KEYS if k in payload and k not in ("op", "impl", "nproc")}
        if payload.get("solution_source") is not None:
            fd, tmp_solution = tempfile.mkstemp(suffix=".py", prefix="pkb_remote_candidate_")
            with os.fdopen(fd, "w", encoding="utf-8") as fh:
                fh.write(payload["solution_source"])
            kw["solution"] = tmp_solution
        job = launch.run_job(payload["op"], payload["impl"], int(payload["nproc"]), **kw)
        names = []
        jd = job.get("job_dir") or ""
        if os.path.isdir(jd):
            for base, _dirs, files in os.walk(jd):
                for f in files:
                    if f.endswith(ARTIFACT_SUFFIXES) or "traces" in base:
                        rel = os.path.relpath(os.path.join(base, f), jd)
                        os.makedirs(os.path.dirname(os.path.join(art_dir, rel)) or art_dir, exist_ok=True)
                        shutil.copyfile(os.path.join(base, f), os.path.join(art_dir, rel))
                        names.append(rel)
            shutil.rmtree(jd, ignore_errors=True)
        result = {k: v for k, v in job.items() if k not in ("job_dir", "worker_logs_dir", "stdout", "stderr")}
        result.update({"stdout": (job.get("stdout") or "")[-20000:], "stderr": (job.get("stderr") or "")[-20000:],
                       "artifact_names_remote": sorted(names)})
    except Exception as e:                                              # a broken payload must not stop the worker
        result = {"returncode": 3, "artifact_count": 0, "artifact_names": [], "stdout": "", "timed_out": False, "interrupted": False,
                  "elastic_error_files": [], "seconds": 0.0,
                  "stderr": f"remote worker could not run the job: {type(e).__name__}: {e}\n{traceback.format_exc()[-2000:]}"}
    finally:
        if tmp_solution:
            try:
                os.remove(tmp_solution)
            except OSError:
                pass
    result["job_id"] = job_id
    tmp = os.path.join(out_dir, f"result.json.tmp{secrets.token_hex(4)}")
    with open(tmp, "w", encoding="utf-8") as fh:
        json.dump(result, fh)
    os.replace(tmp, os.path.join(out_dir, "result.json"))               # written last: its presence means "complete"
    for leftover in (job_id + ".json", job_id + ".json.owner"):
        try:
            os.remove(os.path.join(spool, "running", leftover))
        except OSError:
            pass
    return result


def _owner_gone(owner_file: str) -> bool:
    """True if the worker that claimed a job ran on this host and no longer exists (or left no record). A claim by a worker on
    another host is left alone: this process cannot tell whether that worker is alive."""
    try:
        with open(owner_file, encoding="utf-8") as fh:
            host, pid = fh.read().split()
    except (OSError, ValueError):
        return True
    if host != socket.gethostname():
        return False
    try:
        os.kill(int(pid), 0)
    except ProcessLookupError:
        return True
    except (PermissionError, ValueError):
        return False
    return int(pid) == os.getpid()          # a claim by this very process from an earlier serve() call that was stopped


def serve(spool: str, once: bool = False, poll_s: float = 0.5, stop: threading.Event | None = None, log=print) -> int:
    """Queue worker: claim jobs from ``<spool>/incoming`` in name order, run them here, publish results. Returns the number of
    jobs served (``once``: return after the first job or when the queue is empty). On start a worker also takes back jobs that
    a worker on this host had claimed and not finished before it died (left in ``running/`` by a crash or a kill; the claim
    records host and pid): they go back to ``incoming/`` and run again, so a client waiting for them is not stranded. Claims of
    live workers, and of workers on other hosts, are left alone, so several workers can serve one spool."""
    LocalTransport(spool)                                               # creates the three directories
    try:
        from . import hygiene

        health = hygiene.gpu_health()                                   # read-only device listing, as the reference's worker does
        log(f"[remote-worker] GPUs visible: {health['gpus']}" + ("" if health["ok"] else f" ({health['detail']})"))
    except Exception as e:
        log(f"[remote-worker] GPU listing failed: {type(e).__name__}: {e}")
    for n in sorted(os.listdir(os.path.join(spool, "running"))):
        path = os.path.join(spool, "running", n)
        if n.endswith(".json") and not os.path.exists(os.path.join(spool, "done", n[:-5], "result.json")) and _owner_gone(path + ".owner"):
            try:
                os.replace(path, os.path.join(spool, "incoming", n))
                log(f"[remote-worker] re-queued unfinished job {n[:-5]}")
            except OSError:
                pass
            try:
                os.remove(path + ".owner")
            except OSError:
                pass
    served = 0
    while not (stop is not None and stop.is_set()):
        claimed = _claim(spool)
        if claimed is None:
            if once:
                break
            time.sleep(poll_s)
            continue
        job_id, payload = claimed
        log(f"[remote-worker] {job_id}: {payload.get('op')} / {payload.get('impl')} / nproc {payload.get('nproc')} / trial {payload.get('trial')}")
        res = _serve_one(spool, job_id, payload)
        log(f"[remote-worker] {job_id}: rc={res.get('returncode')} artifacts={res.get('artifact_count')}")
        try:
            # leftovers of a job that died (shared-memory segments whose owner is gone) must not meet the next job
            # (reference: run_together/worker.py cleans up between jobs on the GPU side as well)
            from . import hygiene

            removed = hygiene.between_jobs().get("removed_segments") or []
            if removed:
                log(f"[remote-worker] removed {len(removed)} stale shared-memory segment(s)")
        except Exception as e:                                          # hygiene is best effort
            log(f"[remote-worker] hygiene failed: {type(e).__name__}: {e}")
        served += 1
        if once:
            break
    return served


# ---------------------------------------------------------------------------------------------------------------------
# client side
# ---------------------------------------------------------------------------------------------------------------------
class RemoteRunner:
    """Drop-in for ``launch.run_job``: submits the job to the spool, waits for its result and brings the artifacts into a local
    job directory."""

    def __init__(self, transport, poll_s: float = 1.0, wait_s: float = 3600.0, keep_remote: bool = False):
        self.transport, self.poll_s, self.wait_s, self.keep_remote = transport, poll_s, wait_s, keep_remote

    def submit(self, payload: dict) -> str:
        job_id = f"{time.strftime('%Y%m%dT%H%M%S')}_{os.getpid()}_{secrets.token_hex(4)}"
        self.transport.put_text_atomic(f"incoming/{job_id}.json", json.dumps(payload))
        return job_id

    def wait(self, job_id: str) -> dict | None:
        t0 = time.time()
        while time.time() - t0 < self.wait_s:
            text = self.transport.get_text(f"done/{job_id}/result.json")
            if text is not None:
                try:
                    return json.loads(text)
                except ValueError:
                    pass                                                 # not complete yet on a transport without atomic rename
            time.sleep(self.poll_s)
        return None

    def run_job(self, op: str, impl: str, nproc: int, trial: int = 0, config: str = "default", overrides=None, dtype="bfloat16",
                backend=None, measure_perf=False, warmup=500, iters=100, graph=False, profile=False, timeout_s=1800.0,
                extra_worker_args=None, pg_timeout_s=None, solution: str | None = None) -> dict:
        from . import launch

        job_dir = launch._job_dir(op, impl, trial)
        payload = {"op": op, "impl": impl, "nproc": nproc, "trial": trial, "config": config, "overrides": overrides or {},
                   "dtype": dtype, "backend": backend, "measure_perf": measure_perf, "warmup": warmup, "iters": iters, "graph": graph,
                   "profile": profile, "timeout_s": timeout_s, "pg_timeout_s": pg_timeout_s, "extra_worker_args": list(extra_worker_args or [])}
        base = {"op": op, "impl": impl, "trial": trial, "nproc": nproc, "job_dir": job_dir, "worker_logs_dir": job_dir, "stdout": "",
                "timed_out": False, "interrupted": False, "elastic_error_files": [], "artifact_count": 0, "artifact_names": [], "seconds": 0.0}
        if impl == "file":
            from ..utils.source_screen import screen_source

            try:
                with open(solution or "", encoding="utf-8", errors="replace") as fh:
                    payload["solution_source"] = fh.read()
            except OSError as e:
                return {**base, "returncode": 2, "stderr": f"cannot read solution: {e}"}
            hits = screen_source(payload["solution_source"])            # refused here already: nothing is sent
            if hits:
                return {**base, "returncode": 2, "stderr": "solution rejected by the source screen:\n  " + "\n  ".join(hits)}
        t0 = time.time()
        try:
            job_id = self.submit(payload)
            res = self.wait(job_id)
        except KeyboardInterrupt:
            return {**base, "returncode": 130, "interrupted": True, "stderr": "interrupted while waiting for the remote job", "seconds": time.time() - t0}
        except Exception as e:                                          # transport trouble is an environment failure, not a mismatch
            return {**base, "returncode": 4, "stderr": f"remote transport failed: {type(e).__name__}: {e}", "seconds": time.time() - t0}
        if res is None:
            return {**base, "returncode": 124, "timed_out": True, "stderr": f"no result for remote job {job_id} within {self.wait_s:.0f} s",
                    "seconds": time.time() - t0}
        names = self.transport.fetch_tree(f"done/{job_id}/artifacts", job_dir)
        if not self.keep_remote:
            self.transport.remove_tree(f"done/{job_id}")
        rank_files = [n for n in names if os.path.basename(n).startswith("rank_") and n.endswith(".pt")]
        return {**base, **{k: v for k, v in res.items() if k not in ("job_id", "artifact_names_remote")}, "job_dir": job_dir,
                "worker_logs_dir": job_dir, "artifact_count": len(rank_files), "artifact_names": sorted(rank_files),
                "seconds": time.time() - t0, "remote_job_id": job_id}


def make_runner(spool: str, ssh: str | None = None, **kw) -> RemoteRunner:
    return RemoteRunner(SshTransport(ssh, spool) if ssh else LocalTransport(spool), **kw)


__all__ = ["LocalTransport", "SshTransport", "RemoteRunner", "serve", "make_runner"]
