"""Launcher CLI: run one implementation, evaluate ours against the reference, sweep ops x world
sizes, list the registry, and inspect stored results.

    python -m parallelkernelbench_b200.harness.launch doctor                        # what is installed, built and visible
    python -m parallelkernelbench_b200.harness.launch list
    python -m parallelkernelbench_b200.harness.launch run   --op allreduce --impl ours --nproc 2
    python -m parallelkernelbench_b200.harness.launch eval  --op tp_mlp --nproc 8 --measure-perf
    python -m parallelkernelbench_b200.harness.launch eval  --op plumbing --nproc 2 --backend gloo --atol 1e-5 --rtol 1e-5
    python -m parallelkernelbench_b200.harness.launch remote-worker --spool /shared/pkb_spool                    # on the GPU box
    python -m parallelkernelbench_b200.harness.launch eval  --op allreduce --nproc 8 --remote-spool /shared/pkb_spool   # anywhere
    python -m parallelkernelbench_b200.harness.launch sweep --ops allreduce,allgather --worlds 1,2,4,8 --resume
    python -m parallelkernelbench_b200.harness.launch report --format markdown      # the sweep ledger as a table
    python -m parallelkernelbench_b200.harness.launch headline --nproc 8            # the headline configurations, timed
    python -m parallelkernelbench_b200.harness.launch inspect --op allreduce
    python -m parallelkernelbench_b200.harness.launch perf-diff --op allreduce

``eval`` runs, for every trial, the reference job, a cool-down, the candidate job, then compares the
per-rank dumps and (with ``--measure-perf``) reports ``ref_max_ms / ours_max_ms`` and the fraction
of roofline; it stops at the first failing trial and ends with one machine-readable line
``EVAL_JSON:{...}``. Exit codes: 0 all trials match, 1 mismatch or failure, 130 interrupted.
One torchrun job per (implementation, trial), one process per GPU, rendezvous on 127.0.0.1 with a
random port so back-to-back jobs never collide (same orchestration role as reference:
run_local.py:72-482).
"""
from __future__ import annotations

import argparse
import json
import os
import random
import shutil
import signal
import subprocess
import sys
import time

from ..utils import env

from . import compare, hygiene, report

def _free_port() -> int:
    """A TCP port nobody listens on right now (asked from the kernel, so two back-to-back jobs never share one and a
    port held by an unrelated process is never picked); falls back to a random high port."""
    import socket

    try:
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sk:
            sk.bind(("127.0.0.1", 0))
            return int(sk.getsockname()[1])
    except OSError:
        return random.randint(29500, 39500)


LOGS_ROOT = os.environ.get("PKB_LOGS_DIR", os.path.join(str(env.REPO_ROOT), "logs"))


def _job_dir(op: str, impl: str, trial: int) -> str:
    d = os.path.join(LOGS_ROOT, "pkb200_worker", f"{op}_{impl}_t{trial}_{random.randrange(1 << 30):08x}")
    os.makedirs(d, exist_ok=True)
    return d


def final_dir(op: str, impl: str, trial: int, world: int) -> str:
    return os.path.join(LOGS_ROOT, f"op_{op}", f"w{world}", impl, f"trial_{trial}")


def run_job(op: str, impl: str, nproc: int, trial: int = 0, config: str = "default", overrides=None, dtype="bfloat16",
            backend=None, measure_perf=False, warmup=500, iters=100, graph=False, profile=False, timeout_s=1800.0,
            extra_worker_args=None, pg_timeout_s=None, solution: str | None = None) -> dict:
    """Start one torchrun job and wait for it. Never raises; the dict says what happened.
    ``impl="file"`` runs the candidate in ``solution`` (a copy staged into the job directory, so that the evaluated
    source is kept with its outputs)."""
    job_dir = _job_dir(op, impl, trial)
    if impl == "file":
        staged = os.path.join(job_dir, "candidate_solution.py")
        try:
            shutil.copyfile(solution or "", staged)
        except OSError as e:
            return {"returncode": 2, "artifact_count": 0, "job_dir": job_dir, "stdout": "", "stderr": f"cannot stage solution: {e}",
                    "timed_out": False, "interrupted": False, "elastic_error_files": [], "worker_logs_dir": job_dir, "seconds": 0.0}
        from ..utils.source_screen import screen_source

        try:
            with open(staged, encoding="utf-8", errors="replace") as fh:
                hits = screen_source(fh.read())
        except OSError as e:
            hits = [f"cannot read staged solution: {e}"]
        if hits:     # refused before any process is started: the file names a construct that must not run on the shared GPUs
            try:
                os.remove(staged)          # the refused text is not kept among the job artifacts either
            except OSError:
                pass
            return {"op": op, "impl": impl, "trial": trial, "nproc": nproc, "returncode": 2, "artifact_count": 0, "job_dir": job_dir,
                    "stdout": "", "stderr": "solution rejected by the source screen:\n  " + "\n  ".join(hits), "timed_out": False,
                    "interrupted": False, "elastic_error_files": [], "worker_logs_dir": job_dir, "seconds": 0.0}
        extra_worker_args = list(extra_worker_args or []) + ["--solution", staged]
    port = _free_port()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           "-m", "parallelkernelbench_b200.harness.worker", "--op", op, "--impl", impl, "--logs-dir", job_dir,
           "--config", config, "--dtype", dtype, "--trial", str(trial)]
    for k, v in (overrides or {}).items():
        cmd += ["--set", f"{k}={v}"]
    if backend:
        cmd += ["--backend", backend]
    if measure_perf:
        cmd += ["--measure-perf", "--warmup", str(warmup), "--iters", str(iters)]
        if graph:
            cmd.append("--graph")
    if profile:
        cmd.append("--profile")
    cmd += list(extra_worker_args or [])
    child_env = dict(os.environ)
    child_env["TORCHELASTIC_ERROR_FILE"] = os.path.join(job_dir, "torch_elastic_error.json")
    child_env["PYTHONPATH"] = str(env.REPO_ROOT) + os.pathsep + child_env.get("PYTHONPATH", "")
    child_env.setdefault("OMP_NUM_THREADS", "1")
    if pg_timeout_s is not None:
        child_env["PKB_PG_TIMEOUT_SEC"] = str(pg_timeout_s)
    if env.verbose():
        print(" ".join(cmd), flush=True)
    t0 = time.time()
    interrupted = False
    timed_out = False
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=child_env,
                            cwd=str(env.REPO_ROOT), start_new_session=True)
    try:
        out, err = proc.communicate(timeout=timeout_s)
    except subprocess.TimeoutExpired:
        timed_out = True
        out, err = _stop_group(proc)
    except KeyboardInterrupt:
        interrupted = True
        out, err = _stop_group(proc)
        with open(os.path.join(job_dir, "interrupted.txt"), "w") as fh:
            fh.write("interrupted by the user\n")
    artifacts = sorted(f for f in os.listdir(job_dir) if f.startswith("rank_") and f.endswith(".pt"))
    elastic = sorted(f for f in os.listdir(job_dir) if f.startswith("torch_elastic_error"))
    return {"op": op, "impl": impl, "trial": trial, "nproc": nproc, "returncode": proc.returncode if not timed_out else -9,
            "timed_out": timed_out, "interrupted": interrupted, "seconds": time.time() - t0, "job_dir": job_dir,
            "artifact_names": artifacts, "artifact_count": len(artifacts), "elastic_error_files": elastic,
            "stdout": out or "", "stderr": err or ""}


def _stop_group(proc) -> tuple[str, str]:
    """SIGTERM, then SIGKILL, the exact process group this launcher started."""
    try:
        os.killpg(proc.pid, signal.SIGTERM)
    except ProcessLookupError:
        pass
    try:
        return proc.communicate(timeout=10)
    except subprocess.TimeoutExpired:
        try:
            os.killpg(proc.pid, signal.SIGKILL)
        except ProcessLookupError:
            pass
        return proc.communicate()


def _keep(job: dict, world: int) -> str:
    """Move a finished job's artifacts to their final place; failed jobs stay where they are."""
    dst = final_dir(job["op"], job["impl"], job["trial"], world)
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(os.path.dirname(dst), exist_ok=True)
    shutil.move(job["job_dir"], dst)
    job["job_dir"] = dst
    return dst


STRICT_ATOL, STRICT_RTOL = compare.STRICT_ATOL, compare.STRICT_RTOL


def _gate(spec_name: str, nproc: int, trial: int, ref_job: dict, cand_job: dict, atol: float, rtol: float, use_oracle: bool,
          job_kw: dict, runner=None) -> tuple[dict | None, dict]:
    """Decide one trial. Returns (comparison used for the verdict, record of how the gate was applied).

    1. candidate within 1e-2 / 1e-2 of the reference (the reference harness's own gate): pass, ``gate = "strict"``.
    2. otherwise the op's own, looser gate must hold AND the loosening must be earned: the reference code is run once
       more on the same inputs widened to fp32 (``--impl oracle``) and the candidate may be at most twice as far from
       that result as the bf16 reference itself is (max and mean absolute error per rank file). ``gate = "oracle"``.
    3. if the fp32 run is impossible for this op (the reference code needs the low-precision dtype), the op gate alone
       decides and the record says so: ``gate = "op_override_unverified"``.
    """
    info: dict = {"atol": atol, "rtol": rtol}
    if not (ref_job["artifact_count"] and cand_job["artifact_count"]):
        return None, info
    strict = compare.compare_dirs(ref_job["job_dir"], cand_job["job_dir"], STRICT_ATOL, STRICT_RTOL, expected_ranks=nproc)
    info["strict_ok"] = strict["ok"]
    if strict["ok"] or (atol <= STRICT_ATOL and rtol <= STRICT_RTOL):
        info["gate"] = "strict" if strict["ok"] else "op"
        return (strict if strict["ok"] else compare.compare_dirs(ref_job["job_dir"], cand_job["job_dir"], atol, rtol, expected_ranks=nproc)), info
    cmp = compare.compare_dirs(ref_job["job_dir"], cand_job["job_dir"], atol, rtol, expected_ranks=nproc)
    info["gate"] = "op_override_unverified"
    if not cmp["ok"] or not use_oracle:
        return cmp, info
    kw = {k: v for k, v in job_kw.items() if k in ("config", "overrides", "dtype", "backend", "timeout_s", "pg_timeout_s")}
    oracle_job = (runner or run_job)(spec_name, "oracle", nproc, trial=trial, **kw)
    if oracle_job["returncode"] != 0 or oracle_job["artifact_count"] < nproc:
        tail = [ln for ln in (oracle_job.get("stderr") or "").strip().splitlines() if ln.strip()]
        info["oracle"] = "unavailable" + (f": {tail[-1][:200]}" if tail else "")
        return cmp, info
    big = float("inf")
    e_ref = compare.compare_dirs(oracle_job["job_dir"], ref_job["job_dir"], big, 0.0, expected_ranks=nproc)
    e_our = compare.compare_dirs(oracle_job["job_dir"], cand_job["job_dir"], big, 0.0, expected_ranks=nproc)
    shutil.rmtree(oracle_job["job_dir"], ignore_errors=True)
    if not (e_ref["ok"] and e_our["ok"]):            # structure differs or a NaN: the fp32 run is no yardstick here
        info["oracle"] = "unusable: " + "; ".join((e_ref["errors"] + e_our["errors"])[:2])
        return cmp, info
    worst = {"ref_max": 0.0, "ours_max": 0.0, "ref_mean": 0.0, "ours_mean": 0.0}
    earned = True
    for fr, fo in zip(e_ref["per_file"], e_our["per_file"]):
        rm, om = fr.get("max_abs_diff") or 0.0, fo.get("max_abs_diff") or 0.0
        ra, oa = fr.get("mean_abs_diff") or 0.0, fo.get("mean_abs_diff") or 0.0
        worst = {"ref_max": max(worst["ref_max"], rm), "ours_max": max(worst["ours_max"], om),
                 "ref_mean": max(worst["ref_mean"], ra), "ours_mean": max(worst["ours_mean"], oa)}
        earned = earned and om <= 2.0 * rm + 1e-3 and oa <= 2.0 * ra + 1e-4
    info.update({"gate": "oracle", "oracle": worst, "oracle_ok": earned})
    if not earned:
        cmp = dict(cmp, ok=False, kind="tensor_mismatch",
                   errors=[f"within the op gate but further from the fp32 result than twice the reference's own error: {worst}"] + cmp["errors"])
    return cmp, info


def eval_op(op: str, nproc: int, trials: int = 5, atol: float | None = None, rtol: float | None = None, measure_perf=False,
            cooldown: float | None = None, solution: str | None = None, oracle: bool = True, runner=None, **job_kw) -> dict:
    """``runner``: a callable with the signature and result of ``run_job`` that executes the jobs somewhere else
    (``harness.remote.RemoteRunner.run_job``); comparison, gate and classification stay here."""
    from ..workloads import registry

    run = runner or run_job
    spec = registry.get(op)
    op_atol, op_rtol = spec.tolerance(job_kw.get("config", "default"))
    atol = op_atol if atol is None else atol
    rtol = op_rtol if rtol is None else rtol
    cooldown = env.cooldown_sec() if cooldown is None else cooldown
    results, all_ok, interrupted, env_failed = [], True, False, False
    for t in range(trials):
        hygiene.between_jobs()
        ref_job = run(spec.name, "reference", nproc, trial=t, measure_perf=measure_perf, **job_kw)
        time.sleep(cooldown)
        cand_job = run(spec.name, "file" if solution else "ours", nproc, trial=t, measure_perf=measure_perf,
                       solution=solution, **job_kw)
        cmp, gate = _gate(spec.name, nproc, t, ref_job, cand_job, atol, rtol, oracle, job_kw, runner=runner)
        verdict = report.classify_trial(ref_job, cand_job, cmp)
        ref_perf = report.summarize_perf(ref_job["job_dir"]) if measure_perf else None
        cand_perf = report.summarize_perf(cand_job["job_dir"]) if measure_perf else None
        print(report.trial_line(t, verdict, ref_perf, cand_perf, gate), flush=True)
        ok = verdict["result"] == "match"
        entry = {"trial": t, **verdict, "compare": cmp, "gate": gate, "reference_returncode": ref_job["returncode"],
                 "ours_returncode": cand_job["returncode"], "reference_artifact_names": ref_job["artifact_names"],
                 "ours_artifact_names": cand_job["artifact_names"], "reference_perf": ref_perf, "ours_perf": cand_perf}
        if ref_perf and cand_perf:
            entry["speedup"] = ref_perf["wall_time_ms_max"] / cand_perf["wall_time_ms_max"]
        if not ok:
            for name, job in (("reference_job", ref_job), ("ours_job", cand_job)):
                if job["returncode"] != 0 or job["artifact_count"] == 0:
                    entry[name] = {"returncode": job["returncode"], "artifact_count": job["artifact_count"],
                                   "elastic_error_files": job["elastic_error_files"], "worker_logs_dir": job["job_dir"],
                                   **report.bounded_output(job["stdout"], job["stderr"])}
                    print(f"--- {job['impl']} job failed (rc={job['returncode']}), logs kept in {job['job_dir']}", flush=True)
                    print(job["stderr"][-2000:], flush=True)
        else:
            _keep(ref_job, nproc)
            _keep(cand_job, nproc)
        results.append(entry)
        interrupted = interrupted or verdict["result"] == "interrupted"
        env_failed = env_failed or verdict["result"] == "harness_environment"
        if not ok:
            all_ok = False
            entry["early_stop"] = True
            break
    summary = {"version": 1, "backend": "remote" if runner is not None else "local", "mode": "eval", "op": spec.name, "problem_ids": list(spec.problem_ids),
               "all_ok": all_ok, "interrupted": interrupted, "harness_environment_failed": env_failed,
               "trials": results, "nproc_per_node": nproc, "atol": atol, "rtol": rtol, "git_sha": env.git_sha()}
    print("all trials match" if all_ok else "mismatch", flush=True)
    print("EVAL_JSON:" + json.dumps(summary), flush=True)
    return summary


def cmd_list(_args) -> int:
    from ..workloads import registry

    if getattr(_args, "tolerances", False):
        # every op whose gate is looser than the reference harness's 1e-2 / 1e-2, with the reason
        for s in registry.all_ops():
            if s.atol > compare.STRICT_ATOL or s.rtol > compare.STRICT_RTOL:
                print(f"{s.name:36s} atol={s.atol:<6g} rtol={s.rtol:<6g} {s.tol_note}")
        return 0
    if getattr(_args, "json", False):
        # machine-readable registry: what tooling around the harness (sweeps, dashboards, generators) starts from
        print(json.dumps([{"op": s.name, "group": s.group, "problem_ids": list(s.problem_ids), "configs": s.configs, "atol": s.atol, "rtol": s.rtol,
                           "has_ours": s.ours is not None, "needs_cuda": s.ours_needs_cuda, "explicit_only": s.explicit_only,
                           "has_cost_model": s.cost is not None} for s in registry.all_ops()], indent=1))
        return 0
    for s in registry.all_ops():
        impl = "ours+ref" if s.ours is not None else "ref only"
        print(f"{s.name:32s} group={s.group:12s} problems={','.join(map(str, s.problem_ids)) or '-':12s} {impl:8s} configs={','.join(s.configs)}")
    cov = registry.coverage()
    print(f"{len(registry.all_ops())} ops; reference problems covered: {len(cov)}/87")
    return 0


def _overrides(a) -> dict:
    """``--set key=value`` pairs plus the reference launcher's two size knobs: ``--m`` / ``--n`` set the keys ``m`` / ``n`` of
    the op's config where it has them (reference: run_local.py:517-518; ops whose sizes have other names say so)."""
    from ..workloads import registry

    out = registry.parse_overrides(a.set)
    cfg = registry.get(a.op).configs.get(a.config, {})
    for key in ("m", "n"):
        val = getattr(a, key, None)
        if val is None:
            continue
        if key in cfg:
            out.setdefault(key, val)
        else:
            print(f"note: --{key} ignored: config {a.config!r} of {registry.get(a.op).name} has no key {key!r} (keys: {', '.join(sorted(cfg))})")
    return out


def cmd_run(a) -> int:
    from ..workloads import registry

    job = run_job(registry.get(a.op).name, a.impl, a.nproc, trial=a.trial, config=a.config,
                  overrides=_overrides(a), dtype=a.dtype, backend=a.backend, measure_perf=a.measure_perf,
                  warmup=a.warmup, iters=a.iters, graph=a.graph, profile=a.profile, timeout_s=a.timeout,
                  extra_worker_args=["--determinism", str(a.determinism)] if a.determinism > 0 else None)
    ok = job["returncode"] == 0 and job["artifact_count"] == a.nproc
    if a.determinism > 0:
        for line in job["stdout"].splitlines():
            if "determinism:" in line:
                print(line)
    if ok:
        perf = report.summarize_perf(job["job_dir"])
        _keep(job, a.nproc)
        print(f"dry run ok: {job['artifact_count']} rank files in {job['job_dir']}")
        if perf:
            print(f"Perf: max wall time (across ranks) {perf['wall_time_ms_max']:.4f} ms (mean {perf['wall_time_ms_mean']:.4f} ms, ranks={perf['n_ranks']})")
        return 0
    hint = report.environment_hint(job["stdout"] + job["stderr"])
    print(f"job failed rc={job['returncode']} artifacts={job['artifact_count']} logs={job['job_dir']}" + (f" environment: {hint}" if hint else ""))
    print(job["stderr"][-4000:])
    return 130 if job["interrupted"] else 1


def _remote_runner(a):
    """``run_job`` of a remote queue when ``--remote-spool`` was given, else None (jobs run on this machine)."""
    if not getattr(a, "remote_spool", None):
        return None
    from . import remote

    return remote.make_runner(a.remote_spool, ssh=a.remote_ssh, wait_s=a.remote_wait).run_job


def _remote_args(sp) -> None:
    sp.add_argument("--remote-spool", default=None, help="run the jobs through the queue in this spool directory (see harness/remote.py)")
    sp.add_argument("--remote-ssh", default=None, metavar="USER@HOST", help="the spool directory lives on this host (SFTP)")
    sp.add_argument("--remote-wait", type=float, default=3600.0, help="seconds to wait for one remote job")


def cmd_eval(a) -> int:
    from ..workloads import registry

    if a.solutions_dir and not a.solution:
        a.solution = os.path.join(a.solutions_dir, f"{registry.get(a.op).name}.py")     # the naming rule of ``sweep --solutions-dir``
        if not os.path.isfile(a.solution):
            print(f"no candidate file {a.solution}")
            return 2
    runner = _remote_runner(a)
    s = eval_op(a.op, a.nproc, trials=a.trials, atol=a.atol, rtol=a.rtol, measure_perf=a.measure_perf, config=a.config,
                overrides=_overrides(a), dtype=a.dtype, backend=a.backend, warmup=a.warmup, iters=a.iters,
                graph=a.graph, profile=a.profile, timeout_s=a.timeout, solution=a.solution, runner=runner)
    if s["interrupted"]:
        return 130
    return 0 if s["all_ok"] else 1


def doctor() -> dict:
    """What a first run needs, checked without launching anything on a GPU: interpreter and torch versions, the compiler, the
    in-tree native libraries and a few entry points each must export, the devices ``nvidia-smi -L`` lists (read-only),
    room in /dev/shm for the CPU twin of the symmetric heap, and which roofline denominators are in use. The reference
    prints hints of this kind only after a job has failed (reference: utils/run_utils.py:126-139)."""
    import platform
    import shutil as _sh

    import torch

    from .. import _native as nv
    from ..utils import env as _env

    out: dict = {"python": platform.python_version(), "torch": torch.__version__, "torch_cuda": torch.version.cuda,
                 "nccl_backend": bool(torch.distributed.is_available() and torch.distributed.is_nccl_available()),
                 "gloo_backend": bool(torch.distributed.is_available() and torch.distributed.is_gloo_available()),
                 "nvcc": os.environ.get("NVCC") or _sh.which("nvcc"), "git_sha": _env.git_sha()}
    libs = {}
    for what, avail, loader, symbols in (
            ("cuda", nv.cuda_lib_available, nv.cuda_lib, ("pkb_gemm_bf16_pair", "pkb_flash_attn_fwd", "pkb_coll_allreduce_nvls", "pkb_tp_ag_gemm", "pkb_heap_create")),
            ("host", nv.host_lib_available, nv.host_lib, ("pkbh_ctrl_bytes",))):
        rec = {"built": bool(avail()), "loads": False, "missing_symbols": []}
        if rec["built"]:
            try:
                lib = loader()
                rec["loads"] = True
                rec["missing_symbols"] = [s for s in symbols if not hasattr(lib, s)]
            except Exception as e:
                rec["error"] = f"{type(e).__name__}: {e}"[:300]
        libs[what] = rec
    out["native_libraries"] = libs
    out["gpus"] = hygiene.gpu_health()
    try:
        st = os.statvfs("/dev/shm")
        out["dev_shm_free_mib"] = st.f_bavail * st.f_frsize >> 20
    except OSError:
        out["dev_shm_free_mib"] = None
    pk = _env.measured_peaks()
    out["roofline_peaks"] = {k: pk.get(k) for k in ("source", "hbm_gbs", "bf16_tflops", "bf16_tflops_sustained")}
    problems = []
    if not libs["cuda"]["built"] or not libs["host"]["built"]:
        problems.append("native libraries are not built: run `python -m parallelkernelbench_b200.build` (needs nvcc)")
    for what, rec in libs.items():
        if rec["built"] and (not rec["loads"] or rec["missing_symbols"]):
            problems.append(f"the {what} library is stale or broken: rebuild with `python -m parallelkernelbench_b200.build --force`")
    if not out["nvcc"]:
        problems.append("nvcc not found (set $NVCC or put CUDA >= 12.8 on PATH): needed to build, not to run")
    if not out["gpus"]["ok"]:
        problems.append("no GPU visible: only the CPU / gloo configurations (`--backend gloo`) can run here")
    if out["dev_shm_free_mib"] is not None and out["dev_shm_free_mib"] < 256:
        problems.append("/dev/shm has less than 256 MiB free: the CPU twin of the symmetric heap may not fit")
    out["problems"] = problems
    return out


def cmd_doctor(a) -> int:
    d = doctor()
    if a.json:
        print(json.dumps(d, indent=1))
    else:
        for k, v in d.items():
            if k != "problems":
                print(f"{k}: {v}")
        print("problems: none" if not d["problems"] else "problems:\n  - " + "\n  - ".join(d["problems"]))
    return 0 if not [p for p in d["problems"] if "not built" in p or "stale or broken" in p] else 1


def cmd_remote_worker(a) -> int:
    from . import remote

    remote.serve(a.spool, once=a.once, poll_s=a.poll)
    return 0


def cmd_sweep(a) -> int:
    """ops x world sizes; one JSON line per cell appended to the ledger, finished cells skipped with --resume."""
    from ..workloads import registry

    ops = [s.name for s in registry.all_ops() if s.ours is not None and not s.explicit_only] if a.ops == "all" else a.ops.split(",")
    worlds = [int(w) for w in a.worlds.split(",")]
    ledger = a.ledger or os.path.join(LOGS_ROOT, "results.jsonl")
    os.makedirs(os.path.dirname(ledger), exist_ok=True)
    done = set()
    if a.resume and os.path.exists(ledger):
        with open(ledger) as fh:
            for line in fh:
                try:
                    d = json.loads(line)
                    if d.get("git_sha") == env.git_sha() or a.any_sha:
                        done.add((d["op"], d["world"], d.get("config", "default")))
                except ValueError:
                    pass
    rc = 0
    runner = _remote_runner(a)
    for op in ops:
        solution = None
        if a.solutions_dir:
            # a directory of candidate files named after the ops (<op>.py): ops without a file are left out
            solution = os.path.join(a.solutions_dir, f"{registry.get(op).name}.py")
            if not os.path.isfile(solution):
                print(f"skip {op} (no {solution})")
                continue
        for w in worlds:
            if (op, w, a.config) in done:
                print(f"skip {op} w={w} (already in {ledger})")
                continue
            s = eval_op(op, w, trials=a.trials, measure_perf=a.measure_perf, config=a.config, backend=a.backend,
                        dtype=a.dtype, warmup=a.warmup, iters=a.iters, timeout_s=a.timeout, solution=solution, runner=runner)
            last = s["trials"][-1] if s["trials"] else {}
            cell = {"op": op, "world": w, "config": a.config, "all_ok": s["all_ok"], "git_sha": s["git_sha"],
                    "result": last.get("result"), "speedup": last.get("speedup"),
                    "ref_ms": (last.get("reference_perf") or {}).get("wall_time_ms_max"),
                    "ours_ms": (last.get("ours_perf") or {}).get("wall_time_ms_max"),
                    "pct_of_roofline": (last.get("ours_perf") or {}).get("pct_of_roofline"),
                    "limiter": (last.get("ours_perf") or {}).get("limiter"), "time": time.time(),
                    "gate": (last.get("gate") or {}).get("gate"), "solution": solution}
            with open(ledger, "a") as fh:
                fh.write(json.dumps(cell) + "\n")
            rc = rc or (0 if s["all_ok"] else 1)
    return rc


# The configurations the published comparison is made on: (label, op, named config).
HEADLINE = (("1 plumbing AR->AG->RS", "plumbing", "default"),
            ("2 TP MLP block", "tp_mlp", "default"),
            ("3 EP MoE 256 experts top-8", "moe_layer", "deepseek"),
            ("4 CP ring attention fwd+bwd 131072 zigzag", "ring_attention_fwd_bwd", "cp131k"),
            ("5 FSDP Llama-8B training step", "fsdp_llama_step", "llama8b"))


def cmd_headline(a) -> int:
    """Evaluate and time the headline configurations at one world size and print them as a markdown table; every cell also
    goes to the ledger, so `report` can fold several world sizes into one table later."""
    ledger = a.ledger or os.path.join(LOGS_ROOT, "headline.jsonl")
    os.makedirs(os.path.dirname(ledger) or ".", exist_ok=True)
    only = {x.strip() for x in a.only.split(",")} if a.only else None
    rows, rc = [], 0
    for label, op, config in HEADLINE:
        if only and label.split()[0] not in only:
            continue
        s = eval_op(op, a.nproc, trials=1, measure_perf=True, config=config, backend=a.backend, dtype=a.dtype, warmup=a.warmup,
                    iters=a.iters, timeout_s=a.timeout)
        last = s["trials"][-1] if s["trials"] else {}
        cell = {"op": op, "world": a.nproc, "config": config, "all_ok": s["all_ok"], "git_sha": s["git_sha"], "label": label,
                "result": last.get("result"), "speedup": last.get("speedup"),
                "ref_ms": (last.get("reference_perf") or {}).get("wall_time_ms_max"),
                "ours_ms": (last.get("ours_perf") or {}).get("wall_time_ms_max"),
                "pct_of_roofline": (last.get("ours_perf") or {}).get("pct_of_roofline"),
                "limiter": (last.get("ours_perf") or {}).get("limiter"), "time": time.time()}
        with open(ledger, "a") as fh:
            fh.write(json.dumps(cell) + "\n")
        rows.append(cell)
        rc = rc or (0 if s["all_ok"] else 1)
    sys.stdout.write(report.ledger_table(rows, "markdown"))
    return rc


def cmd_report(a) -> int:
    """Print the sweep ledger as a markdown table or CSV."""
    ledger = a.ledger or os.path.join(LOGS_ROOT, "results.jsonl")
    if not os.path.exists(ledger):
        print(f"no ledger at {ledger}", file=sys.stderr)
        return 2
    text = report.ledger_table(report.ledger_rows(ledger, latest_only=not a.all_lines), a.format)
    if a.out:
        with open(a.out, "w") as fh:
            fh.write(text)
    else:
        sys.stdout.write(text)
    return 0


def cmd_inspect(a) -> int:
    from . import inspect_outputs

    return inspect_outputs.main_compare(a)


def cmd_perf_diff(a) -> int:
    from . import inspect_outputs

    return inspect_outputs.main_perf(a)


def _common(sp, need_impl=False):
    sp.add_argument("--op", "--problem", dest="op", required=True, help="op name or the reference's problem number")
    if need_impl:
        sp.add_argument("--impl", default="ours", choices=["reference", "ours", "oracle"])
    sp.add_argument("--nproc", "--nproc-per-node", "--num-gpus", dest="nproc", type=int, default=1)
    sp.add_argument("--config", default="default")
    sp.add_argument("--set", action="append", default=[])
    sp.add_argument("--m", type=int, default=None, help="shorthand for --set m=M on ops whose config has that key")
    sp.add_argument("--n", type=int, default=None, help="shorthand for --set n=N on ops whose config has that key")
    sp.add_argument("--dtype", default="bfloat16")
    sp.add_argument("--backend", default=None, choices=[None, "nccl", "gloo"])
    sp.add_argument("--measure-perf", action="store_true")
    sp.add_argument("--warmup", type=int, default=500)
    sp.add_argument("--iters", type=int, default=100)
    sp.add_argument("--graph", action="store_true")
    sp.add_argument("--profile", action="store_true")
    sp.add_argument("--timeout", type=float, default=1800.0)
    sp.add_argument("--trial", type=int, default=0)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="parallelkernelbench_b200.harness.launch", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--logs-dir", default=None, help="base directory of job directories, kept artifacts and ledgers (default: PKB_LOGS_DIR or <repo>/logs)")
    sub = ap.add_subparsers(dest="verb", required=True)
    sp = sub.add_parser("list"); sp.set_defaults(fn=cmd_list)
    sp.add_argument("--tolerances", action="store_true", help="list the ops compared with a gate looser than 1e-2 / 1e-2, and why")
    sp.add_argument("--json", action="store_true", help="the registry as JSON (op, group, problem ids, configs, tolerances)")
    sp = sub.add_parser("run"); _common(sp, need_impl=True); sp.set_defaults(fn=cmd_run)
    sp.add_argument("--determinism", type=int, default=0, metavar="N",
                    help="repeat the run N times on identical inputs and require bit-identical outputs (exit 1 otherwise)")
    sp = sub.add_parser("eval"); _common(sp)
    sp.add_argument("--trials", type=int, default=5)
    sp.add_argument("--solution", default=None, help="evaluate this file's solution(rc, *inputs) instead of the built-in implementation")
    sp.add_argument("--solutions-dir", default=None, help="evaluate DIR/<op>.py (used when --solution is not given)")
    sp.add_argument("--atol", type=float, default=None)
    sp.add_argument("--rtol", type=float, default=None)
    _remote_args(sp)
    sp.set_defaults(fn=cmd_eval)
    sp = sub.add_parser("doctor", help="check interpreter, compiler, native libraries, visible GPUs and /dev/shm without launching anything")
    sp.add_argument("--json", action="store_true")
    sp.set_defaults(fn=cmd_doctor)
    sp = sub.add_parser("remote-worker", help="serve the job queue of a spool directory on this machine")
    sp.add_argument("--spool", required=True)
    sp.add_argument("--once", action="store_true", help="serve at most one job, or return at once when the queue is empty")
    sp.add_argument("--poll", type=float, default=0.5)
    sp.set_defaults(fn=cmd_remote_worker)
    sp = sub.add_parser("sweep")
    sp.add_argument("--ops", default="all")
    sp.add_argument("--worlds", default="1,2,4,8")
    sp.add_argument("--config", default="default")
    sp.add_argument("--dtype", default="bfloat16")
    sp.add_argument("--trials", type=int, default=1)
    sp.add_argument("--backend", default=None, choices=[None, "nccl", "gloo"])
    sp.add_argument("--measure-perf", action="store_true")
    sp.add_argument("--warmup", type=int, default=500)
    sp.add_argument("--iters", type=int, default=100)
    sp.add_argument("--timeout", type=float, default=1800.0)
    sp.add_argument("--ledger", default=None)
    sp.add_argument("--resume", action="store_true")
    sp.add_argument("--any-sha", action="store_true", help="with --resume: accept cells recorded at another commit")
    sp.add_argument("--solutions-dir", default=None, help="evaluate DIR/<op>.py instead of the built-in implementation; ops without a file are skipped")
    _remote_args(sp)
    sp.set_defaults(fn=cmd_sweep)
    sp = sub.add_parser("headline")
    sp.add_argument("--nproc", "--nproc-per-node", dest="nproc", type=int, default=1)
    sp.add_argument("--only", default=None, help="comma-separated configuration numbers, e.g. 2,3")
    sp.add_argument("--dtype", default="bfloat16")
    sp.add_argument("--backend", default=None, choices=[None, "nccl", "gloo"])
    sp.add_argument("--warmup", type=int, default=500)
    sp.add_argument("--iters", type=int, default=100)
    sp.add_argument("--timeout", type=float, default=3600.0)
    sp.add_argument("--ledger", default=None)
    sp.set_defaults(fn=cmd_headline)
    sp = sub.add_parser("report")
    sp.add_argument("--ledger", default=None)
    sp.add_argument("--format", default="markdown", choices=["markdown", "csv"])
    sp.add_argument("--all-lines", action="store_true", help="every ledger line instead of the latest per (op, world, config)")
    sp.add_argument("--out", default=None)
    sp.set_defaults(fn=cmd_report)
    for name, fn in (("inspect", cmd_inspect), ("perf-diff", cmd_perf_diff)):
        sp = sub.add_parser(name)
        sp.add_argument("--op", required=True)
        sp.add_argument("--world", type=int, default=None)
        sp.add_argument("--trial", type=int, default=0)
        sp.add_argument("--atol", type=float, default=1e-2)
        sp.add_argument("--rtol", type=float, default=1e-2)
        sp.add_argument("--max-print", type=int, default=8)
        sp.set_defaults(fn=fn)
    args = ap.parse_args(argv)
    if args.logs_dir:
        global LOGS_ROOT
        LOGS_ROOT = os.path.abspath(args.logs_dir)
    try:
        return args.fn(args)
    except KeyboardInterrupt:
        return 130


if __name__ == "__main__":
    sys.exit(main())
