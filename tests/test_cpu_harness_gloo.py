"""End-to-end harness runs with no GPU: torchrun + gloo ranks, ours = shared-memory twin."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _launch(*args, timeout=300):
    env = dict(os.environ, PKB_LOGS_DIR=os.path.join(ROOT, "logs", "pytest"), PKB_COOLDOWN_SEC="0")
    r = subprocess.run([sys.executable, "-m", "parallelkernelbench_b200.harness.launch", *args], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=timeout)
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("EVAL_JSON:")]
    return r, (json.loads(line[-1][len("EVAL_JSON:"):]) if line else None)


def test_plumbing_config_world2_matches_gloo_to_1e5():
    r, js = _launch("eval", "--op", "plumbing", "--nproc", "2", "--backend", "gloo", "--dtype", "float32", "--trials", "2",
                    "--atol", "1e-5", "--rtol", "1e-5")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert js["all_ok"] and len(js["trials"]) == 2 and js["trials"][0]["result"] == "match"
    assert js["trials"][0]["ours_artifact_names"] == ["rank_0.pt", "rank_1.pt"]


@pytest.mark.parametrize("op", ["allreduce", "allgather", "reducescatter", "alltoall", "broadcast", "reduce", "scatter", "gather"])
def test_collectives_world2_gloo(op):
    r, js = _launch("eval", "--op", op, "--nproc", "2", "--backend", "gloo", "--dtype", "float32", "--trials", "1",
                    "--config", "small")
    assert r.returncode == 0 and js["all_ok"], r.stdout[-1500:] + r.stderr[-1500:]


def test_perf_artifacts_and_speedup_line():
    r, js = _launch("eval", "--op", "allreduce", "--nproc", "2", "--backend", "gloo", "--dtype", "float32", "--trials", "1",
                    "--config", "small", "--measure-perf", "--warmup", "3", "--iters", "5")
    assert r.returncode == 0
    t = js["trials"][0]
    assert t["reference_perf"]["n_ranks"] == 2 and t["ours_perf"]["wall_time_ms_max"] > 0 and t["speedup"] > 0
    assert "speedup" in r.stdout


def test_rank_that_raises_is_reported_not_hung():
    from parallelkernelbench_b200.harness import launch

    job = launch.run_job("allreduce", "ours", 2, backend="gloo", dtype="float32", config="small",
                         extra_worker_args=["--fail-rank", "1"], timeout_s=120, pg_timeout_s=20)
    assert job["returncode"] != 0 and job["artifact_count"] == 0 and not job["timed_out"]
    assert "injected failure on rank 1" in job["stderr"]


def test_rank_that_exits_nonzero_is_reported():
    from parallelkernelbench_b200.harness import launch

    job = launch.run_job("allreduce", "reference", 2, backend="gloo", dtype="float32", config="small",
                         extra_worker_args=["--exit-rank", "0"], timeout_s=120, pg_timeout_s=20)
    assert job["returncode"] != 0 and job["artifact_count"] == 0


def test_unknown_op_is_a_clean_failure():
    r, js = _launch("run", "--op", "no_such_op", "--nproc", "1", "--backend", "gloo")
    assert r.returncode != 0


def test_project_derived_and_sequence_parallel_ops_world2_gloo():
    """Every op of the 'ulysses' and 'wild' groups and the 2-D mesh attention blocks: ours (host shared-memory backend,
    PyTorch math) against the process-group restatement, two CPU ranks, fp32."""
    import subprocess
    import sys

    from parallelkernelbench_b200.workloads import registry

    names = [s.name for s in registry.all_ops() if s.group in ("ulysses", "wild")] + ["ring_attention_tp", "ring_attention_pp",
                                                                                       "ring_attention_backward_dp"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29577", os.path.join(root, "tests", "mp", "all_ops_worker.py"), "--backend", "gloo", "--dtype", "float32",
           "--ops", ",".join(names)]
    r = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "TOTAL_FAILS 0" in r.stdout, r.stdout[-3000:] + r.stderr[-2000:]
    assert r.stdout.count("PASS rank0") >= len(names)


def test_external_solution_file_is_evaluated_against_the_reference(tmp_path):
    """A candidate written by a user of the harness: one file with solution(rc, *inputs), evaluated like the built-in one."""
    good = tmp_path / "my_allreduce.py"
    good.write_text("def solution(rc, x):\n    return rc.comm.all_reduce(x)\n")
    r, js = _launch("eval", "--op", "allreduce", "--nproc", "2", "--backend", "gloo", "--dtype", "float32", "--trials", "1",
                    "--config", "small", "--solution", str(good))
    assert r.returncode == 0 and js["all_ok"], r.stdout[-1500:] + r.stderr[-1500:]
    bad = tmp_path / "wrong.py"
    bad.write_text("def solution(rc, x):\n    return x * 3\n")
    r, js = _launch("eval", "--op", "allreduce", "--nproc", "2", "--backend", "gloo", "--dtype", "float32", "--trials", "1",
                    "--config", "small", "--solution", str(bad))
    assert r.returncode != 0 and not js["all_ok"] and js["trials"][0]["result"] != "match"


def test_list_sweep_resume_inspect_and_perf_diff(tmp_path):
    """The remaining launcher subcommands on CPU: list, a one-cell sweep with its ledger, resume skipping the finished cell,
    and the offline inspectors over the stored per-rank files."""
    r, _ = _launch("list")
    assert r.returncode == 0 and "allreduce" in r.stdout and "reference problems covered: 87/87" in r.stdout
    ledger = str(tmp_path / "results.jsonl")
    args = ["sweep", "--ops", "allreduce", "--worlds", "2", "--config", "small", "--backend", "gloo", "--dtype", "float32", "--trials", "1",
            "--measure-perf", "--warmup", "2", "--iters", "3", "--ledger", ledger]
    r, _ = _launch(*args)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    cells = [json.loads(ln) for ln in open(ledger)]
    assert len(cells) == 1 and cells[0]["op"] == "allreduce" and cells[0]["world"] == 2 and cells[0]["all_ok"] and cells[0]["speedup"] > 0
    r, _ = _launch(*args, "--resume")
    assert r.returncode == 0 and "skip allreduce w=2" in r.stdout and len(open(ledger).readlines()) == 1
    r, _ = _launch("report", "--ledger", ledger)
    assert r.returncode == 0 and "| allreduce | small | 2 | match |" in r.stdout and "1 of 1 cells match" in r.stdout
    r, _ = _launch("report", "--ledger", ledger, "--format", "csv")
    assert r.returncode == 0 and r.stdout.splitlines()[0].startswith("op,config,world,result") and "allreduce,small,2,match" in r.stdout
    r, _ = _launch("inspect", "--op", "allreduce")
    assert r.returncode == 0 and "verdict: match" in r.stdout
    r, _ = _launch("perf-diff", "--op", "allreduce")
    assert r.returncode == 0 and "speed" in r.stdout.lower()
    sol_dir = tmp_path / "solutions"
    sol_dir.mkdir()
    (sol_dir / "allreduce.py").write_text("def solution(rc, x):\n    return rc.comm.all_reduce(x)\n")
    ledger2 = str(tmp_path / "results_candidates.jsonl")
    r, _ = _launch("sweep", "--ops", "allreduce,allgather", "--worlds", "2", "--config", "small", "--backend", "gloo", "--dtype", "float32",
                   "--trials", "1", "--ledger", ledger2, "--solutions-dir", str(sol_dir))
    assert r.returncode == 0 and "skip allgather (no " in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]
    cells2 = [json.loads(ln) for ln in open(ledger2)]
    assert len(cells2) == 1 and cells2[0]["op"] == "allreduce" and cells2[0]["all_ok"] and cells2[0]["solution"].endswith("allreduce.py")


def test_headline_verb_runs_the_plumbing_configuration_on_cpu(tmp_path):
    ledger = str(tmp_path / "headline.jsonl")
    r, _ = _launch("headline", "--only", "1", "--nproc", "2", "--backend", "gloo", "--dtype", "float32", "--warmup", "2", "--iters", "3",
                   "--ledger", ledger)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    assert "| plumbing | default | 2 | match |" in r.stdout and "1 of 1 cells match" in r.stdout
    cell = json.loads(open(ledger).readline())
    assert cell["label"].startswith("1 ") and cell["ours_ms"] > 0


def test_run_with_determinism_check_on_cpu():
    r, _ = _launch("run", "--op", "allreduce", "--impl", "ours", "--nproc", "2", "--backend", "gloo", "--dtype", "float32", "--config", "small",
                   "--determinism", "3")
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    assert "determinism: 3/3 repeat runs bit-identical" in r.stdout


def test_bit_identical_helper_sees_single_bit_and_structure_differences():
    import torch

    from parallelkernelbench_b200.harness.worker import _bit_identical

    a = torch.tensor([1.0, float("nan"), -0.0])
    assert _bit_identical(a, a.clone()) and _bit_identical((a, {"k": a}), (a.clone(), {"k": a.clone()}))
    assert not _bit_identical(a, torch.tensor([1.0, float("nan"), 0.0]))          # -0.0 against +0.0: equal values, other bits
    assert not _bit_identical(a, a.double()) and not _bit_identical((a,), (a, a)) and not _bit_identical({"k": a}, {"j": a})
    assert _bit_identical(torch.empty(0), torch.empty(0)) and _bit_identical(3, 3) and not _bit_identical(3, 4)


def test_fsdp_llama_step_is_an_explicit_only_op_whose_reference_runs_on_cpu():
    """The engine-sized workload is in the registry (so `eval`, `headline` and the prompt tooling reach it) but stays out of
    "all" selections; its PyTorch implementation trains one step on a CPU rank and the loss is near ln(vocab)."""
    import math

    import torch

    from parallelkernelbench_b200.harness import launch
    from parallelkernelbench_b200.workloads import registry

    spec = registry.get("fsdp_llama_step")
    assert spec.explicit_only and spec.ours_needs_cuda and "llama8b" in spec.configs
    assert [h for h in launch.HEADLINE if h[1] == "fsdp_llama_step"] == [("5 FSDP Llama-8B training step", "fsdp_llama_step", "llama8b")]
    job = launch.run_job("fsdp_llama_step", "reference", 1, backend="gloo", dtype="bfloat16", config="small", timeout_s=300)
    assert job["returncode"] == 0 and job["artifact_count"] == 1, job["stderr"][-1500:]
    loss = torch.load(os.path.join(job["job_dir"], "rank_0.pt"))
    loss = loss["output_0"] if isinstance(loss, dict) else loss
    assert abs(float(loss.reshape(-1)[0]) - math.log(1024)) < 0.5
    c = spec.cost(spec.configs["llama8b"], 8)
    assert 1.5e14 < c.flops < 3e14 and c.nvlink_bytes > 1e10


def test_reference_style_flags_are_accepted(tmp_path, capsys, monkeypatch):
    """--problem / --num-gpus / --m / --n / --logs-dir: the spelling of the reference's launcher maps onto op, nproc, config
    overrides and the log root."""
    from parallelkernelbench_b200.harness import launch

    monkeypatch.setattr(launch, "LOGS_ROOT", launch.LOGS_ROOT)          # restored after the test: --logs-dir rebinds it
    logs = tmp_path / "my_logs"
    rc = launch.main(["--logs-dir", str(logs), "run", "--problem", "1", "--num-gpus", "1", "--backend", "gloo", "--dtype", "float32",
                      "--config", "small", "--m", "4", "--n", "32"])
    out = capsys.readouterr().out
    assert rc == 0 and "dry run ok" in out
    kept = logs / "op_allreduce" / "w1" / "ours" / "trial_0"
    assert (kept / "rank_0.pt").exists()
    import torch

    y = torch.load(kept / "rank_0.pt")
    shape = tuple((y["output"] if isinstance(y, dict) and "output" in y else y).shape) if not isinstance(y, (list, tuple)) else None
    assert shape is None or shape == (4, 32), shape                       # the size knobs reached the input factory
    rc = launch.main(["--logs-dir", str(logs), "run", "--problem", "80", "--num-gpus", "1", "--backend", "gloo", "--dtype", "float32",
                      "--config", "small", "--m", "4"])
    out = capsys.readouterr().out
    assert rc == 0 and "--m ignored" in out and "prototypes" in out


def test_doctor_reports_the_environment_without_launching_anything(capsys):
    from parallelkernelbench_b200.harness import launch

    d = launch.doctor()
    assert d["native_libraries"]["cuda"] == {"built": True, "loads": True, "missing_symbols": []}
    assert d["native_libraries"]["host"]["loads"] and d["gloo_backend"] and d["roofline_peaks"]["hbm_gbs"] > 1000
    assert isinstance(d["problems"], list) and not any("not built" in p or "stale" in p for p in d["problems"])
    assert launch.main(["doctor"]) == 0
    out = capsys.readouterr().out
    assert "native_libraries" in out and "problems" in out
    assert launch.main(["doctor", "--json"]) == 0
    import json

    assert json.loads(capsys.readouterr().out)["python"]


def test_list_as_json_covers_every_reference_problem(capsys):
    import json

    from parallelkernelbench_b200.harness import launch

    assert launch.main(["list", "--json"]) == 0
    ops = json.loads(capsys.readouterr().out)
    covered = {p for o in ops for p in o["problem_ids"]}
    assert covered >= set(range(1, 88)) and all(o["has_ours"] for o in ops if o["problem_ids"])
    assert {"default"} <= set(ops[0]["configs"])
