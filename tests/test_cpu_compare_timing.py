"""Harness units that need no GPU: compare semantics, timing bookkeeping, roofline, report classification."""
import json
import os

import torch

from parallelkernelbench_b200.harness import compare, report, roofline, timing
from parallelkernelbench_b200.utils import clocks


def test_normalize_and_compare_nested(tmp_path):
    y = (torch.ones(3), {"a": torch.zeros(2, 2), "n": 4})
    compare.save_output(y, str(tmp_path / "ref"), 0)
    compare.save_output(y, str(tmp_path / "cand"), 0)
    res = compare.compare_dirs(str(tmp_path / "ref"), str(tmp_path / "cand"))
    assert res["ok"] and res["kind"] == "match"


def test_compare_detects_mismatch_shape_missing_and_corrupt(tmp_path):
    ref, cand = str(tmp_path / "r"), str(tmp_path / "c")
    compare.save_output(torch.ones(8), ref, 0)
    compare.save_output(torch.ones(8) * 1.5, cand, 0)
    res = compare.compare_dirs(ref, cand)
    assert not res["ok"] and res["kind"] == "tensor_mismatch" and res["per_file"][0]["max_abs_diff"] == 0.5
    compare.save_output(torch.ones(4), cand, 0)
    assert compare.compare_dirs(ref, cand)["kind"] == "tensor_mismatch"
    assert compare.compare_dirs(ref, str(tmp_path / "nothing"))["kind"] == "missing_artifacts"
    compare.save_output(torch.ones(8), cand, 1)
    assert compare.compare_dirs(ref, cand)["kind"] == "path_mismatch"
    os.remove(os.path.join(cand, "rank_1.pt"))
    with open(os.path.join(cand, "rank_0.pt"), "wb") as fh:
        fh.write(b"not a torch file")
    assert compare.compare_dirs(ref, cand)["kind"] == "load_error"


def test_compare_tolerances_and_dtypes():
    a = torch.randn(100, dtype=torch.float64)
    assert compare.compare_objects(a, a + 1e-7, atol=1e-5, rtol=1e-5)["ok"]
    assert not compare.compare_objects(a, a + 1e-3, atol=1e-5, rtol=1e-5)["ok"]
    assert compare.compare_objects(a.to(torch.bfloat16), a.to(torch.bfloat16).float())["ok"]
    assert not compare.compare_objects({"x": 1}, {"y": 1})["ok"]
    assert not compare.compare_objects([a], [a, a])["ok"]


def test_num_groups_policy():
    l2 = 100
    assert timing.num_groups(300, l2) == 1
    assert timing.num_groups(1000, l2) == 1
    assert timing.num_groups(100, l2) == 4
    assert timing.num_groups(1, l2) == timing.MAX_GROUPS
    assert timing.num_groups(0, l2) == 1


def test_measure_on_cpu_reports_reference_keys():
    calls = []
    x = torch.ones(16)
    perf = timing.measure(lambda t: calls.append(t.data_ptr()), (x,), warmup=3, iters=5, device=torch.device("cpu"))
    for k in ("wall_time_ms", "wall_time_total_ms", "wall_time_std_ms", "min_time_ms", "max_time_ms", "iterations",
              "warmup_iterations", "num_input_groups", "l2_cache_size_bytes", "timed_tensor_bytes"):
        assert k in perf
    assert len(calls) == 8 and len(set(calls)) > 1      # inputs were rotated


def test_roofline_limiter_and_fraction():
    r = roofline.estimate(roofline.Cost(flops=1.4e15 * 1e-3, nvlink_bytes=0.0), measured_ms=2.0)
    assert r["limiter"] == "compute" and 30 < r["pct_of_roofline"] < 70
    r = roofline.estimate(roofline.Cost(flops=0.0, nvlink_bytes=770e9 * 1e-3), measured_ms=1.0)
    assert r["limiter"] == "nvlink" and abs(r["roofline_ms"] - 1.0) < 1e-6


def test_report_classification_and_perf_summary(tmp_path):
    ok = {"impl": "reference", "returncode": 0, "artifact_count": 2, "stdout": "", "stderr": ""}
    bad = {"impl": "ours", "returncode": 1, "artifact_count": 0, "stdout": "", "stderr": "RuntimeError: CUDA out of memory"}
    assert report.classify_trial(ok, bad, None)["result"] == "harness_environment"
    bad2 = dict(bad, stderr="ValueError: kernel bug")
    assert report.classify_trial(ok, bad2, None)["result"] == "no_artifacts"
    assert report.classify_trial(ok, dict(ok, impl="ours"), {"ok": True, "kind": "match"})["result"] == "match"
    assert report.classify_trial(ok, dict(ok, impl="ours"), {"ok": False, "kind": "tensor_mismatch"})["result"] == "tensor_mismatch"
    assert report.classify_trial(dict(ok, interrupted=True), ok, None)["result"] == "interrupted"
    # outputs were saved and compare equal, but the candidate job failed afterwards (guard band, determinism, timing loop)
    late = dict(ok, impl="ours", returncode=4)
    assert report.classify_trial(ok, late, {"ok": True, "kind": "match"})["result"] == "candidate_failed"
    assert report.classify_trial(ok, dict(ok, impl="ours", timed_out=True, returncode=-9), {"ok": True, "kind": "match"})["result"] == "candidate_failed"
    assert report.classify_trial(dict(ok, returncode=1), dict(ok, impl="ours"), {"ok": True, "kind": "match"})["result"] == "reference_failed"
    assert report.environment_hint("OSError: [Errno 98] Address already in use")
    for r, ms in enumerate((1.0, 3.0)):
        with open(tmp_path / f"rank_{r}_perf.json", "w") as fh:
            json.dump({"wall_time_ms": ms, "roofline_ms": 1.5, "limiter": "compute"}, fh)
    s = report.summarize_perf(str(tmp_path))
    assert s["wall_time_ms_max"] == 3.0 and s["n_ranks"] == 2 and abs(s["pct_of_roofline"] - 50.0) < 1e-9
    out = report.bounded_output("x" * 100000, "y" * 100000)
    assert len(out["stderr"]) < 50000 and "elided" in out["stderr"]


def test_clock_csv_summary(tmp_path):
    p = tmp_path / "clocks.csv"
    p.write_text("0, 1965, 1965, 180.0, 0x0, Not Active, Not Active, Not Active, Not Active\n"
                 "0, 1350, 1965, 990.0, 0x4, Not Active, Not Active, Not Active, Active\n"
                 "0, 1365, 1965, 985.0, 0x4, Not Active, Not Active, Not Active, Active\n")
    s = clocks.summarize_clock_rows(clocks.parse_clock_csv(str(p)))
    assert s["sm_max_mhz"] == 1965 and 1350 <= s["sm_mhz"] <= 1365 and s["reasons"] == ["sw_power_cap"]


def test_hygiene_removes_only_segments_of_dead_owners(tmp_path):
    import os
    import subprocess
    import sys

    from parallelkernelbench_b200.harness import hygiene

    child = subprocess.Popen([sys.executable, "-c", "pass"])
    child.wait()                                                     # a pid that no longer exists
    mine, dead, odd = tmp_path / f"pkb200_{os.getpid()}_29500", tmp_path / f"pkb200_{child.pid}_29501", tmp_path / "pkb200_legacy"
    for f in (mine, dead, odd):
        f.write_bytes(b"x")
    removed = hygiene.clean_shared_segments(directory=str(tmp_path))
    assert sorted(os.path.basename(p) for p in removed) == sorted([dead.name, odd.name])
    assert mine.exists() and not dead.exists()
    assert set(hygiene.gpu_health()) >= {"ok", "gpus", "detail"}


def test_nan_in_either_output_is_a_mismatch():
    import torch

    from parallelkernelbench_b200.harness import compare

    a = torch.tensor([1.0, float("nan"), 3.0])
    assert not compare.compare_objects(a, a.clone())["ok"]              # NaN on both sides is still a failure
    assert not compare.compare_objects(torch.tensor([1.0, 2.0, 3.0]), a)["ok"]
    assert compare.compare_objects(torch.tensor([1.0, 2.0]), torch.tensor([1.0, 2.0]))["ok"]



def test_loose_gate_must_be_earned_against_the_fp32_result(tmp_path, monkeypatch):
    """A candidate outside 1e-2/1e-2 of the bf16 reference passes only if the op's gate holds AND it is at most twice as far
    from the fp32 result as the reference is; a candidate that merely fits the loose gate fails."""
    import torch

    from parallelkernelbench_b200.harness import compare, launch

    torch.manual_seed(0)
    exact = torch.randn(4096) * 20
    ref = exact.to(torch.bfloat16)                                    # one rounding
    good = (exact + 0.3 * (exact.abs() / 256) * torch.sign(torch.randn(4096))).to(torch.bfloat16)   # a comparable error
    sloppy = (exact + 0.4).to(torch.bfloat16)                         # inside atol 0.5, but four times the reference's error

    def job(name, t):
        d = tmp_path / name
        compare.save_output(t, str(d), 0)
        return {"impl": name, "returncode": 0, "artifact_count": 1, "job_dir": str(d)}

    ref_job, good_job, sloppy_job = job("reference", ref), job("good", good), job("sloppy", sloppy)
    calls = []

    def fake_run_job(op, impl, nproc, trial=0, **kw):
        calls.append(impl)
        return dict(job(f"oracle{len(calls)}", exact), stderr="")

    monkeypatch.setattr(launch, "run_job", fake_run_job)
    cmp, gate = launch._gate("x", 1, 0, ref_job, job("same", ref.clone()), 0.5, 2e-2, True, {})
    assert cmp["ok"] and gate["gate"] == "strict" and calls == []     # the fp32 run is only made when it is needed
    tiny = ref.float().clone()
    tiny[ref.float().abs() < 0.5] += 0.02                             # near zero, 0.02 breaks atol 1e-2 but is within bf16 noise elsewhere
    cmp, gate = launch._gate("x", 1, 0, ref_job, good_job, 0.5, 2e-2, True, {})
    if gate["gate"] == "oracle":
        assert cmp["ok"] and gate["oracle_ok"]
    cmp, gate = launch._gate("x", 1, 0, ref_job, sloppy_job, 0.5, 2e-2, True, {})
    assert gate["gate"] == "oracle" and not gate["oracle_ok"] and not cmp["ok"]
    cmp, gate = launch._gate("x", 1, 0, ref_job, sloppy_job, 0.5, 2e-2, False, {})
    assert cmp["ok"] and gate["gate"] == "op_override_unverified"     # without the fp32 run the record says so
