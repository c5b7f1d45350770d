"""Remote job queue: a worker thread serves a spool directory, the client submits jobs through it and compares locally."""
import json
import os
import threading

from parallelkernelbench_b200.harness import launch, remote


def test_eval_through_the_spool_queue_matches_local_behaviour(tmp_path, monkeypatch):
    monkeypatch.setattr(launch, "LOGS_ROOT", str(tmp_path / "logs"))
    spool = str(tmp_path / "spool")
    stop = threading.Event()
    served = []
    th = threading.Thread(target=lambda: served.append(remote.serve(spool, poll_s=0.05, stop=stop, log=lambda *_: None)), daemon=True)
    th.start()
    try:
        runner = remote.make_runner(spool, poll_s=0.05, wait_s=600.0)
        s = launch.eval_op("allreduce", 2, trials=1, config="small", backend="gloo", dtype="float32", cooldown=0.0, runner=runner.run_job)
    finally:
        stop.set()
        th.join(timeout=30)
    assert s["all_ok"] and s["backend"] == "remote", json.dumps(s)[:2000]
    t = s["trials"][0]
    assert t["result"] == "match" and t["reference_artifact_names"] == ["rank_0.pt", "rank_1.pt"]
    assert served and served[0] >= 2                                    # reference job and our job went through the worker
    assert os.listdir(os.path.join(spool, "incoming")) == [] and os.listdir(os.path.join(spool, "running")) == []
    assert os.listdir(os.path.join(spool, "done")) == []                # results are removed once fetched


def test_worker_survives_a_broken_payload_and_reports_it(tmp_path, monkeypatch):
    monkeypatch.setattr(launch, "LOGS_ROOT", str(tmp_path / "logs"))
    spool = str(tmp_path / "spool")
    tr = remote.LocalTransport(spool)
    tr.put_text_atomic("incoming/a_bad.json", "{not json")
    tr.put_text_atomic("incoming/b_unknown_op.json", json.dumps({"op": "no_such_op", "impl": "ours", "nproc": 1, "backend": "gloo", "timeout_s": 120}))
    assert remote.serve(spool, once=True, log=lambda *_: None) == 1
    assert remote.serve(spool, once=True, log=lambda *_: None) == 1
    bad = json.loads(tr.get_text("done/a_bad/result.json"))
    assert bad["returncode"] == 3 and "could not run" in bad["stderr"]
    unk = json.loads(tr.get_text("done/b_unknown_op/result.json"))
    assert unk["returncode"] != 0 and unk["artifact_count"] == 0
    assert remote.serve(spool, once=True, log=lambda *_: None) == 0     # queue empty


def test_candidate_is_screened_before_it_is_sent(tmp_path, monkeypatch):
    monkeypatch.setattr(launch, "LOGS_ROOT", str(tmp_path / "logs"))
    spool = str(tmp_path / "spool")
    cand = tmp_path / "cand.py"
    cand.write_text("def solution(rc, x):\n    src = '__tr' + 'ap();'\n    return x\n" + "# " + "__tr" + "ap()\n")
    runner = remote.make_runner(spool, poll_s=0.05, wait_s=5.0)
    job = runner.run_job("allreduce", "file", 2, solution=str(cand), backend="gloo")
    assert job["returncode"] == 2 and "rejected" in job["stderr"]
    assert os.listdir(os.path.join(spool, "incoming")) == []            # nothing was submitted
