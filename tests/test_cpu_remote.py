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


class _FakeSftp:
    """The subset of paramiko's SFTP client the transport uses, mapped onto a local directory that plays the remote host."""

    def __init__(self, host_root):
        self.host_root = host_root

    def _l(self, path):
        return os.path.join(self.host_root, path.lstrip("/"))

    def stat(self, path):
        return os.stat(self._l(path))

    def mkdir(self, path):
        os.mkdir(self._l(path))

    def open(self, path, mode="r"):
        return open(self._l(path), mode + "b")

    def posix_rename(self, src, dst):
        os.replace(self._l(src), self._l(dst))

    def listdir_attr(self, path):
        out = []
        for name in os.listdir(self._l(path)):
            st = os.stat(os.path.join(self._l(path), name))
            out.append(type("Attr", (), {"filename": name, "st_mode": st.st_mode})())
        return out

    def get(self, remote, local):
        import shutil

        shutil.copyfile(self._l(remote), local)

    def remove(self, path):
        os.remove(self._l(path))

    def rmdir(self, path):
        os.rmdir(self._l(path))


class _FakeFile:
    def __init__(self, fh):
        self.fh = fh

    def write(self, data):
        self.fh.write(data.encode("utf-8") if isinstance(data, str) else data)

    def read(self):
        return self.fh.read()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.fh.close()


def test_sftp_transport_against_a_fake_sftp_client(tmp_path, monkeypatch):
    """The SSH transport's own logic (remote mkdir -p, atomic put, recursive fetch and removal) over a stand-in SFTP client."""
    import paramiko

    host_root = tmp_path / "remote_host"
    host_root.mkdir()
    sftp = _FakeSftp(str(host_root))
    real_open = sftp.open
    sftp.open = lambda path, mode="r": _FakeFile(real_open(path, mode))
    seen = {}

    class FakeClient:
        def load_system_host_keys(self):
            seen["host_keys"] = True

        def set_missing_host_key_policy(self, policy):
            seen["policy"] = type(policy).__name__

        def connect(self, host, port=22, username=None):
            seen["connect"] = (host, port, username)

        def open_sftp(self):
            return sftp

    monkeypatch.setattr(paramiko, "SSHClient", FakeClient)
    monkeypatch.setattr(launch, "LOGS_ROOT", str(tmp_path / "logs"))
    tr = remote.SshTransport("bench@gpubox", "/scratch/spool", port=2222)
    assert seen == {"host_keys": True, "policy": "RejectPolicy", "connect": ("gpubox", 2222, "bench")}     # unknown hosts are refused
    spool_on_host = str(host_root / "scratch" / "spool")
    assert sorted(os.listdir(spool_on_host)) == ["done", "incoming", "running"]
    tr.put_text_atomic("incoming/j1.json", json.dumps({"op": "no_such_op", "impl": "ours", "nproc": 1, "backend": "gloo", "timeout_s": 60}))
    assert os.listdir(os.path.join(spool_on_host, "incoming")) == ["j1.json"]                              # no temporary name left behind
    assert remote.serve(spool_on_host, once=True, log=lambda *_: None) == 1                               # the worker runs on the "host"
    res = json.loads(tr.get_text("done/j1/result.json"))
    assert res["returncode"] != 0 and res["job_id"] == "j1"
    os.makedirs(os.path.join(spool_on_host, "done", "j1", "artifacts", "traces"), exist_ok=True)
    for rel in ("rank_0.pt", "traces/rank_0.json"):
        with open(os.path.join(spool_on_host, "done", "j1", "artifacts", rel), "w") as fh:
            fh.write("x")
    got = tr.fetch_tree("done/j1/artifacts", str(tmp_path / "fetched"))
    assert got == ["rank_0.pt", "traces/rank_0.json"] and os.path.exists(tmp_path / "fetched" / "traces" / "rank_0.json")
    assert tr.get_text("done/missing/result.json") is None
    tr.remove_tree("done/j1")
    assert os.listdir(os.path.join(spool_on_host, "done")) == []


def test_a_restarted_worker_requeues_what_its_predecessor_left_unfinished(tmp_path, monkeypatch):
    monkeypatch.setattr(launch, "LOGS_ROOT", str(tmp_path / "logs"))
    spool = str(tmp_path / "spool")
    tr = remote.LocalTransport(spool)
    tr.put_text_atomic("running/orphan.json", json.dumps({"op": "no_such_op", "impl": "ours", "nproc": 1, "backend": "gloo", "timeout_s": 60}))
    lines = []
    assert remote.serve(spool, once=True, log=lines.append) == 1
    assert any("re-queued unfinished job orphan" in ln for ln in lines)
    assert json.loads(tr.get_text("done/orphan/result.json"))["job_id"] == "orphan"
    assert os.listdir(os.path.join(spool, "running")) == []


def test_claims_of_live_or_foreign_workers_are_left_alone(tmp_path, monkeypatch):
    import socket

    monkeypatch.setattr(launch, "LOGS_ROOT", str(tmp_path / "logs"))
    spool = str(tmp_path / "spool")
    tr = remote.LocalTransport(spool)
    payload = json.dumps({"op": "no_such_op", "impl": "ours", "nproc": 1, "backend": "gloo", "timeout_s": 60})
    tr.put_text_atomic("running/live.json", payload)
    tr.put_text_atomic("running/live.json.owner", f"{socket.gethostname()} {os.getppid()}")       # a process that exists
    tr.put_text_atomic("running/elsewhere.json", payload)
    tr.put_text_atomic("running/elsewhere.json.owner", "some-other-host 1")
    tr.put_text_atomic("running/dead.json", payload)
    tr.put_text_atomic("running/dead.json.owner", f"{socket.gethostname()} 2147483646")           # no such pid
    assert remote.serve(spool, once=True, log=lambda *_: None) == 1
    assert sorted(n for n in os.listdir(os.path.join(spool, "running")) if n.endswith(".json")) == ["elsewhere.json", "live.json"]
    assert os.path.exists(os.path.join(spool, "done", "dead", "result.json"))
