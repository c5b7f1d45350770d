"""Prompt assembly and the generate -> evaluate -> feedback loop (a recorded wrong candidate, then a right one)."""
import os


def test_prompt_contains_contract_reference_and_hardware():
    from parallelkernelbench_b200.kernelgen import build_prompt

    p = build_prompt("gemm_allreduce", nproc=8)
    assert "def solution(rc, *inputs)" in p and "tcgen05" in p and "_gar_ref" in p and "--solution" in p
    assert "Result of your previous attempt" not in p
    assert "verdict: tensor_mismatch" in build_prompt("allreduce", feedback="verdict: tensor_mismatch")


def test_loop_stops_at_first_matching_candidate(tmp_path):
    from parallelkernelbench_b200.kernelgen import ReplayProposer, optimise

    cands = tmp_path / "cands"
    cands.mkdir()
    (cands / "a_wrong.py").write_text("def solution(rc, x):\n    return x * 2\n")
    (cands / "b_right.py").write_text("def solution(rc, x):\n    return rc.comm.all_reduce(x)\n")
    (cands / "c_unused.py").write_text("def solution(rc, x):\n    raise RuntimeError('never evaluated')\n")
    out = optimise("allreduce", ReplayProposer(str(cands)), str(tmp_path / "work"), nproc=2, max_iters=3, backend="gloo",
                   dtype="float32", config="small", timeout_s=300)
    assert out["solved"] and len(out["attempts"]) == 2
    assert not out["attempts"][0]["all_ok"] and "verdict" in out["attempts"][0]["feedback"]
    assert os.path.isfile(out["attempts"][1]["path"])


def test_worked_examples_are_in_the_prompt_and_pass_the_evaluation():
    """Every example file is a solution that matches its op's reference (2 CPU ranks), and the prompt of another op shows
    the pairs while the prompt of the same op does not give its own answer away."""
    from parallelkernelbench_b200.harness import launch
    from parallelkernelbench_b200.kernelgen import build_prompt
    from parallelkernelbench_b200.kernelgen.examples import EXAMPLES, example_path

    p = build_prompt("allgather")
    assert "Worked examples" in p and "rc.comm.all_reduce(x)" in p and "all_to_all" in p
    assert "allreduce_symmetric_heap" not in build_prompt("allreduce") and "Example solution for the op `allreduce`" not in build_prompt("allreduce")
    import importlib.util

    spec = importlib.util.spec_from_file_location("example_own_kernel", example_path("tp_rmsnorm"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert hasattr(mod._kernels(), "ex_row_scale")            # the example's CUDA source builds for sm_100a without a GPU
    for op in EXAMPLES:
        if op in ("allreduce", "gemm_allreduce"):    # the one-line solution is evaluated by the loop tests of this file; the
            continue                                  # GEMM example takes its PyTorch branch on CPU ranks (nothing of its own to check)
        s = launch.eval_op(op, 2, trials=1, backend="gloo", dtype="float32", config="small", solution=str(example_path(op)),
                           timeout_s=300)
        assert s["all_ok"], (op, s["trials"][-1].get("result"))


def test_prompt_cli_selects_ops_by_name_number_list_and_all(tmp_path):
    from parallelkernelbench_b200.kernelgen.__main__ import main
    from parallelkernelbench_b200.kernelgen.prompt import build_prompt, select_ops
    from parallelkernelbench_b200.workloads import registry

    assert select_ops("13") == ["gemm_allreduce"] and select_ops("[1, allreduce, 8]") == ["allreduce", "alltoall"]
    assert len(select_ops("all")) == len(registry.all_ops())
    assert "fp32 and round once" in build_prompt("allreduce", precision="bfloat16").replace("\n", " ")
    assert main(["prompt", "--op", "1,13", "--out-dir", str(tmp_path)]) == 0
    assert sorted(p.name for p in tmp_path.iterdir()) == ["prompt_allreduce.md", "prompt_gemm_allreduce.md"]
    assert "def solution(rc, *inputs)" in (tmp_path / "prompt_allreduce.md").read_text()


def test_command_proposer_extracts_code_and_loop_records_the_run(tmp_path):
    """A stand-in "model" (a script that prints prose with a fenced block) drives the loop through CommandProposer."""
    import json
    import sys

    from parallelkernelbench_b200.kernelgen import CommandProposer, extract_code, optimise

    assert extract_code("text\n```python\nx = 1\n```\nmore\n```python\ny = 2\n```") == "x = 1\n"
    assert extract_code("```\nz = 3\n```") == "z = 3\n" and extract_code("w = 4") == "w = 4\n"
    model = tmp_path / "model.py"
    model.write_text("import sys\nprompt = sys.stdin.read()\nassert 'def solution(rc, *inputs)' in prompt\n"
                     "print('Here is my answer:\\n```python\\ndef solution(rc, x):\\n    return rc.comm.all_reduce(x)\\n```')\n")
    work = tmp_path / "work"
    out = optimise("allreduce", CommandProposer([sys.executable, str(model)], log_dir=str(work / "ex")), str(work), nproc=2, max_iters=2,
                   backend="gloo", dtype="float32", config="small", timeout_s=300)
    assert out["solved"] and len(out["attempts"]) == 1
    rec = json.loads((work / "allreduce_run.json").read_text())
    assert rec["solved"] and rec["op"] == "allreduce"
    ex = json.loads((work / "ex" / "exchange_0.json").read_text())
    assert "Here is my answer" in ex["reply"] and ex["returncode"] == 0
    failing = CommandProposer([sys.executable, "-c", "import sys; sys.exit(3)"])
    out = optimise("allreduce", failing, str(tmp_path / "w2"), nproc=2, max_iters=2, backend="gloo", dtype="float32", config="small")
    assert not out["solved"] and out["attempts"] == []


def test_loop_screens_candidates_keeps_a_trajectory_and_resumes(tmp_path):
    """A candidate that names a forbidden construct is never launched and its attempt is fed back; every event of the run is
    in the trajectory file; a resumed run continues the attempt numbering and keeps the best matching candidate."""
    import json

    from parallelkernelbench_b200.kernelgen import optimise

    bad = "SRC = '" + "cuda" + "Memcpy" + "Batch" + "Async(a, b, c)'\ndef solution(rc, x):\n    return x\n"
    good = "def solution(rc, x):\n    return rc.comm.all_reduce(x)\n"
    replies = iter([bad, good])
    seen_feedback = []

    def propose(prompt, feedback):
        seen_feedback.append(feedback)
        return next(replies)

    out = optimise("allreduce", propose, str(tmp_path), nproc=2, max_iters=3, backend="gloo", dtype="float32", config="small")
    assert out["solved"] and len(out["attempts"]) == 2
    assert out["attempts"][0]["screened_out"] and out["attempts"][0]["path"] is None
    assert "rejected before evaluation" in seen_feedback[1]
    assert out["best"]["iteration"] == 1 and os.path.exists(out["best"]["path"])
    assert not os.path.exists(tmp_path / "allreduce_candidate_0.py")            # the refused text is not kept as a runnable file
    events = [json.loads(line)["event"] for line in open(tmp_path / "allreduce_trajectory.jsonl")]
    assert events == ["prompt", "screened_out", "prompt", "candidate", "evaluated"]

    more = optimise("allreduce", lambda p, f: good, str(tmp_path), nproc=2, max_iters=1, backend="gloo", dtype="float32",
                    config="small", resume=True)
    assert [a["iteration"] for a in more["attempts"]] == [0, 1, 2] and more["solved"]


def test_http_proposer_talks_to_a_chat_completions_endpoint(tmp_path, monkeypatch):
    """A local HTTP server stands in for the model endpoint: first reply wrong, second right (prose around a fenced block);
    the key goes out as a bearer token and is not written to the exchange log."""
    import json
    import threading
    from http.server import BaseHTTPRequestHandler, HTTPServer

    from parallelkernelbench_b200.kernelgen import HttpProposer, optimise

    replies = ["Here you go:\n```python\ndef solution(rc, x):\n    return x * 2\n```\n",
               "Fixed, the sum was missing.\n```python\ndef solution(rc, x):\n    return rc.comm.all_reduce(x)\n```\nDone."]
    seen = []

    class Handler(BaseHTTPRequestHandler):
        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            seen.append({"path": self.path, "auth": self.headers.get("Authorization"), "model": body["model"],
                         "roles": [m["role"] for m in body["messages"]], "user": body["messages"][-1]["content"]})
            if len(seen) > len(replies):
                self.send_response(500)
                self.end_headers()
                return
            out = json.dumps({"choices": [{"message": {"role": "assistant", "content": replies[len(seen) - 1]}}]}).encode()
            self.send_response(200)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(out)))
            self.end_headers()
            self.wfile.write(out)

        def log_message(self, *a):
            pass

    srv = HTTPServer(("127.0.0.1", 0), Handler)
    th = threading.Thread(target=srv.serve_forever, daemon=True)
    th.start()
    monkeypatch.setenv("PKB_KERNELGEN_API_KEY", "sk-test-123")
    try:
        prop = HttpProposer(f"http://127.0.0.1:{srv.server_port}/v1", "local-model", log_dir=str(tmp_path / "ex"), timeout_s=30)
        out = optimise("allreduce", prop, str(tmp_path / "work"), nproc=2, max_iters=3, backend="gloo", dtype="float32", config="small",
                       timeout_s=300)
        assert out["solved"] and len(out["attempts"]) == 2
        assert [s["path"] for s in seen] == ["/v1/chat/completions"] * 2 and seen[0]["auth"] == "Bearer sk-test-123"
        assert seen[0]["model"] == "local-model" and seen[0]["roles"] == ["system", "user"]
        assert "Result of your previous attempt" in seen[1]["user"] and "Result of your previous attempt" not in seen[0]["user"]
        logged = (tmp_path / "ex" / "exchange_0.json").read_text()
        assert "sk-test-123" not in logged and "def solution" in logged
        # an endpoint that fails ends the run instead of raising
        out2 = optimise("allgather", prop, str(tmp_path / "work2"), nproc=2, max_iters=2, backend="gloo", dtype="float32", config="small")
        assert not out2["solved"] and out2["attempts"] == []
    finally:
        srv.shutdown()


def test_prompt_templates_come_from_toml_and_can_be_overridden(tmp_path):
    from parallelkernelbench_b200.kernelgen import build_prompt
    from parallelkernelbench_b200.kernelgen.__main__ import main
    from parallelkernelbench_b200.kernelgen.prompt import load_templates

    base = load_templates()
    assert {"contract", "hardware", "precision"} <= set(base) and "b200_8" in base["hardware"] and "{op}" in base["contract"]
    extra = tmp_path / "mine.toml"
    extra.write_text("[hardware]\nlab_2 = '''two GPUs of the lab machine, NVLink bridge'''\n[precision]\nbfloat16 = '''keep sums in fp32 (site rule)'''\n")
    p = build_prompt("allreduce", hardware="lab_2", nproc=2, precision="bfloat16", templates=str(extra))
    assert "two GPUs of the lab machine" in p and "site rule" in p and "def solution(rc, *inputs)" in p        # contract kept
    assert "lab_2" not in load_templates()["hardware"]                                                       # the packaged file is untouched
    out_dir = tmp_path / "prompts"
    assert main(["prompt", "--op", "[1, 13]", "--hardware", "lab_2", "--nproc", "2", "--prompts", str(extra), "--out-dir", str(out_dir)]) == 0
    assert sorted(f.name for f in out_dir.iterdir()) == ["prompt_allreduce.md", "prompt_gemm_allreduce.md"]
    assert "two GPUs of the lab machine" in (out_dir / "prompt_gemm_allreduce.md").read_text()


def test_generate_wants_exactly_one_source_of_candidates():
    import pytest

    from parallelkernelbench_b200.kernelgen.__main__ import main

    for argv in (["generate", "--op", "allreduce"],
                 ["generate", "--op", "allreduce", "--command", "cat", "--endpoint", "http://127.0.0.1:1/v1", "--model", "m"],
                 ["generate", "--op", "allreduce", "--endpoint", "http://127.0.0.1:1/v1"]):
        with pytest.raises(SystemExit) as e:
            main(argv)
        assert e.value.code == 2
