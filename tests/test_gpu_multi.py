"""Multi-rank GPU tests: each launches torchrun children (one rank per GPU) and checks their verdicts.

The single-rank forms run on any GPU box; the N > 1 forms need at least two GPUs.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _torchrun(script, nproc, *args, port=29600, timeout=900):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, script), *args]
    return subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=timeout)


def _assert_ok(r):
    assert r.returncode == 0 and "TOTAL_FAILS 0" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_collectives_single_rank():
    _assert_ok(_torchrun("tests/mp/collectives_worker.py", 1, port=29601))


def test_tp_mlp_single_rank():
    _assert_ok(_torchrun("tests/mp/tp_mlp_worker.py", 1, port=29602))


@pytest.mark.multigpu
@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_collectives_multi_rank(nproc):
    if _ngpus() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    _assert_ok(_torchrun("tests/mp/collectives_worker.py", nproc, port=29610 + nproc))


@pytest.mark.multigpu
@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_tp_mlp_multi_rank(nproc):
    if _ngpus() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    _assert_ok(_torchrun("tests/mp/tp_mlp_worker.py", nproc, port=29620 + nproc))


def test_moe_single_rank():
    _assert_ok(_torchrun("tests/mp/moe_worker.py", 1, port=29603))


def test_all_ops_single_rank():
    _assert_ok(_torchrun("tests/mp/all_ops_worker.py", 1, port=29604))


@pytest.mark.multigpu
@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_moe_and_all_ops_multi_rank(nproc):
    if _ngpus() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    _assert_ok(_torchrun("tests/mp/moe_worker.py", nproc, port=29630 + nproc))
    _assert_ok(_torchrun("tests/mp/all_ops_worker.py", nproc, port=29640 + nproc))


def test_ring_attention_single_rank():
    r = _torchrun("tests/mp/all_ops_worker.py", 1, "--ops", "ring_attention,flash_attention", port=29605)
    _assert_ok(r)


@pytest.mark.multigpu
@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_ring_attention_multi_rank(nproc):
    if _ngpus() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    _assert_ok(_torchrun("tests/mp/all_ops_worker.py", nproc, "--ops", "ring_attention", "--config", "default", port=29650 + nproc))


def test_fsdp_llama_single_rank():
    _assert_ok(_torchrun("tests/mp/llama_worker.py", 1, port=29606))


@pytest.mark.multigpu
@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_fsdp_llama_multi_rank(nproc):
    if _ngpus() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    _assert_ok(_torchrun("tests/mp/llama_worker.py", nproc, port=29660 + nproc))


def test_harness_eval_on_gpu_single_rank():
    env = dict(os.environ, PKB_LOGS_DIR=os.path.join(ROOT, "logs", "pytest_gpu"), PKB_COOLDOWN_SEC="0")
    r = subprocess.run([sys.executable, "-m", "parallelkernelbench_b200.harness.launch", "eval", "--op", "allreduce",
                        "--nproc", "1", "--trials", "1", "--measure-perf", "--warmup", "5", "--iters", "10"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "all trials match" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
