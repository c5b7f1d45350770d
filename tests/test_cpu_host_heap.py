"""The CPU twin of the symmetric heap: protocol correctness, stress, and host-side fault injection.

Ranks are plain child processes sharing a POSIX segment; no GPU and no torch.distributed involved.
Failures are made on the host: a rank that drops a signal, a rank that never arrives, a late rank.
"""
import multiprocessing as mp
import os
import time

import pytest
import torch

from parallelkernelbench_b200.parallel.host_heap import HostCollectiveTimeout, HostHeap

CTX = mp.get_context("spawn")


def _run(target, world, *args, timeout=120):
    name = f"/pkb200_test_{os.getpid()}_{time.time_ns() % 10**9}"
    q = CTX.Queue()
    procs = [CTX.Process(target=target, args=(name, r, world, q, *args)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    deadline = time.time() + timeout
    while len(out) < world and time.time() < deadline:
        try:
            r, v = q.get(timeout=1.0)
            out[r] = v
        except Exception:
            if not any(p.is_alive() for p in procs) and q.empty():
                break
    for p in procs:
        p.join(timeout=10)
        if p.is_alive():
            p.kill()
    return out


def _collectives_body(name, rank, world, q):
    h = HostHeap.create(nbytes=8 << 20, name=name, rank=rank, world=world, timeout_ms=20000)
    try:
        g = torch.Generator().manual_seed(rank)
        x = torch.randn(4096, generator=g)
        ar = h.all_reduce(x)
        ag = h.all_gather(ar).reshape(-1)
        rs = h.reduce_scatter(ag)
        a2a = h.all_to_all(torch.full((world, 5), float(10 * rank)) + torch.arange(world).view(-1, 1))
        bc = h.broadcast(torch.full((7,), float(rank)), src=world - 1)
        mx = h.all_reduce(torch.tensor([float(rank)]), op="max")
        i64 = h.all_reduce(torch.tensor([rank + 1], dtype=torch.int64))
        bf = h.all_reduce(torch.full((33,), 1.5, dtype=torch.bfloat16))
        for _ in range(200):                      # epoch protocol under repetition
            s = h.all_reduce(torch.ones(16))
            assert float(s[0]) == world
        res = {"ar": ar, "rs": rs, "a2a": a2a, "bc": bc, "mx": mx, "i64": i64, "bf": bf.float()}
        q.put((rank, {k: v.numpy().copy() for k, v in res.items()}))   # plain arrays: no shared-storage hand-off
    finally:
        h.close()


@pytest.mark.parametrize("world", [2, 4])
def test_host_collectives_match_closed_form(world):
    out = _run(_collectives_body, world)
    assert sorted(out) == list(range(world))
    xs = [torch.randn(4096, generator=torch.Generator().manual_seed(r)) for r in range(world)]
    total = xs[0].clone()
    for v in xs[1:]:
        total = total + v
    out = {r: {k: torch.from_numpy(v) for k, v in d.items()} for r, d in out.items()}
    for r in range(world):
        torch.testing.assert_close(out[r]["ar"], total, atol=1e-5, rtol=1e-5)
        expect_rs = (total.repeat(world) * world).reshape(world, -1)[r]
        torch.testing.assert_close(out[r]["rs"], expect_rs, atol=1e-4, rtol=1e-5)
        assert torch.equal(out[r]["a2a"][:, 0], torch.tensor([10.0 * s + r for s in range(world)]))
        assert torch.equal(out[r]["bc"], torch.full((7,), float(world - 1)))
        assert float(out[r]["mx"]) == world - 1 and int(out[r]["i64"]) == world * (world + 1) // 2
        assert torch.all(out[r]["bf"] == 1.5 * world)


def _dropped_signal_body(name, rank, world, q):
    h = HostHeap.create(nbytes=2 << 20, name=name, rank=rank, world=world, timeout_ms=20000)
    try:
        h.barrier()
        if rank == 1:
            h.drop_signals(1)                     # injected fault: rank 1 never signals this barrier
        try:
            h.all_reduce(torch.ones(8), timeout_ms=400)
            q.put((rank, "ok"))
        except HostCollectiveTimeout as e:
            q.put((rank, ("timeout", e.missing_peer)))
    finally:
        h.close()


def test_dropped_signal_is_detected_and_names_the_peer():
    out = _run(_dropped_signal_body, 2)
    assert out[0] == ("timeout", 1)              # the survivor names the silent rank within its budget


def _missing_rank_body(name, rank, world, q):
    if rank == world - 1:
        q.put((rank, "never joined"))            # this rank exits before mapping the heap
        return
    try:
        h = HostHeap.create(nbytes=2 << 20, name=name, rank=rank, world=world, timeout_ms=3000)
    except RuntimeError as e:
        q.put((rank, ("create_failed", str(e))))
        return
    try:
        t0 = time.time()
        try:
            h.barrier(timeout_ms=300)
            q.put((rank, "ok"))
        except HostCollectiveTimeout as e:
            q.put((rank, ("timeout", e.missing_peer, time.time() - t0)))
    finally:
        h.close()


def test_rank_that_never_joins_times_out_the_others():
    out = _run(_missing_rank_body, 3)
    for r in (0, 1):
        assert out[r][0] == "timeout" and out[r][1] == 2 and out[r][2] < 5.0


def _late_rank_body(name, rank, world, q):
    h = HostHeap.create(nbytes=2 << 20, name=name, rank=rank, world=world, timeout_ms=20000)
    try:
        if rank == 0:
            h.delay_ms(150)                       # a slow rank inside the budget is not an error
        s = h.all_reduce(torch.full((4,), float(rank + 1)), timeout_ms=5000)
        q.put((rank, float(s[0])))
    finally:
        h.close()


def test_late_rank_inside_budget_still_completes():
    out = _run(_late_rank_body, 2)
    assert out == {0: 3.0, 1: 3.0}


def test_guard_bands_catch_single_byte_overruns_and_underruns(monkeypatch):
    import ctypes
    import os

    import pytest

    from parallelkernelbench_b200 import _native as nv
    from parallelkernelbench_b200.parallel import guards
    from parallelkernelbench_b200.parallel.host_heap import HostHeap

    monkeypatch.setenv("PKB_HEAP_GUARD", "1")
    heap = HostHeap.create(nbytes=4 << 20, name=f"/pkb200_{os.getpid()}_guardtest", rank=0, world=1)
    try:
        a, b = heap.alloc_bytes(100), heap.alloc_bytes(4096)
        assert a % 64 == 0 and b % 64 == 0 and b >= a + 100 + guards.GUARD_BYTES
        assert heap.check_guards() == []
        base = nv.host_lib().pkbh_heap_local(heap.handle)
        ctypes.memset(base + a, 0x11, 100)                              # the allocation itself may be written freely
        assert heap.check_guards() == []
        ctypes.memset(base + a + 100, 0x22, 1)                          # one byte past the end of the first allocation
        ctypes.memset(base + b - 3, 0x33, 2)                            # bytes 3 and 2 before the second one
        with pytest.raises(guards.GuardViolation, match="1 byte\\(s\\) after"):
            heap.check_guards()
        bad = heap.check_guards(raise_on_violation=False)
        assert {(v["offset"], v["side"], v["distance"]) for v in bad} == {(a, "after", 1), (b, "before", 2)}
    finally:
        heap.close()


def test_collectives_run_clean_under_guard_bands():
    """The plumbing sequence (all-reduce, all-gather, reduce-scatter) on two CPU ranks with every heap allocation guarded."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "parallelkernelbench_b200.harness.launch", "run", "--op", "plumbing", "--impl", "ours", "--nproc", "2",
                        "--backend", "gloo", "--dtype", "float32"], cwd=root, capture_output=True, text=True, timeout=300,
                       env={**os.environ, "PKB_HEAP_GUARD": "1"})
    assert r.returncode == 0 and "dry run ok" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]
