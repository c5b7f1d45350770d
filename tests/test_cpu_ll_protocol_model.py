"""Host model of the no-barrier (data + epoch in one store) exchange used by the small all-reduce and all-gather.

The device kernels (`coll_allreduce_ll_kernel`, `coll_allgather_ll_kernel`) keep two slot sets that alternate with the parity
of a per-rank epoch and never wait for a peer except on the words they are about to read. This model runs the same protocol
with Python threads as ranks - every (data, epoch) pair is one atomic tuple store, ranks are delayed at random between the
steps - and checks the claim the kernels rest on: a rank can run at most one call ahead of any peer, so two parities are
enough and no call ever reads a word of another call."""
import random
import threading
import time


class _Rank:
    def __init__(self, world, cap):
        self.epoch = 0                                                       # header word, advanced at the end of a call
        self.slots = [[[(0, 0)] * cap for _ in range(world)] for _ in range(2)]     # [parity][source][unit] = (data, epoch)


def _all_reduce_call(ranks, me, values, rng, budget_s=20.0):
    world, mine = len(ranks), ranks[me]
    epoch = mine.epoch + 1
    par = epoch & 1
    for i, w in enumerate(values):                                           # send: my word into slot [par][me] of everyone
        for g in range(world):
            ranks[g].slots[par][me][i] = (w, epoch)
            if rng.random() < 0.02:
                time.sleep(0)
    out = []
    t0 = time.time()
    for i in range(len(values)):                                             # receive: poll the pairs of every source
        acc = 0
        for g in range(world):
            while True:
                w, e = mine.slots[par][g][i]
                if e == epoch:
                    break
                assert e < epoch, f"rank {me} call {epoch}: unit {i} of source {g} carries a FUTURE epoch {e}"
                assert time.time() - t0 < budget_s, "peer never arrived"
                time.sleep(0)
            acc += w
        out.append(acc)
    mine.epoch = epoch                                                       # the last block advances the epoch
    return out


def _run(world, calls, cap, seed):
    ranks = [_Rank(world, cap) for _ in range(world)]
    master = random.Random(seed)
    sizes = [master.randint(1, cap) for _ in range(calls)]
    inputs = [[[master.randint(-1000, 1000) for _ in range(sizes[c])] for c in range(calls)] for _ in range(world)]
    errors, results = [], [[None] * calls for _ in range(world)]

    def body(r):
        rng = random.Random(seed * 100 + r)
        try:
            for c in range(calls):
                if rng.random() < 0.3:
                    time.sleep(rng.random() * 0.002)                         # this rank falls behind for a while
                results[r][c] = _all_reduce_call(ranks, r, inputs[r][c], rng)
        except BaseException as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=body, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(120)
    assert not errors, errors[0]
    for c in range(calls):
        want = [sum(inputs[r][c][i] for r in range(world)) for i in range(sizes[c])]
        for r in range(world):
            assert results[r][c] == want, (r, c)


def test_two_parities_suffice_for_any_interleaving():
    for world, seed in ((2, 1), (4, 2), (8, 3)):
        _run(world, calls=60, cap=24, seed=seed)


def test_one_parity_would_not_be_enough():
    """The same protocol with a single slot set must be caught by the model (a fast rank overwrites words a slow rank has
    not read yet): this guards the model itself against being vacuous."""
    world, cap = 2, 4
    ranks = [_Rank(world, cap) for _ in range(world)]
    for r in ranks:
        r.slots[1] = r.slots[0]                                              # both parities alias one buffer
    # rank 0 completes call 1 only after rank 1 has sent; then it races ahead into call 2 and overwrites its own slot in
    # rank 1 before rank 1 has read call 1
    rng = random.Random(0)
    done = {}

    def fast():
        done["a1"] = _all_reduce_call(ranks, 0, [1, 2, 3, 4], rng)
        for g in range(world):                                               # the send phase of call 2
            for i in range(4):
                ranks[g].slots[0][0][i] = (100 + i, 2)

    ranks[1].slots[0][1] = [(10 * (i + 1), 1) for i in range(4)]             # rank 1 has sent call 1 to rank 0 ...
    ranks[0].slots[0][1] = [(10 * (i + 1), 1) for i in range(4)]
    fast()
    # ... but only now reads it: the words of rank 0 already belong to call 2
    try:
        _all_reduce_call(ranks, 1, [10, 20, 30, 40], rng, budget_s=0.5)
    except AssertionError as e:
        assert "FUTURE epoch" in str(e)
    else:
        raise AssertionError("the single-buffer variant must fail")


def test_two_result_buffers_and_one_closing_barrier_are_enough():
    """Model of the fused GEMV + all-gather (`tp_gemv_allgather_kernel`): every call stores this rank's block into buffer
    (call & 1) of every rank and ends with one barrier; the caller reads the buffer only after its own call has ended. A rank
    that races ahead may already be storing call c+1 (other buffer) while a slow rank still reads call c, but it cannot reach
    call c+2 before the slow rank has passed the barrier of c+1, i.e. has finished reading c."""
    world, calls = 4, 80
    bufs = [[[None] * world for _ in range(2)] for _ in range(world)]        # [rank][parity][source block] = call index
    barrier = threading.Barrier(world)
    errors = []

    def body(r):
        rng = random.Random(r)
        try:
            for c in range(calls):
                for g in range(world):
                    bufs[g][c & 1][r] = c                                    # my block lands in everyone's buffer of this call
                    if rng.random() < 0.1:
                        time.sleep(0)
                barrier.wait(30)                                             # the kernel's closing barrier
                if rng.random() < 0.3:
                    time.sleep(rng.random() * 0.002)                         # the consumer is slow to read
                got = list(bufs[r][c & 1])
                assert got == [c] * world, f"rank {r} call {c} read {got}"
        except BaseException as e:  # noqa: BLE001
            errors.append(e)
            barrier.abort()

    threads = [threading.Thread(target=body, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(120)
    assert not errors, errors[0]


def test_native_stress_of_the_exchange_protocol_with_real_threads(tmp_path):
    """The C++ form of the model above (relaxed 64-bit atomics for the {data, epoch} pairs, one thread per rank), also under
    ThreadSanitizer when the toolchain has it; the single-slot-set variant must fail."""
    import os
    import shutil
    import subprocess

    gxx = shutil.which("g++")
    if gxx is None:
        import pytest

        pytest.skip("no g++")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(root, "parallelkernelbench_b200", "csrc", "hosttests", "ll_protocol_stress.cpp")
    exe = str(tmp_path / "ll_stress")
    subprocess.run([gxx, "-O2", "-std=c++17", "-pthread", src, "-o", exe], check=True, capture_output=True)
    for args in (("4", "600", "64"), ("8", "300", "32")):
        r = subprocess.run([exe, *args], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0 and "OK" in r.stdout, r.stdout + r.stderr
    # with one slot set a rank that runs ahead overwrites unread words: a timing matter, so allow a few attempts
    assert any(subprocess.run([exe, "2", "3000", "16", "single"], capture_output=True, text=True, timeout=120).returncode == 1
               for _ in range(4))
    tsan = str(tmp_path / "ll_stress_tsan")
    built = subprocess.run([gxx, "-O1", "-g", "-std=c++17", "-pthread", "-fsanitize=thread", src, "-o", tsan], capture_output=True)
    if built.returncode == 0:
        r = subprocess.run([tsan, "4", "150", "32"], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0 and "ThreadSanitizer" not in r.stderr, r.stdout + r.stderr[-2000:]


def test_native_model_of_the_grid_wide_barrier(tmp_path):
    """Threads as blocks of several ranks run the grid-wide cross-rank barrier with the device code's memory orders; payloads
    are plain stores read by another block index of another rank, so ThreadSanitizer checks the happens-before chain. The
    per-block-index barrier in its place must be caught."""
    import os
    import shutil
    import subprocess

    gxx = shutil.which("g++")
    if gxx is None:
        import pytest

        pytest.skip("no g++")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(root, "parallelkernelbench_b200", "csrc", "hosttests", "grid_barrier_stress.cpp")
    exe = str(tmp_path / "gb")
    subprocess.run([gxx, "-O2", "-std=c++17", "-pthread", src, "-o", exe], check=True, capture_output=True)
    for args in (("4", "6", "400"), ("2", "12", "400")):
        r = subprocess.run([exe, *args], capture_output=True, text=True, timeout=180)
        assert r.returncode == 0 and "OK" in r.stdout, r.stdout + r.stderr
    assert any(subprocess.run([exe, "4", "6", "2000", "blockonly"], capture_output=True, text=True, timeout=180).returncode == 1
               for _ in range(4))
    tsan = str(tmp_path / "gb_tsan")
    if subprocess.run([gxx, "-O1", "-g", "-std=c++17", "-pthread", "-fsanitize=thread", src, "-o", tsan], capture_output=True).returncode == 0:
        r = subprocess.run([tsan, "3", "4", "120"], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0 and "ThreadSanitizer" not in r.stderr, r.stdout + r.stderr[-2000:]
