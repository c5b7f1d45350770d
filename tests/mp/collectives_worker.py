"""Per-rank body of the multi-GPU collective tests (launched by torchrun, one rank per GPU).

Every symmetric-heap collective is compared against torch.distributed (NCCL) on the same inputs.
Prints one ``PASS``/``FAIL`` line per case and exits non-zero if anything failed.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from parallelkernelbench_b200 import _native as nv  # noqa: E402
from parallelkernelbench_b200.ops import collectives as C  # noqa: E402
from parallelkernelbench_b200.parallel import init_context  # noqa: E402


def main() -> int:
    os.environ.setdefault("PKB_HEAP_GIB", "4")       # the bandwidth lines keep several 128 MiB x W buffers in the heap
    ctx = init_context()
    heap = ctx.heap()
    g = heap.world_group
    W, r = ctx.world, ctx.rank
    dev = ctx.device
    fails = 0

    def report(name, ok, extra=""):
        nonlocal fails
        if not ok:
            fails += 1
        if r == 0 or not ok:
            print(f"{'PASS' if ok else 'FAIL'} rank{r} {name} {extra}", flush=True)

    if r == 0:
        print(f"heap base={heap.base:#x} stride={heap.stride:#x} mc_base={heap.mc_base:#x} world={W}", flush=True)
    gen = torch.Generator(device=dev).manual_seed(100 + r)
    for dtype in (torch.bfloat16, torch.float32):
        for n in (8, 1000, 4096, 65536 + 24, 1 << 20, (1 << 22) + 8):
            x = torch.randn(n, device=dev, dtype=dtype, generator=gen)
            ref = x.clone()
            dist.all_reduce(ref)
            tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
            algos = ["oneshot", "twoshot"] + (["nvls"] if heap.mc_base else []) + (["ll"] if n * x.element_size() <= (1 << 20) and W > 1 else [])
            for algo in algos:
                if algo not in ("oneshot", "ll") and n % 8 != 0:
                    continue
                y = C.all_reduce(x, g, algo=algo)
                torch.cuda.synchronize()
                ok = torch.allclose(y.float(), ref.float(), atol=tol * (W ** 0.5), rtol=tol)
                report(f"all_reduce[{algo}] {dtype} n={n}", ok, f"maxerr={(y.float() - ref.float()).abs().max().item():.3g}")
    # max / min / int
    x = torch.randn(4099, device=dev, generator=gen)
    for op, rop in (("max", dist.ReduceOp.MAX), ("min", dist.ReduceOp.MIN)):
        ref = x.clone(); dist.all_reduce(ref, op=rop)
        report(f"all_reduce {op}", torch.equal(C.all_reduce(x, g, op=op), ref))
    xi = torch.randint(-1000, 1000, (777,), device=dev, dtype=torch.int64, generator=gen)
    ref = xi.clone(); dist.all_reduce(ref)
    report("all_reduce int64", torch.equal(C.all_reduce(xi, g), ref))
    # exactly representable inputs -> bitwise equality expected (constant rank+1 pattern)
    xc = torch.full((1024, 1024), float(r + 1), device=dev, dtype=torch.bfloat16)
    ref = xc.clone(); dist.all_reduce(ref)
    for algo in ["oneshot", "twoshot"] + (["nvls"] if heap.mc_base else []):
        report(f"all_reduce[{algo}] constant 2MiB bitwise", torch.equal(C.all_reduce(xc, g, algo=algo), ref))

    # all_gather
    x = torch.randn(513, 64, device=dev, dtype=torch.bfloat16, generator=gen)
    ref = torch.empty(W, 513, 64, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(ref.view(W * 513, 64), x)
    report("all_gather", torch.equal(C.all_gather(x, g), ref))
    for rows in (1, 7, 4096):                     # no-barrier path (small), and the staged path (large)
        x = torch.randn(rows, 96, device=dev, dtype=torch.float32, generator=gen)
        ref = torch.empty(W, rows, 96, device=dev)
        dist.all_gather_into_tensor(ref.view(W * rows, 96), x)
        report(f"all_gather fp32 rows={rows}", torch.equal(C.all_gather(x, g), ref))
    same = True
    for i in range(30):                            # back-to-back calls of alternating sizes: epochs and slot parity
        xi = torch.full((16 + (i % 3) * 5,), float(r * 100 + i), device=dev)
        got = C.all_gather(xi, g)
        same &= all(bool((got[s] == float(s * 100 + i)).all()) for s in range(W))
    report("all_gather no-barrier path x30 alternating sizes", same)
    # reduce_scatter
    x = torch.randn(W * 300, 40, device=dev, dtype=torch.float32, generator=gen)
    ref = torch.empty(300, 40, device=dev)
    dist.reduce_scatter_tensor(ref, x)
    y = C.reduce_scatter(x, g)
    report("reduce_scatter", torch.allclose(y, ref, atol=1e-5, rtol=1e-5))
    # all_to_all
    x = torch.randn(W, 1000, device=dev, dtype=torch.bfloat16, generator=gen)
    ref = torch.empty_like(x)
    dist.all_to_all_single(ref, x)
    report("all_to_all", torch.equal(C.all_to_all(x, g), ref))
    if W > 1:
        # push form (TMA bulk stores into the receivers): odd chunk sizes, a chunk smaller than one ring stage, a result
        # that lives in the symmetric heap (no copy out), and back-to-back calls that reuse the receive buffer
        for n_el in (8, 1000, 40 * 1024 + 8, (1 << 20) + 24):
            x = torch.randn(W, n_el, device=dev, dtype=torch.bfloat16, generator=gen)
            ref = torch.empty_like(x)
            dist.all_to_all_single(ref, x)
            ok = torch.equal(C.all_to_all(x, g, algo="push"), ref)
            yh = heap.named(("a2a_push_out", n_el), (W, n_el), torch.bfloat16)
            C.all_to_all(x, g, out=yh.local, algo="push")
            ok &= torch.equal(yh.local, ref)
            x2 = x + 1
            dist.all_to_all_single(ref, x2)
            ok &= torch.equal(C.all_to_all(x2, g, algo="push"), ref)
            report(f"all_to_all push {n_el} elements per chunk", ok)
    # broadcast / scatter / gather / reduce
    x = torch.randn(3000, device=dev, generator=gen)
    ref = x.clone(); dist.broadcast(ref, src=W - 1)
    report("broadcast", torch.equal(C.broadcast(x, g, src=W - 1), ref))
    if heap.mc_base and W > 1:
        xb = torch.randn(1 << 18, device=dev, generator=gen) + r
        refb = xb.clone(); dist.broadcast(refb, src=1)
        okb = torch.equal(C.broadcast(xb, g, src=1, algo="nvls"), refb)
        okb &= torch.equal(C.broadcast(xb + 1, g, src=0, algo="nvls"), (lambda t: (dist.broadcast(t, src=0), t)[1])((xb + 1).clone()))
        report("broadcast through the switch (multimem.st by the root)", okb)
    x = torch.randn(W, 129, device=dev, generator=gen)
    ref = torch.empty(129, device=dev)
    dist.scatter(ref, list(x.unbind(0)) if r == 0 else None, src=0)
    report("scatter", torch.equal(C.scatter(x, g, src=0), ref))
    x = torch.randn(257, device=dev, generator=gen)
    got = C.gather(x, g, dst=0)
    lst = [torch.empty_like(x) for _ in range(W)] if r == 0 else None
    dist.gather(x, lst, dst=0)
    report("gather", torch.equal(got, torch.stack(lst)) if r == 0 else torch.equal(got, x))
    ref = x.clone(); dist.reduce(ref, dst=0)
    got = C.reduce(x, g, dst=0)
    report("reduce", torch.allclose(got, ref, atol=1e-5) if r == 0 else torch.equal(got, x))
    # all_to_all_v with uneven, rank-dependent counts (including a zero)
    counts = torch.tensor([(3 * r + 5 * d) % 7 for d in range(W)], device=dev, dtype=torch.int64)
    counts[(r + 1) % W] = 0 if W > 1 else counts[0]
    rows = int(counts.sum().item())
    x = torch.randn(rows, 24, device=dev, dtype=torch.bfloat16, generator=gen)
    all_counts = torch.empty(W, W, device=dev, dtype=torch.int64)
    dist.all_gather_into_tensor(all_counts, counts)
    recv = all_counts[:, r].tolist()
    ref = torch.empty(sum(recv), 24, device=dev, dtype=torch.bfloat16)
    dist.all_to_all_single(ref, x, output_split_sizes=recv, input_split_sizes=counts.tolist())
    out, rc, total = C.all_to_all_v(x, counts, g, out_capacity_rows=64)
    torch.cuda.synchronize()
    ok = int(total.item()) == sum(recv) and rc.tolist() == recv and torch.equal(out[:sum(recv)], ref)
    report("all_to_all_v", ok)

    # sub-groups: pairs (0,1), (2,3), ... on their own channels
    if W >= 4:
        pair = [r - r % 2, r - r % 2 + 1]
        pgs = [dist.new_group([2 * i, 2 * i + 1]) for i in range(W // 2)]
        sg = None
        for i in range(W // 2):
            gi = heap.group([2 * i, 2 * i + 1])
            if r in (2 * i, 2 * i + 1):
                sg = gi
        x = torch.randn(5000, device=dev, generator=gen)
        ref = x.clone(); dist.all_reduce(ref, group=pgs[r // 2])
        report("all_reduce sub-group", torch.allclose(C.all_reduce(x, sg), ref, atol=1e-5))

    # repeat-run determinism (cheap race detector)
    x = torch.randn(1 << 18, device=dev, dtype=torch.bfloat16, generator=gen)
    first = C.all_reduce(x, g, algo="twoshot").clone()
    same = all(torch.equal(C.all_reduce(x, g, algo="twoshot"), first) for _ in range(20))
    report("all_reduce twoshot determinism x20", same)

    if heap.mc_base and W > 1:
        # in-place form on a heap-resident tensor: the sums replace the inputs on every rank
        for dtype, n in ((torch.bfloat16, 1 << 20), (torch.float32, 123456 // 4 * 4)):
            xs = heap.named(("inplace_x", str(dtype)), (n,), dtype)
            xs.local.copy_(torch.randn(n, device=dev, generator=torch.Generator(device=dev).manual_seed(50 + r)).to(dtype))
            ref = xs.local.clone(); dist.all_reduce(ref)
            torch.cuda.synchronize(); dist.barrier()
            y = C.all_reduce_(xs.local, g)
            torch.cuda.synchronize()
            report(f"all_reduce_ in place {dtype}", torch.allclose(y.float(), ref.float(), atol=2e-2, rtol=2e-2) and y.data_ptr() == xs.local.data_ptr(),
                   f"maxerr={(y.float() - ref.float()).abs().max().item():.3g}")

    if heap.mc_base and W > 1:
        # the switch-side forms of all-gather and reduce-scatter against NCCL
        xa = torch.randn(3 * 4096 + 8, device=dev, dtype=torch.bfloat16, generator=torch.Generator(device=dev).manual_seed(70 + r))
        ref = torch.empty(W * xa.numel(), device=dev, dtype=torch.bfloat16); dist.all_gather_into_tensor(ref, xa)
        report("all_gather nvls", torch.equal(C.all_gather(xa, g, algo="nvls").view(-1), ref))
        for dtype in (torch.bfloat16, torch.float32):
            xr = torch.randn(W * 2048, 8, device=dev, generator=torch.Generator(device=dev).manual_seed(80 + r)).to(dtype)
            ref = torch.empty(2048, 8, device=dev, dtype=dtype); dist.reduce_scatter_tensor(ref, xr)
            got = C.reduce_scatter(xr, g, algo="nvls")
            report(f"reduce_scatter nvls {dtype}", torch.allclose(got.float(), ref.float(), atol=2e-2, rtol=2e-2),
                   f"maxerr={(got.float() - ref.float()).abs().max().item():.3g}")

    # quick timing vs NCCL (device time, max over ranks)
    def timeit(fn, n=30, warm=10):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()
    for nbytes in (4096, 65536, 1 << 20, 1 << 24, 1 << 27):
        x = torch.randn(nbytes // 2, device=dev, dtype=torch.bfloat16)
        y = torch.empty_like(x)
        t_nccl = timeit(lambda: dist.all_reduce(y))
        line = f"PERF all_reduce {nbytes}B nccl={t_nccl * 1e3:.1f}us"
        for algo in ["oneshot", "twoshot"] + (["nvls"] if heap.mc_base else []) + (["ll"] if nbytes <= (1 << 20) and W > 1 else []):
            if algo == "oneshot" and nbytes > (1 << 24):
                continue
            t = timeit(lambda: C.all_reduce(x, g, algo=algo, out=y))
            line += f" {algo}={t * 1e3:.1f}us"
        if heap.mc_base and W > 1:
            xs = heap.named(("perf_inplace", nbytes), (nbytes // 2,), torch.bfloat16)
            xs.local.zero_()
            t = timeit(lambda: C.all_reduce_(xs.local, g))
            line += f" nvls_inplace={t * 1e3:.1f}us (bus {2 * (W - 1) / W * nbytes / t / 1e6:.0f} GB/s; nccl bus {2 * (W - 1) / W * nbytes / t_nccl / 1e6:.0f} GB/s)"
        if r == 0:
            print(line, flush=True)

    for nbytes in (1 << 24, 1 << 27):
        # reduce-scatter and all-to-all of `nbytes` per rank: time and bytes received per rank and direction
        x = torch.randn(nbytes // 2, device=dev, dtype=torch.bfloat16).view(W, -1)
        yr = torch.empty(nbytes // 2 // W, device=dev, dtype=torch.bfloat16)
        t_nccl = timeit(lambda: dist.reduce_scatter_tensor(yr, x.view(-1)))
        t_ours = timeit(lambda: C.reduce_scatter(x.view(W * (x.shape[1] // 8), 8), g, algo="pull"))
        t_nvls = timeit(lambda: C.reduce_scatter(x.view(W * (x.shape[1] // 8), 8), g, algo="nvls")) if heap.mc_base and W > 1 else float("nan")
        ya = torch.empty_like(x)
        t_nccl_a = timeit(lambda: dist.all_to_all_single(ya.view(-1), x.view(-1)))
        t_ours_a = timeit(lambda: C.all_to_all(x, g, out=ya, algo="pull"))
        t_push_a = t_push_h = float("nan")
        if W > 1:
            t_push_a = timeit(lambda: C.all_to_all(x, g, out=ya, algo="push"))
            yah = heap.named(("perf_a2a_out", nbytes), tuple(x.shape), torch.bfloat16)
            t_push_h = timeit(lambda: C.all_to_all(x, g, out=yah.local, algo="push"))
        if r == 0:
            per_dir = (W - 1) / W * nbytes
            print(f"PERF reduce_scatter {nbytes}B nccl={t_nccl * 1e3:.1f}us pull={t_ours * 1e3:.1f}us ({per_dir / t_ours / 1e6:.0f} GB/s per direction) "
                  f"nvls={t_nvls * 1e3:.1f}us ({per_dir / t_nvls / 1e6:.0f} GB/s)", flush=True)
            print(f"PERF all_to_all {nbytes}B nccl={t_nccl_a * 1e3:.1f}us pull={t_ours_a * 1e3:.1f}us ({per_dir / t_ours_a / 1e6:.0f} GB/s per direction) "
                  f"push={t_push_a * 1e3:.1f}us ({per_dir / t_push_a / 1e6:.0f} GB/s) push_into_heap={t_push_h * 1e3:.1f}us ({per_dir / t_push_h / 1e6:.0f} GB/s)", flush=True)

    if heap.mc_base and W > 1:
        for nbytes in (1 << 20, 1 << 27):
            xb = torch.randn(nbytes // 2, device=dev, dtype=torch.bfloat16)
            t_nccl = timeit(lambda: dist.broadcast(xb, src=0))
            t_pull = timeit(lambda: C.broadcast(xb, g, src=0, algo="pull"))
            t_nvls = timeit(lambda: C.broadcast(xb, g, src=0, algo="nvls"))
            if r == 0:
                print(f"PERF broadcast {nbytes}B nccl={t_nccl * 1e3:.1f}us pull={t_pull * 1e3:.1f}us nvls={t_nvls * 1e3:.1f}us", flush=True)

    for nbytes in (1 << 20, 1 << 24, 1 << 27):
        x = torch.randn(nbytes // 2, device=dev, dtype=torch.bfloat16)
        yn = torch.empty(W * (nbytes // 2), device=dev, dtype=torch.bfloat16)
        yo = torch.empty(W, nbytes // 2, device=dev, dtype=torch.bfloat16)
        t_nccl = timeit(lambda: dist.all_gather_into_tensor(yn, x))
        t_ours = timeit(lambda: C.all_gather(x, g, out=yo, algo="pull"))
        line = (f"PERF all_gather {nbytes}B/rank nccl={t_nccl * 1e3:.1f}us pull={t_ours * 1e3:.1f}us "
                f"({(W - 1) * nbytes / t_ours / 1e6:.0f} GB/s in per rank)")
        if heap.mc_base and W > 1:
            t_nvls = timeit(lambda: C.all_gather(x, g, out=yo, algo="nvls"))
            yh = heap.named(("perf_ag_out", nbytes), (W, nbytes // 2), torch.bfloat16)
            t_nvls_h = timeit(lambda: C.all_gather(x, g, out=yh.local, algo="nvls"))
            line += (f" nvls={t_nvls * 1e3:.1f}us ({(W - 1) * nbytes / t_nvls / 1e6:.0f} GB/s) "
                     f"nvls_into_heap={t_nvls_h * 1e3:.1f}us ({(W - 1) * nbytes / t_nvls_h / 1e6:.0f} GB/s)")
        if r == 0:
            print(line, flush=True)

    # the same comparison with both sides replayed from a CUDA graph (launch overhead of either host path removed),
    # inputs and outputs living in the symmetric heap so that no staging copy is involved
    def graph_time(fn, n=20):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(3):
                fn()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize(); dist.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(n):
                fn()
        torch.cuda.synchronize(); dist.barrier()
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            gr.replay()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / (5 * n)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()
    if W > 1 and "--graphs" in sys.argv:
        for nbytes in (4096, 65536, 1 << 20, 1 << 24, 1 << 27):
            xs = heap.named(("perf_x", nbytes), (nbytes // 2,), torch.bfloat16)
            xs.local.normal_()
            y = torch.empty(nbytes // 2, device=dev, dtype=torch.bfloat16)
            yn = xs.local.clone()
            line = f"GRAPH all_reduce {nbytes}B nccl={graph_time(lambda: dist.all_reduce(yn)) * 1e3:.1f}us"
            for algo in ["oneshot", "twoshot"] + (["nvls"] if heap.mc_base else []) + (["ll"] if nbytes <= (1 << 20) else []):
                if algo == "oneshot" and nbytes > (1 << 24):
                    continue
                line += f" {algo}={graph_time(lambda: C.all_reduce(xs.local, g, algo=algo, out=y)) * 1e3:.1f}us"
            if r == 0:
                print(line, flush=True)

    torch.cuda.synchronize()
    st = nv.read_status()
    report("device status clean", st[0] == 0, str(st[:8]))
    tot = torch.tensor([fails], device=dev)
    dist.all_reduce(tot)
    ctx.finalize()
    if r == 0:
        print("TOTAL_FAILS", int(tot.item()), flush=True)
    return 1 if tot.item() else 0


if __name__ == "__main__":
    sys.exit(main())
