"""Measure the all-reduce algorithms over message sizes and write the selection table.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m parallelkernelbench_b200.tuning.tune --out tuning.json [--merge parallelkernelbench_b200/tuning/collectives_b200.json]

Every (algorithm, size) is timed on the device as the max over ranks (CUDA events around ``iters`` calls after ``warmup``
calls; inputs rotate through enough buffers to exceed L2). The row for this world size replaces the one in ``--merge``
(or in the packaged table), the other rows are kept.
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", required=True)
    ap.add_argument("--merge", default=None)
    ap.add_argument("--min-bytes", type=int, default=4096)
    ap.add_argument("--max-bytes", type=int, default=128 << 20)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=50)
    a = ap.parse_args(argv)

    import torch
    import torch.distributed as dist

    from ..ops import collectives as C
    from ..parallel import init_context
    from . import DEFAULT_FILE, thresholds_from_timings

    ctx = init_context()
    group = ctx.heap().world_group
    W = ctx.world
    if W < 2:
        print("tuning needs at least two ranks", file=sys.stderr)
        return 2
    sizes, s = [], a.min_bytes
    while s <= a.max_bytes:
        sizes.append(s)
        s *= 4
    timings: dict[str, dict[int, float]] = {}
    for algo in ("ll", "oneshot", "twoshot", "nvls"):
        for nbytes in sizes:
            if algo == "ll" and nbytes > C.LL_MAX_BYTES:
                continue
            if algo == "oneshot" and nbytes > (64 << 20):
                continue
            if algo == "nvls" and not group.heap.mc_base:
                continue
            n = nbytes // 2
            nbuf = max(2, min(16, (256 << 20) // nbytes))
            xs = [torch.randn(n, device=ctx.device, dtype=torch.bfloat16) for _ in range(nbuf)]
            out = torch.empty_like(xs[0])
            for i in range(a.warmup):
                C.all_reduce(xs[i % nbuf], group, out=out, algo=algo)
            torch.cuda.synchronize()
            ctx.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(a.iters):
                C.all_reduce(xs[i % nbuf], group, out=out, algo=algo)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) * 1e3 / a.iters], device=ctx.device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            timings.setdefault(algo, {})[nbytes] = float(t.item())
            del xs, out
    if ctx.rank == 0:
        with open(a.merge or DEFAULT_FILE) as fh:
            table = json.load(fh)
        table.setdefault("all_reduce", {})[str(W)] = thresholds_from_timings(timings)
        table.setdefault("measurements_us", {})[str(W)] = {al: {str(k): round(v, 2) for k, v in t.items()} for al, t in timings.items()}
        with open(a.out, "w") as fh:
            json.dump(table, fh, indent=2)
        print(json.dumps(table["all_reduce"][str(W)]))
    ctx.finalize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
