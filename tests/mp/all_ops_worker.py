"""Run every registered op (reference and ours) inside ONE process group and compare per rank.

Used on CPU (gloo ranks, shared-memory transport) and on GPUs (NCCL + symmetric heap):
    torchrun --nproc-per-node 2 tests/mp/all_ops_worker.py [--backend gloo] [--dtype float32] [--config small] [--ops a,b]
Prints one PASS/FAIL line per op and ``TOTAL_FAILS n``; exits non-zero on any failure.
"""
import argparse
import os
import sys
import traceback

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from parallelkernelbench_b200.harness import compare  # noqa: E402
from parallelkernelbench_b200.parallel import init_context  # noqa: E402
from parallelkernelbench_b200.workloads import registry  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default=None)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--config", default="small", help="preferred config name; ops without it use 'default'")
    ap.add_argument("--ops", default="all")
    ap.add_argument("--skip", default="")
    ap.add_argument("--trials", type=int, default=1)
    ap.add_argument("--no-oracle", action="store_true", help="skip the fp32 run that loose gates have to be earned against")
    args = ap.parse_args()
    ctx = init_context(backend=args.backend)
    names = [s.name for s in registry.all_ops()] if args.ops == "all" else args.ops.split(",")
    skip = set(filter(None, args.skip.split(",")))
    fails = 0
    for name in names:
        if name in skip:
            continue
        spec = registry.get(name)
        if spec.ours is None or (spec.ours_needs_cuda and not ctx.is_cuda) or (spec.explicit_only and args.ops == "all"):
            continue
        cfg_name = args.config if args.config in spec.configs else "default"
        for trial in range(args.trials):
            ok, detail = False, ""
            try:
                cfg = spec.config(cfg_name)
                rc_ref = registry.RunCtx(ctx, spec.name, trial=trial, dtype=registry.DTYPES[args.dtype])
                rc_ours = registry.RunCtx(ctx, spec.name, trial=trial, dtype=registry.DTYPES[args.dtype])
                with torch.no_grad():
                    a = compare.normalize_output(spec.reference(rc_ref, *spec.make_inputs(rc_ref, cfg)))
                    b = compare.normalize_output(spec.ours(rc_ours, *spec.make_inputs(rc_ours, cfg)))

                def oracle():
                    # the reference code on the same seeded inputs widened to fp32 (collective: every rank calls it or none does)
                    from parallelkernelbench_b200.harness.worker import _widen

                    rc_o = registry.RunCtx(ctx, spec.name, trial=trial, dtype=registry.DTYPES[args.dtype])
                    inputs = _widen(spec.make_inputs(rc_o, cfg))
                    rc_o.dtype = torch.float32
                    with torch.no_grad():
                        return compare.normalize_output(spec.reference(rc_o, *inputs))

                if ctx.is_cuda:
                    torch.cuda.synchronize()
                    from parallelkernelbench_b200 import _native as nv

                    st = nv.read_status()
                    if st[0] != 0:
                        nv.clear_status()
                        raise RuntimeError(f"device status {st[:8]}")
                atol, rtol = spec.tolerance(cfg_name)
                strict = compare.compare_objects(a, b, compare.STRICT_ATOL, compare.STRICT_RTOL)["ok"]
                need = torch.tensor([0 if strict else 1], device=ctx.device)
                if ctx.world > 1:
                    dist.all_reduce(need)          # the fp32 run contains collectives: all ranks make it if any rank needs it
                exact = None
                if need.item() and (atol > compare.STRICT_ATOL or rtol > compare.STRICT_RTOL) and not args.no_oracle:
                    try:
                        exact = oracle()
                    except Exception as e:
                        exact = None
                        print(f"note rank{ctx.rank} {name}: fp32 run unavailable ({type(e).__name__}: {str(e)[:120]})", flush=True)
                res = compare.accuracy_gate(a, b, atol, rtol, oracle=(lambda: exact) if exact is not None else None)
                ok = res["ok"]
                detail = f"gate={res['gate']} max_abs_diff={res.get('max_abs_diff')} " + (f"vs_fp32={res['oracle_err']} " if "oracle_err" in res else "") + "; ".join(res["errors"][:2])
            except Exception as e:
                detail = f"{type(e).__name__}: {e}\n{traceback.format_exc(limit=6)}"
            flag = torch.tensor([0 if ok else 1], device=ctx.device)
            if ctx.world > 1:
                dist.all_reduce(flag)
            if flag.item():
                fails += 1
            if ctx.rank == 0 or not ok:
                print(f"{'PASS' if not flag.item() else 'FAIL'} rank{ctx.rank} {name} [{cfg_name}] trial={trial} {detail}", flush=True)
    ctx.finalize()
    if ctx.rank == 0:
        print("TOTAL_FAILS", fails, flush=True)
    return 1 if fails else 0


if __name__ == "__main__":
    sys.exit(main())
