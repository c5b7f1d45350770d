"""Per-rank worker, started once per GPU (or CPU rank) by torchrun.

Flow: bind the rank, create the process group -> build the op's seeded inputs -> run the chosen
implementation once -> synchronise and barrier -> save ``rank_<r>.pt`` -> optionally time it
(500 warm-up / 100 timed by default) into ``rank_<r>_perf.json`` -> optionally record a
torch-profiler trace -> tear the group down in ``finally``. The native library is prebuilt, so no
rank compiles anything (the reference JIT-compiles per rank and isolates extension caches to
avoid races: reference: scripts/worker.py:49-55,118-237).

    torchrun --nproc-per-node N -m parallelkernelbench_b200.harness.worker --op allreduce \
        --impl ours --logs-dir DIR [--config default] [--set m=2048] [--dtype bfloat16] [--trial 0] \
        [--measure-perf --warmup 500 --iters 100 --graph] [--profile] [--backend gloo]
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import traceback

import torch
import torch.distributed as dist


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", required=True)
    ap.add_argument("--impl", required=True, choices=["reference", "ours", "file", "oracle"])
    ap.add_argument("--solution", default=None, help="with --impl file: a Python file that defines solution(rc, *inputs)")
    ap.add_argument("--logs-dir", required=True)
    ap.add_argument("--config", default="default")
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--trial", type=int, default=0)
    ap.add_argument("--backend", default=None, choices=[None, "nccl", "gloo"])
    ap.add_argument("--measure-perf", action="store_true")
    ap.add_argument("--warmup", type=int, default=500)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--graph", action="store_true", help="time CUDA-graph replays of the op")
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--determinism", type=int, default=0, metavar="N",
                    help="run the implementation N more times on identical inputs and require bit-identical outputs (a cheap race detector)")
    ap.add_argument("--fail-rank", type=int, default=-1, help="test hook: this rank raises before the first collective")
    ap.add_argument("--exit-rank", type=int, default=-1, help="test hook: this rank exits non-zero before the first collective")
    return ap.parse_args(argv)


def load_solution(path: str):
    """Import a candidate implementation from a file: it must define ``solution(rc, *inputs)`` with the same inputs and
    outputs as the op's reference (``rc`` is the :class:`RunCtx`: rank, world, device, ``rc.comm`` for the symmetric-heap
    collectives). Same role as the solution loader of the reference's worker (reference: scripts/worker.py:109-115)."""
    import importlib.util

    if not path or not os.path.isfile(path):
        raise FileNotFoundError(f"solution file not found: {path!r}")
    spec = importlib.util.spec_from_file_location("pkb_candidate_solution", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    fn = getattr(mod, "solution", None)
    if not callable(fn):
        raise AttributeError(f"{path} does not define a callable `solution(rc, *inputs)`")
    return fn


def _bit_identical(a, b) -> bool:
    """Recursive bitwise comparison of outputs (tensors, tuples / lists, dicts, plain values); NaNs compare by their bits."""
    import torch

    if isinstance(a, torch.Tensor):
        if not isinstance(b, torch.Tensor) or a.shape != b.shape or a.dtype != b.dtype:
            return False
        if a.numel() == 0:
            return True
        ab, bb = a.detach().contiguous().cpu(), b.detach().contiguous().cpu()
        return bool(torch.equal(ab.view(torch.uint8).reshape(-1) if ab.dtype != torch.bool else ab,
                                bb.view(torch.uint8).reshape(-1) if bb.dtype != torch.bool else bb))
    if isinstance(a, (tuple, list)):
        return isinstance(b, (tuple, list)) and len(a) == len(b) and all(_bit_identical(x, y) for x, y in zip(a, b))
    if isinstance(a, dict):
        return isinstance(b, dict) and a.keys() == b.keys() and all(_bit_identical(a[k], b[k]) for k in a)
    return a == b


def _widen(x):
    """bf16 / fp16 tensors -> fp32, containers walked, everything else untouched."""
    if isinstance(x, torch.Tensor):
        return x.float() if x.dtype in (torch.bfloat16, torch.float16) else x
    if isinstance(x, (tuple, list)):
        return type(x)(_widen(v) for v in x)
    if isinstance(x, dict):
        return {k: _widen(v) for k, v in x.items()}
    return x


def _check_guards(ctx) -> None:
    """PKB_HEAP_GUARD=1: raise if any guard band around a symmetric-heap allocation was overwritten."""
    heap = getattr(ctx, "_heap", None)
    if heap is not None and hasattr(heap, "check_guards"):
        heap.check_guards()


def run_worker(args) -> int:
    from ..parallel import init_context
    from ..workloads import registry
    from . import compare, timing
    from .roofline import estimate

    if "RANK" not in os.environ and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        print("worker must be started by torchrun", file=sys.stderr)
        return 2
    rank_env = int(os.environ.get("RANK", "0"))
    if args.fail_rank == rank_env:
        raise RuntimeError(f"injected failure on rank {rank_env} (test hook)")
    if args.exit_rank == rank_env:
        return 3
    ctx = init_context(backend=args.backend, timeout_s=float(os.environ.get("PKB_PG_TIMEOUT_SEC", "600")))
    rc = 0
    try:
        spec = registry.get(args.op)
        cfg = spec.config(args.config, registry.parse_overrides(args.set))
        dtype = registry.DTYPES[args.dtype]
        if spec.heap_gib is not None:       # the heap is created on first use: an op with large exchange buffers sizes it
            need = float(spec.heap_gib(cfg, ctx.world))
            if need > float(os.environ.get("PKB_HEAP_GIB", "1")):
                os.environ["PKB_HEAP_GIB"] = str(need)
        run = registry.RunCtx(ctx, spec.name, trial=args.trial, dtype=dtype)
        if args.impl == "file":
            impl = load_solution(args.solution)
        else:
            impl = spec.reference if args.impl in ("reference", "oracle") else spec.ours
        if impl is None:
            raise NotImplementedError(f"op {spec.name} has no '{args.impl}' implementation")
        if args.impl == "ours" and spec.ours_needs_cuda and not ctx.is_cuda:
            raise RuntimeError(f"op {spec.name}: our implementation is a CUDA kernel and needs a GPU")
        print(f"[Rank {ctx.rank}/{ctx.world}] {spec.name} impl={args.impl} cfg={cfg} dtype={args.dtype} "
              f"device={ctx.device} backend={ctx.backend}", flush=True)
        inputs = spec.make_inputs(run, cfg)
        if args.impl == "oracle":
            # the same seeded values as every other implementation sees, widened to fp32, through the reference code: an
            # accuracy yardstick for gates looser than 1e-2 (how far is each implementation from the fp32 result?)
            inputs = _widen(inputs)
            run.dtype = torch.float32
        with torch.no_grad():
            y = impl(run, *inputs)
        uses_native = ctx.is_cuda and args.impl in ("ours", "file")     # a candidate file may call the package's kernels too
        if uses_native:
            from .. import _native as nv
        if ctx.is_cuda:
            torch.cuda.synchronize()
            if uses_native:
                nv.raise_on_status(sync=False)
        ctx.barrier()
        _check_guards(ctx)                # a write outside a symmetric allocation fails the job before anything is saved
        compare.save_output(y, args.logs_dir, ctx.rank)

        if args.determinism > 0:
            # same seeded inputs, same implementation, N more runs: any differing bit is a race (or an atomic-order dependence)
            differing = 0
            for _ in range(args.determinism):
                again_inputs = spec.make_inputs(run, cfg) if spec.mutates_inputs else inputs
                with torch.no_grad():
                    y2 = impl(run, *again_inputs)
                if ctx.is_cuda:
                    torch.cuda.synchronize()
                differing += 0 if _bit_identical(compare.normalize_output(y), compare.normalize_output(y2)) else 1
                ctx.barrier()
            with open(os.path.join(args.logs_dir, f"rank_{ctx.rank}_determinism.json"), "w") as fh:
                json.dump({"runs": args.determinism, "differing": differing}, fh)
            print(f"[Rank {ctx.rank}] determinism: {args.determinism - differing}/{args.determinism} repeat runs bit-identical", flush=True)
            if differing:
                rc = 4

        if args.measure_perf:
            sampler = None
            if ctx.is_cuda and getattr(ctx, "local_rank", ctx.rank) == 0:
                # clocks and throttle reasons of the first GPU while it is being timed (read-only nvidia-smi query; one sampler per
                # job, not one per rank, so the query itself stays out of the measurement)
                try:
                    from ..utils.clocks import ClockSampler

                    sampler = ClockSampler(device=ctx.device, period_ms=100).start()
                except Exception:
                    sampler = None
            with torch.no_grad():
                perf = timing.measure(lambda *a: impl(run, *a), inputs, warmup=args.warmup, iters=args.iters,
                                      device=ctx.device, use_graph=args.graph)
            if uses_native:
                nv.raise_on_status(sync=True)      # a device wait that ran out inside the timed loop invalidates the time
            if sampler is not None:
                try:
                    sampler.stop()
                    perf["clocks"] = sampler.summary()
                except Exception:
                    perf["clocks"] = None
            from ..utils import env as _env

            perf["git_sha"] = _env.git_sha()
            if spec.cost is not None:
                perf.update(estimate(spec.cost(cfg, ctx.world), perf["wall_time_ms"]))
            perf.update({"op": spec.name, "impl": args.impl, "world": ctx.world, "rank": ctx.rank, "config": cfg,
                         "dtype": args.dtype})
            with open(os.path.join(args.logs_dir, f"rank_{ctx.rank}_perf.json"), "w") as fh:
                json.dump(perf, fh)
            print(f"[Rank {ctx.rank}] {perf['wall_time_ms']:.4f} +- {perf['wall_time_std_ms']:.4f} ms "
                  f"(min {perf['min_time_ms']:.4f}, {perf['iterations']} iters after {perf['warmup_iterations']} warm-up)",
                  flush=True)

        _check_guards(ctx)                # again after the repeat runs and the timed loop

        if args.profile and ctx.is_cuda:
            from torch.profiler import ProfilerActivity, profile

            os.makedirs(os.path.join(args.logs_dir, "traces"), exist_ok=True)
            with torch.no_grad():
                for _ in range(3):
                    impl(run, *inputs)
                torch.cuda.synchronize()
                with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], record_shapes=True) as prof:
                    for _ in range(10):
                        with torch.cuda.nvtx.range(f"{spec.name}:{args.impl}"):
                            impl(run, *inputs)
                    torch.cuda.synchronize()
            prof.export_chrome_trace(os.path.join(args.logs_dir, "traces", f"rank_{ctx.rank}.json"))
    except Exception:
        rc = 1
        traceback.print_exc()
        err = os.environ.get("TORCHELASTIC_ERROR_FILE")
        if err:
            try:
                with open(err + f".rank{ctx.rank}", "w") as fh:
                    fh.write(traceback.format_exc())
            except OSError:
                pass
    finally:
        ctx.finalize()
    return rc


def main(argv=None) -> int:
    return run_worker(parse_args(argv))


if __name__ == "__main__":
    sys.exit(main())
