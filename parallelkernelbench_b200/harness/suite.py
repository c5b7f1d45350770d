"""The headline configurations besides the tensor-parallel MLP block, run inside an already initialised job.

``launch headline`` evaluates them as separate torchrun jobs (reference job, our job, file comparison). A benchmark
script that is itself one torchrun job cannot start nested jobs on the GPUs it holds, so this module runs the same
workloads in process: for each configuration the PyTorch + NCCL implementation and ours are built from the registry on the
same seeded inputs, compared on every rank through the accuracy gate, and timed back to back with the same loop
(``harness.timing.measure``: rotated inputs, one CUDA event per iteration, max over ranks).

    from parallelkernelbench_b200.harness import suite
    rows = suite.run(ctx, suite.select("3,4"), warmup=3, iters=10)
"""
from __future__ import annotations

import gc

import torch
import torch.distributed as dist

from . import compare, timing
from .roofline import estimate

# label -> (op, named config)
CONFIGS = {
    "3": ("moe_layer", "deepseek"),                      # fp8 dispatch, bf16 experts
    "3f": ("moe_layer", "deepseek_fp8_experts"),         # fp8 dispatch feeding block-scaled fp8 expert GEMMs
    "4": ("ring_attention_fwd_bwd", "cp131k"),
    "5": ("fsdp_llama_step", "llama8b"),
}


def select(only: str = "") -> list[str]:
    keys = [k.strip() for k in only.split(",") if k.strip()] or list(CONFIGS)
    for k in keys:
        if k not in CONFIGS:
            raise KeyError(f"unknown suite entry {k!r}; known: {sorted(CONFIGS)}")
    return keys


def heap_gib(keys: list[str], world: int) -> float:
    """Symmetric-heap size the selected configurations need (the heap is created once per job)."""
    from ..workloads import registry

    need = 1.0
    for k in keys:
        op, cfg_name = CONFIGS[k]
        spec = registry.get(op)
        if spec.heap_gib is not None:
            need = max(need, float(spec.heap_gib(spec.config(cfg_name), world)))
    return need


def _all_max(ctx, v: float) -> float:
    t = torch.tensor([v], device=ctx.device, dtype=torch.float64)
    if ctx.world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_one(ctx, op: str, cfg_name: str, warmup: int = 3, iters: int = 10, time_reference: bool = True) -> dict:
    from .. import _native as nv
    from ..workloads import registry

    spec = registry.get(op)
    cfg = spec.config(cfg_name)
    atol, rtol = spec.tolerance(cfg_name)
    row: dict = {"op": op, "config": cfg_name, "world": ctx.world, "warmup": warmup, "iters": iters}
    rc_ref = registry.RunCtx(ctx, spec.name, trial=0, dtype=torch.bfloat16)
    rc_ours = registry.RunCtx(ctx, spec.name, trial=0, dtype=torch.bfloat16)
    heap = ctx.heap()
    mark = heap.mark()             # symmetric buffers of this configuration are handed back when it is done
    try:
        with torch.no_grad():
            in_ref = spec.make_inputs(rc_ref, cfg)
            y_ref = compare.normalize_output(spec.reference(rc_ref, *in_ref))
            in_ours = spec.make_inputs(rc_ours, cfg)
            y_ours = compare.normalize_output(spec.ours(rc_ours, *in_ours))
        nv.raise_on_status(sync=True)
        res = compare.accuracy_gate(y_ref, y_ours, atol, rtol)          # no fp32 run here: it would not fit next to both engines
        ok = _all_max(ctx, 0.0 if res["ok"] else 1.0) == 0.0
        row.update({"result": "match" if ok else "tensor_mismatch", "gate": res["gate"], "atol": atol, "rtol": rtol,
                    "max_abs_diff": _all_max(ctx, float(res.get("max_abs_diff") or 0.0))})
        if not ok and ctx.rank == 0:
            row["errors"] = res["errors"][:2]
        del y_ref, y_ours
        with torch.no_grad():
            p_ours = timing.measure(lambda *a: spec.ours(rc_ours, *a), in_ours, warmup=warmup, iters=iters, device=ctx.device)
        nv.raise_on_status(sync=True)
        row["ours_ms"] = _all_max(ctx, p_ours["wall_time_ms"])
        if time_reference:
            with torch.no_grad():
                p_ref = timing.measure(lambda *a: spec.reference(rc_ref, *a), in_ref, warmup=warmup, iters=iters, device=ctx.device)
            row["ref_ms"] = _all_max(ctx, p_ref["wall_time_ms"])
            row["speedup"] = row["ref_ms"] / row["ours_ms"]
        if spec.cost is not None:
            est = estimate(spec.cost(cfg, ctx.world), row["ours_ms"])
            row.update({"pct_of_roofline": est.get("pct_of_roofline"), "limiter": est.get("limiter"), "roofline_ms": est.get("roofline_ms")})
    except Exception as e:                                              # one configuration failing must not lose the others
        row.update({"result": "error", "error": f"{type(e).__name__}: {e}"[:400]})
        try:
            nv.clear_status()
        except Exception:
            pass
    finally:
        rc_ref.cache.clear()
        rc_ours.cache.clear()
        gc.collect()
        if ctx.is_cuda:
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
        ctx.barrier()              # no rank may reuse the space while a peer's kernels can still write into it
        heap.release(mark)
    return row


def run(ctx, keys: list[str], warmup: int = 3, iters: int = 10) -> list[dict]:
    rows = []
    for k in keys:
        op, cfg_name = CONFIGS[k]
        row = run_one(ctx, op, cfg_name, warmup=warmup, iters=iters)
        row["label"] = k
        rows.append(row)
        ctx.barrier()
    return rows
