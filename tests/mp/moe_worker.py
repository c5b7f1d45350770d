"""Per-rank body of the MoE tests: grouped GEMM vs per-expert matmuls, then the layer vs the reference."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from parallelkernelbench_b200 import _native as nv  # noqa: E402
from parallelkernelbench_b200.harness import compare  # noqa: E402
from parallelkernelbench_b200.ops.moe import grouped_gemm, interleave_gate_up  # noqa: E402
from parallelkernelbench_b200.parallel import init_context  # noqa: E402
from parallelkernelbench_b200.workloads import registry  # noqa: E402


def main() -> int:
    os.environ.setdefault("PKB_HEAP_GIB", "6" if "--deepseek" in sys.argv else "1")
    ctx = init_context()
    W, r, dev = ctx.world, ctx.rank, ctx.device
    fails = 0

    def report(name, ok, extra=""):
        nonlocal fails
        fails += 0 if ok else 1
        if r == 0 or not ok:
            print(f"{'PASS' if ok else 'FAIL'} rank{r} {name} {extra}", flush=True)

    # grouped GEMM: ragged groups incl. an empty one and a non-multiple-of-128 one
    g = torch.Generator(device=dev).manual_seed(3 + r)
    for (counts, N, K) in [([5, 0, 300, 128, 77], 256, 128), ([1000, 17, 0, 0, 650, 129, 3, 255], 384, 512)]:
        G = len(counts)
        offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=dev)
        rows = int(offs[-1])
        a = torch.randn(rows + 64, K, device=dev, dtype=torch.bfloat16, generator=g)
        w = torch.randn(G, N, K, device=dev, dtype=torch.bfloat16, generator=g) * 0.05
        out = torch.full((rows + 64, N), 7.0, device=dev, dtype=torch.bfloat16)
        grouped_gemm(a, w, offs, out=out)
        ref = torch.full_like(out, 7.0).float()
        for e in range(G):
            ref[offs[e]:offs[e + 1]] = a[offs[e]:offs[e + 1]].float() @ w[e].float().t()
        report(f"grouped_gemm counts={counts}", torch.allclose(out.float(), ref, atol=3e-2, rtol=2e-2),
               f"maxerr={(out.float() - ref).abs().max().item():.3g}")
        wg, wu = w[:, :N // 2].contiguous(), w[:, N // 2:].contiguous()
        out2 = grouped_gemm(a, interleave_gate_up(wg, wu), offs, epilogue="swiglu")
        ref2 = torch.zeros(rows + 64, N // 2, device=dev)
        for e in range(G):
            seg = a[offs[e]:offs[e + 1]].float()
            ref2[offs[e]:offs[e + 1]] = torch.nn.functional.silu(seg @ wg[e].float().t()) * (seg @ wu[e].float().t())
        report("grouped_gemm swiglu", torch.allclose(out2[:rows].float(), ref2[:rows], atol=3e-2, rtol=3e-2),
               f"maxerr={(out2[:rows].float() - ref2[:rows]).abs().max().item():.3g}")

    spec = registry.get("moe_layer")
    cfgs = ["small", "default", "fp8", "balanced", "wide", "lora"] + (["narrow"] if W >= 2 else [])
    if "--deepseek" in sys.argv:
        cfgs = ["deepseek"]
    for cname in cfgs:
        cfg = spec.config(cname)
        try:
            rc1 = registry.RunCtx(ctx, spec.name, trial=0, dtype=torch.bfloat16)
            rc2 = registry.RunCtx(ctx, spec.name, trial=0, dtype=torch.bfloat16)
            inp = spec.make_inputs(rc2, cfg)
            with torch.no_grad():
                ref = spec.reference(rc1, *spec.make_inputs(rc1, cfg))
                out = spec.ours(rc2, *inp)
                torch.cuda.synchronize()
                st = nv.read_status()
                res = compare.compare_objects(ref.cpu(), out.cpu(), spec.atol, spec.rtol)
                ov = int(rc2.cache[next(k for k in rc2.cache if k[0] == "moe_layer")].ex.overflow.item())
                report(f"moe_layer[{cname}]", res["ok"] and st[0] == 0 and ov == 0,
                       f"max_abs_diff={res.get('max_abs_diff'):.4g} overflow={ov} status={st[:4]} {'; '.join(res['errors'][:1])}")
                # determinism and timing

                def timeit(fn, n=10, warm=3):
                    for _ in range(warm):
                        fn()
                    torch.cuda.synchronize()
                    if W > 1:
                        dist.barrier()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(n):
                        fn()
                    e1.record(); torch.cuda.synchronize()
                    t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
                    if W > 1:
                        dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    return t.item()
                t_ours = timeit(lambda: spec.ours(rc2, *inp))
                t_ref = timeit(lambda: spec.reference(rc1, *inp))
                if r == 0:
                    print(f"PERF moe_layer[{cname}] W={W}: ours {t_ours:.3f} ms ref {t_ref:.3f} ms speedup {t_ref / t_ours:.2f}x", flush=True)
            del rc1, rc2
        except Exception as e:
            import traceback
            report(f"moe_layer[{cname}]", False, f"{type(e).__name__}: {e}\n{traceback.format_exc(limit=5)}")
    tot = torch.tensor([fails], device=dev)
    if W > 1:
        dist.all_reduce(tot)
    ctx.finalize()
    if r == 0:
        print("TOTAL_FAILS", int(tot.item()), flush=True)
    return 1 if tot.item() else 0


if __name__ == "__main__":
    sys.exit(main())
