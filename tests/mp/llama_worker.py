"""Per-rank body of the FSDP Llama test: a small decoder trained for a few steps with our kernels and
with the PyTorch+NCCL implementation from the same initial weights; losses must track each other."""
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from parallelkernelbench_b200 import _native as nv  # noqa: E402
from parallelkernelbench_b200.models.llama import FSDPLlama, LlamaConfig  # noqa: E402
from parallelkernelbench_b200.parallel import init_context  # noqa: E402


def main() -> int:
    full = "--full" in sys.argv
    os.environ.setdefault("PKB_HEAP_GIB", "8" if full else "1")
    ctx = init_context()
    W, r, dev = ctx.world, ctx.rank, ctx.device
    if full:
        cfg = LlamaConfig()
        steps = 3
    else:
        cfg = LlamaConfig(layers=2, hidden=512, ffn=1024, heads=4, kv_heads=2, vocab=1024 * max(W, 1), seq=256)
        steps = 4
    g = torch.Generator(device=dev).manual_seed(99 + r)
    toks = [torch.randint(0, cfg.vocab, (cfg.seq,), device=dev, generator=g) for _ in range(steps)]
    tgts = [torch.randint(0, cfg.vocab, (cfg.seq,), device=dev, generator=g) for _ in range(steps)]
    losses, times = {}, {}
    impls = ["ours"] if full and "--ours-only" in sys.argv else ["ours", "torch"]
    for impl in impls:
        model = FSDPLlama(ctx, cfg, impl=impl)
        ls, ts = [], []
        for i in range(steps):
            torch.cuda.synchronize()
            if W > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            loss = model.step(toks[i], tgts[i])
            e1.record()
            torch.cuda.synchronize()
            ls.append(float(loss)); ts.append(e0.elapsed_time(e1))
        losses[impl], times[impl] = ls, ts
        if r == 0:
            print(f"{impl}: losses {['%.4f' % x for x in ls]} ms/step {['%.1f' % t for t in ts]} peak memory {torch.cuda.max_memory_allocated() / 2**30:.1f} GiB", flush=True)
        del model
        import gc
        gc.collect()                      # the engine and its units reference each other
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
    fails = 0
    if "--resume-check" in sys.argv and not full:
        # train 2 steps, save the shards, train 2 more; a fresh engine restored from the shards must repeat those 2 steps
        import shutil
        import tempfile

        ckpt = os.path.join(tempfile.gettempdir(), f"pkb_llama_ckpt_{os.environ.get('MASTER_PORT', '0')}")
        a = FSDPLlama(ctx, cfg, impl="ours")
        for i in range(2):
            a.step(toks[i], tgts[i])
        a.save_sharded(ckpt)
        la = [float(a.step(toks[i], tgts[i])) for i in range(2, 4)]
        b = FSDPLlama(ctx, cfg, impl="ours")
        restored = b.load_sharded(ckpt)
        lb = [float(b.step(toks[i], tgts[i])) for i in range(2, 4)]
        same = restored == 2 and all(abs(x - y) <= 1e-3 * abs(x) for x, y in zip(la, lb))      # dQ sums use atomics: last bits may differ
        same = same and torch.allclose(a.units[0].master, b.units[0].master, rtol=1e-3, atol=1e-5) and a.steps == b.steps == 4
        if r == 0:
            print(f"resume: continued {['%.5f' % x for x in la]} restored {['%.5f' % x for x in lb]} -> {'same' if same else 'DIFFERENT'}", flush=True)
        fails += 0 if same else 1
        torch.cuda.synchronize()
        if W > 1:
            dist.barrier()
        if r == 0:
            shutil.rmtree(ckpt, ignore_errors=True)
        del a, b
    st = nv.read_status()
    if st[0] != 0:
        fails += 1
    if len(impls) == 2:
        for a, b in zip(losses["ours"], losses["torch"]):
            if abs(a - b) > 0.05 * abs(b) + 0.05:
                fails += 1
    import math
    if any(math.isnan(x) for x in losses["ours"]):
        fails += 1
    tot = torch.tensor([fails], device=dev)
    if W > 1:
        dist.all_reduce(tot)
    ctx.finalize()
    if r == 0:
        print("status", st[:6]); print("TOTAL_FAILS", int(tot.item()), flush=True)
    return 1 if tot.item() else 0


if __name__ == "__main__":
    sys.exit(main())
