"""The fused tensor-parallel MLP block on N GPUs of one node, through the public API.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        examples/tp_mlp_block.py [--rows 2048 --hidden 8192 --ffn 28672 --steps 20]

Each rank holds ``rows`` activation rows and 1/N of the two weight matrices; one forward is two launches
(all-gather fused into GEMM1 + SiLU, then GEMM2 with the reduce-scatter in its epilogue and RMSNorm in its consumer phase).
The script checks the result of the first step against the PyTorch + NCCL implementation of the same block, then times the
block with CUDA events (maximum over ranks). ``bench.py`` at the repository root is the full benchmark of this block.
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from parallelkernelbench_b200 import _native as nv  # noqa: E402
from parallelkernelbench_b200.models import TPMLPBlock, TPMLPConfig  # noqa: E402
from parallelkernelbench_b200.parallel import init_context  # noqa: E402
from parallelkernelbench_b200.refs.tp_mlp import TPMLPReference  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=2048, help="activation rows per rank (a multiple of 256)")
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672, help="total intermediate size, split over the ranks")
    ap.add_argument("--steps", type=int, default=20)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        print("this example needs CUDA devices", file=sys.stderr)
        return 2
    os.environ.setdefault("PKB_HEAP_GIB", "1")             # symmetric heap per rank: gather buffer + receive slots
    ctx = init_context()                                    # RANK / WORLD_SIZE / MASTER_* from the environment (one rank also works)
    try:
        cfg = TPMLPConfig(rows_per_rank=args.rows, hidden=args.hidden, ffn=args.ffn)
        w1, w2, gamma = TPMLPBlock.random_weights(cfg, ctx.world, ctx.rank, ctx.device)
        block = TPMLPBlock(ctx.heap().world_group, cfg, w1, w2, gamma)
        x = torch.randn(cfg.rows_per_rank, cfg.hidden, device=ctx.device, dtype=torch.bfloat16)
        y = block(x)
        want = TPMLPReference(ctx.world, cfg.rows_per_rank, cfg.hidden, w1, w2, gamma, cfg.eps)(x)
        err = (y.float() - want.float()).abs().max()
        if ctx.world > 1:
            dist.all_reduce(err, op=dist.ReduceOp.MAX)
        for _ in range(3):
            block(x)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if ctx.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0.record()
        for _ in range(args.steps):
            block(x)
        t1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([t0.elapsed_time(t1) / args.steps], device=ctx.device)
        if ctx.world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        nv.raise_on_status(sync=True)                       # a device-side wait that ran out would be reported here
        if ctx.rank == 0:
            flops = 4.0 * ctx.world * cfg.rows_per_rank * cfg.hidden * cfg.ffn_local(ctx.world)
            print(f"ranks {ctx.world}: {ms.item():.3f} ms per block, {flops / ms.item() / 1e9:.0f} TFLOP/s per GPU, "
                  f"{ctx.world * cfg.rows_per_rank / ms.item() * 1e3:.0f} rows/s, max |error| against PyTorch + NCCL {err.item():.4f}")
        return 0
    finally:
        ctx.finalize()


if __name__ == "__main__":
    sys.exit(main())
