"""Small, self-terminating cases of the main kernels, meant to be run under a profiler.

    python -m parallelkernelbench_b200.harness.profile_cases <case> [--iters N]

Each case allocates a few hundred MB at most (inputs larger than L2 where DRAM figures matter),
launches the kernel a handful of times and exits, so a capture of one launch ends by itself.
Cases: gemm_pair, gemm_single, tp_mlp, fa_fwd, fa_fwd_d64, grouped_gemm, rmsnorm, allreduce.
"""
from __future__ import annotations

import argparse
import sys

import torch


def case_gemm_pair(iters):
    from ..ops import gemm_bf16

    a = torch.randn(4096, 8192, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16) * 0.02
    out = torch.empty(4096, 8192, device="cuda", dtype=torch.bfloat16)
    for _ in range(iters):
        gemm_bf16(a, w, out=out, mode="pair")


def case_gemm_single(iters):
    from ..ops import gemm_bf16

    a = torch.randn(4096, 8192, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16) * 0.02
    out = torch.empty(4096, 8192, device="cuda", dtype=torch.bfloat16)
    for _ in range(iters):
        gemm_bf16(a, w, out=out, mode="single", block_n=256)


def case_tp_mlp(iters):
    from ..models import TPMLPBlock, TPMLPConfig
    from ..parallel import init_context

    ctx = init_context()
    cfg = TPMLPConfig(rows_per_rank=2048, hidden=8192, ffn=7168)
    w1, w2, gamma = TPMLPBlock.random_weights(cfg, 1, 0, ctx.device)
    blk = TPMLPBlock(ctx.heap().world_group, cfg, w1, w2, gamma)
    x = torch.randn(cfg.rows_per_rank, cfg.hidden, device=ctx.device, dtype=torch.bfloat16)
    for _ in range(iters):
        blk(x)
    torch.cuda.synchronize()
    ctx.finalize()


def _fa(iters, d):
    from ..ops.attention import flash_attn_fwd

    q = torch.randn(1, 4096, 16, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, 4096, 4, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(1, 4096, 4, d, device="cuda", dtype=torch.bfloat16)
    for _ in range(iters):
        flash_attn_fwd(q, k, v, causal=True)


def case_fa_fwd(iters):
    _fa(iters, 128)


def case_fa_fwd_d64(iters):
    _fa(iters, 64)


def case_grouped_gemm(iters):
    from ..ops.moe import grouped_gemm

    counts = torch.full((32,), 512, dtype=torch.int32)
    offs = torch.cat([torch.zeros(1, dtype=torch.int32), counts.cumsum(0).to(torch.int32)]).cuda()
    a = torch.randn(32 * 512, 2048, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(32, 1024, 2048, device="cuda", dtype=torch.bfloat16) * 0.02
    for _ in range(iters):
        grouped_gemm(a, w, offs)


def case_rmsnorm(iters):
    from ..ops import rmsnorm

    x = torch.randn(16384, 8192, device="cuda", dtype=torch.bfloat16)
    g = torch.ones(8192, device="cuda", dtype=torch.bfloat16)
    for _ in range(iters):
        rmsnorm(x, g)


def case_allreduce(iters):
    from ..ops import collectives as C
    from ..parallel import init_context

    ctx = init_context()
    g = ctx.heap().world_group
    x = torch.randn(64 << 20, device=ctx.device, dtype=torch.bfloat16)
    for _ in range(iters):
        C.all_reduce(x, g, algo="twoshot")
    torch.cuda.synchronize()
    ctx.finalize()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args(argv)
    fn = globals().get("case_" + a.case)
    if fn is None:
        print("unknown case", a.case)
        return 2
    fn(a.iters)
    torch.cuda.synchronize()
    from .. import _native as nv

    nv.raise_on_status(sync=True)
    print("ok", a.case)
    return 0


if __name__ == "__main__":
    sys.exit(main())
