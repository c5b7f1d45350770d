"""Small, self-terminating cases of the main kernels, meant to be run under a profiler.

    python -m parallelkernelbench_b200.harness.profile_cases <case> [--iters N]

Each case allocates a few hundred MB at most (inputs larger than L2 where DRAM figures matter),
launches the kernel a handful of times and exits, so a capture of one launch ends by itself.
Cases: gemm_pair, gemm_single, tp_mlp, moe_layer, fa_fwd, fa_fwd_d64, fa_bwd, grouped_gemm, grouped_gemm_fp8, rmsnorm, allreduce,
fsdp_adamw, moe_exchange, gsplat, delta_scan, llama_step, llama_step_8l.
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


def case_grouped_gemm_fp8(iters):
    """The same ragged problem as ``grouped_gemm`` on e4m3 operands with block scales."""
    from ..ops.gemm_fp8 import gemm_fp8_blockscaled
    from ..refs.gemm_fp8 import quantize_rows_1x128, quantize_weight_128x128

    counts = torch.full((32,), 512, dtype=torch.int32)
    offs = torch.cat([torch.zeros(1, dtype=torch.int32), counts.cumsum(0).to(torch.int32)]).cuda()
    a8, sa = quantize_rows_1x128(torch.randn(32 * 512, 2048, device="cuda"))
    w8, sb = quantize_weight_128x128(torch.randn(32, 1024, 2048, device="cuda") * 0.02)
    for _ in range(iters):
        gemm_fp8_blockscaled(a8, sa, w8, sb, offsets=offs)


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


def case_fa_bwd(iters):
    from ..ops.attention import flash_attn_bwd, flash_attn_fwd

    q = torch.randn(1, 4096, 16, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, 4096, 4, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(1, 4096, 4, 128, device="cuda", dtype=torch.bfloat16)
    do = torch.randn(1, 4096, 16, 128, device="cuda", dtype=torch.bfloat16)
    out, lse = flash_attn_fwd(q, k, v, causal=True)
    for _ in range(iters):
        flash_attn_bwd(q, k, v, out, lse, do, causal=True)


def case_fsdp_adamw(iters):
    from ..ops import fp8_quantize_1x128
    from ..ops.quant import fsdp_adamw_fp8

    W, n = 8, 32 << 20
    payload = torch.randint(0, 120, (W, n), device="cuda", dtype=torch.uint8)
    scales = torch.rand(W, n // 128, device="cuda") * 1e-3
    p, m, v = torch.randn(n, device="cuda") * 0.02, torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    q_out, s_out = fp8_quantize_1x128(p.view(-1, 128))
    for i in range(iters):
        fsdp_adamw_fp8(payload, scales, p, m, v, q_out.view(-1), s_out.view(-1), lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                       weight_decay=0.1, grad_scale=1.0 / W, step=i + 1)


def case_moe_exchange(iters):
    """Dispatch and combine kernels at one rank (the pushes and pulls stay on this GPU)."""
    from ..models.moe_layer import EPMoELayer, MoEConfig
    from ..parallel import init_context
    from ..parallel.comm import Comm

    ctx = init_context()
    dev = ctx.device
    cfg = MoEConfig(hidden=2048, inter=512, num_experts=32, top_k=8, tokens_per_rank=4096)
    w_router = torch.randn(32, 2048, device=dev, dtype=torch.bfloat16) * 0.02
    wg = torch.randn(32, 512, 2048, device=dev, dtype=torch.bfloat16) * 0.02
    wu = torch.randn(32, 512, 2048, device=dev, dtype=torch.bfloat16) * 0.02
    wd = torch.randn(32, 2048, 512, device=dev, dtype=torch.bfloat16) * 0.02
    comm = Comm(ctx)
    layer = EPMoELayer(comm.group(), comm, cfg, w_router, wg, wu, wd)
    x = torch.randn(cfg.tokens_per_rank, cfg.hidden, device=dev, dtype=torch.bfloat16)
    for _ in range(iters):
        layer(x)
    torch.cuda.synchronize()
    ctx.finalize()


def case_moe_layer(iters):
    """The whole expert-parallel layer at one rank with the per-rank work of the 8-rank headline configuration: 8192 tokens x
    7168, 32 local experts, top-8 (65536 expert rows of 2048 per expert), fp8 dispatch, bf16 experts; PKB_MOE_FP8_EXPERTS=1
    selects the block-scaled fp8 experts."""
    import os

    from ..models.moe_layer import EPMoELayer, MoEConfig
    from ..parallel import init_context
    from ..parallel.comm import Comm

    ctx = init_context()
    dev = ctx.device
    E, H, I = 32, 7168, 2048
    cfg = MoEConfig(hidden=H, inter=I, num_experts=E, top_k=8, tokens_per_rank=8192, fp8_dispatch=True,
                    fp8_experts=os.environ.get("PKB_MOE_FP8_EXPERTS") == "1")
    w_router = torch.randn(E, H, device=dev, dtype=torch.bfloat16) * 0.02
    wg = torch.randn(E, I, H, device=dev, dtype=torch.bfloat16) * 0.02
    wu = torch.randn(E, I, H, device=dev, dtype=torch.bfloat16) * 0.02
    wd = torch.randn(E, H, I, device=dev, dtype=torch.bfloat16) * 0.02
    comm = Comm(ctx)
    layer = EPMoELayer(comm.group(), comm, cfg, w_router, wg, wu, wd)
    x = torch.randn(cfg.tokens_per_rank, cfg.hidden, device=dev, dtype=torch.bfloat16)
    for _ in range(iters):
        layer(x)
    torch.cuda.synchronize()
    ctx.finalize()


def case_gsplat(iters):
    from ..ops.gsplat import gsplat_project_exchange
    from ..parallel import init_context

    ctx = init_context()
    n = 1 << 20
    dev = ctx.device
    means = torch.stack([(torch.rand(n, device=dev) - 0.5) * 1.5, (torch.rand(n, device=dev) - 0.5) * 1.5, torch.rand(n, device=dev) * 2 + 2], -1)
    view = torch.eye(4, device=dev).reshape(1, 4, 4)
    K = torch.tensor([[800.0, 0, 512], [0, 800.0, 512], [0, 0, 1]], device=dev).reshape(1, 3, 3)
    for _ in range(iters):
        gsplat_project_exchange(ctx.heap().world_group, means, torch.randn(n, 4, device=dev), torch.rand(n, 3, device=dev) * 0.02,
                                torch.rand(n, device=dev), torch.rand(n, 3, device=dev), view, K, 1, 1024, 1024)
    torch.cuda.synchronize()
    ctx.finalize()


def case_delta_scan(iters):
    from ..ops.wild import delta_rule_scan

    BH, T, K, V = 64, 2048, 128, 128
    q, k = torch.randn(BH, T, K, device="cuda") * 0.1, torch.nn.functional.normalize(torch.randn(BH, T, K, device="cuda"), dim=-1)
    v, decay, beta = torch.randn(BH, T, V, device="cuda"), torch.rand(BH, T, K, device="cuda") * 0.1 + 0.9, torch.rand(BH, T, device="cuda")
    for _ in range(iters):
        delta_rule_scan(q, k, v, decay, beta)


def case_llama_step(iters):
    """One decoder layer at Llama-8B width (hidden 4096, ffn 14336, 32/8 heads) with a 16k vocabulary, sequence 4096: the
    launch list of a full training step (gather, forward, backward, fp8 gradient exchange, AdamW) at about 5 GB."""
    from ..models.llama import FSDPLlama, LlamaConfig
    from ..parallel import init_context

    ctx = init_context()
    cfg = LlamaConfig(layers=1, vocab=16384)
    model = FSDPLlama(ctx, cfg, impl="ours")
    g = torch.Generator(device=ctx.device).manual_seed(5)
    tok = torch.randint(0, cfg.vocab, (cfg.seq,), device=ctx.device, generator=g)
    tgt = torch.randint(0, cfg.vocab, (cfg.seq,), device=ctx.device, generator=g)
    for _ in range(iters):
        model.step(tok, tgt)
    torch.cuda.synchronize()
    ctx.finalize()


def case_llama_step_8l(iters):
    """Eight decoder layers at Llama-8B width with the full 128256 vocabulary, sequence 4096: the launch list of a training step
    with the per-layer work and the vocabulary-sized head in realistic proportion (about 30 GB on the device)."""
    from ..models.llama import FSDPLlama, LlamaConfig
    from ..parallel import init_context

    ctx = init_context()
    cfg = LlamaConfig(layers=8)
    model = FSDPLlama(ctx, cfg, impl="ours")
    g = torch.Generator(device=ctx.device).manual_seed(5)
    tok = torch.randint(0, cfg.vocab, (cfg.seq,), device=ctx.device, generator=g)
    tgt = torch.randint(0, cfg.vocab, (cfg.seq,), device=ctx.device, generator=g)
    for _ in range(iters):
        model.step(tok, tgt)
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
