"""The FSDP Llama training step as a workload of the registry.

One call = one optimiser step of the sharded decoder (parameter all-gather, forward, backward, gradient exchange, AdamW,
vocabulary-parallel cross-entropy) on this rank's token block; the output is the loss. "ours" runs the engine on this package's
kernels (fp8 parameter gather, fp8 gradient exchange fused with AdamW, tcgen05 GEMMs, flash attention), the reference runs
the same engine on PyTorch + NCCL + cuBLAS + library attention from the same initial weights. Its ancestors among the
reference problems are the FSDP step and its fp8 pieces (reference: reference/47_fsdp_step_e2e.py:37-65,
reference/52_fp8_reducescatter_delayed_scaling.py:38, reference/53_fp8_allgather_delayed_scaling.py:37,
reference/73_vocab_parallel_cross_entropy_loss.py:21-42).

The engine keeps its state between calls, so repeated calls (the timing loop) keep training; the first call of a job is step
one from the seeded initial weights in both implementations, which is what the comparison sees.
"""
from __future__ import annotations

import torch

from ..harness.roofline import Cost
from .registry import OpSpec, RunCtx, register

_KEYS = ("layers", "hidden", "ffn", "heads", "kv_heads", "vocab", "seq")


def _inputs(rc: RunCtx, cfg):
    vocab = cfg["vocab"] // max(rc.world, 1) * max(rc.world, 1)      # the head is sharded over the ranks
    shape = tuple(int(cfg[k]) if k != "vocab" else vocab for k in _KEYS)
    tok = rc.randint(0, vocab, (cfg["seq"],), salt=1)
    tgt = rc.randint(0, vocab, (cfg["seq"],), salt=2)
    return (tok, tgt, shape)


def _engine(rc: RunCtx, shape, impl: str):
    key = ("fsdp_llama", shape, impl)
    if key not in rc.cache:
        from ..models.llama import FSDPLlama, LlamaConfig

        rc.cache[key] = FSDPLlama(rc.dist, LlamaConfig(**dict(zip(_KEYS, shape))), impl=impl)
    return rc.cache[key]


def _step(impl: str):
    def run(rc, tok, tgt, shape):
        with torch.enable_grad():                                    # the harness calls implementations under no_grad
            return _engine(rc, shape, impl).step(tok, tgt).reshape(1).float()
    return run


def _cost(cfg, W):
    d, f, L, V, S = cfg["hidden"], cfg["ffn"], cfg["layers"], cfg["vocab"], cfg["seq"]
    hd = d // cfg["heads"]
    per_layer = (cfg["heads"] + 2 * cfg["kv_heads"]) * hd * d + d * d + 3 * d * f
    params = L * per_layer
    flops = 6.0 * S * (params + V * d) + 3.5 * 4.0 * S * S * d * L / 2          # GEMMs fwd+bwd, causal attention fwd+bwd
    # fp8 parameter gather + fp8 gradient exchange: one byte per parameter each way, (W-1)/W of it over NVLink
    return Cost(flops=flops, nvlink_bytes=2.0 * params * (W - 1) / max(W, 1), hbm_bytes=30.0 * params / max(W, 1))


register(OpSpec(name="fsdp_llama_step", problem_ids=(), group="optim",
                configs={"default": {"layers": 2, "hidden": 512, "ffn": 1024, "heads": 4, "kv_heads": 2, "vocab": 8192, "seq": 256},
                         "small": {"layers": 1, "hidden": 128, "ffn": 256, "heads": 2, "kv_heads": 1, "vocab": 1024, "seq": 64},
                         "llama8b": {"layers": 32, "hidden": 4096, "ffn": 14336, "heads": 32, "kv_heads": 8, "vocab": 128256, "seq": 4096}},
                make_inputs=_inputs, reference=_step("torch"), ours=_step("ours"), atol=1e-1, rtol=2e-2, cost=_cost,
                ours_needs_cuda=True, explicit_only=True,
                heap_gib=lambda cfg, W: 8.0 if cfg["hidden"] >= 4096 else 1.0,
                doc="one optimiser step of the FSDP-sharded Llama decoder; output = the loss"))
