"""Attention workloads: single-device flash attention and context-parallel (ring) attention.

Reference workloads covered: reference/54_ring_attention.py (forward over a context-parallel group),
and the local attention inside reference/39_ulysses_attention_e2e.py / reference/77_magi1_cso_async_attention.py.
"""
from __future__ import annotations

import math

import torch

from ..harness.roofline import Cost
from ..refs.attention import attention_positions_ref, cp_attention_reference
from .registry import OpSpec, RunCtx, register


# ---- single-device flash attention ---------------------------------------------------------------
def _fa_inputs(rc, cfg):
    B, S, Hq, Hkv, D = cfg["b"], cfg["s"], cfg["hq"], cfg["hkv"], cfg["d"]
    return (rc.randn(B, S, Hq, D), rc.randn(B, S, Hkv, D, salt=1), rc.randn(B, S, Hkv, D, salt=2), bool(cfg["causal"]))


def _fa_ref(rc, q, k, v, causal):
    pos = torch.arange(q.shape[1], device=q.device)
    outs = [attention_positions_ref(q[b], k[b], v[b], pos, pos, causal, 1.0 / math.sqrt(q.shape[-1]))[0] for b in range(q.shape[0])]
    return torch.stack(outs).to(q.dtype)


def _fa_ours(rc, q, k, v, causal):
    from ..ops.attention import flash_attn_fwd

    return flash_attn_fwd(q, k, v, causal=causal)[0]


register(OpSpec(name="flash_attention", problem_ids=(), group="attention",
                configs={"default": {"b": 2, "s": 1024, "hq": 8, "hkv": 2, "d": 128, "causal": 1},
                         "small": {"b": 1, "s": 256, "hq": 4, "hkv": 2, "d": 64, "causal": 1},
                         "long": {"b": 1, "s": 16384, "hq": 32, "hkv": 8, "d": 128, "causal": 1}},
                make_inputs=_fa_inputs, reference=_fa_ref, ours=_fa_ours, atol=2e-2, rtol=2e-2, ours_needs_cuda=True,
                cost=lambda cfg, W: Cost(flops=4.0 * cfg["b"] * cfg["s"] ** 2 * cfg["d"] * cfg["hq"] * (0.5 if cfg["causal"] else 1.0))))


# ---- context-parallel attention -------------------------------------------------------------------
def _positions_fn(layout, W, rows):
    from ..ops.attention import zigzag_positions

    if layout == "zigzag":
        return lambda r: zigzag_positions(W, r, rows // 2)
    return lambda r: [r * rows]


def _ring_inputs(rc: RunCtx, cfg):
    rows, Hq, Hkv, D = cfg["rows"], cfg["hq"], cfg["hkv"], cfg["d"]
    return (rc.randn(rows, Hq, D), rc.randn(rows, Hkv, D, salt=1), rc.randn(rows, Hkv, D, salt=2), bool(cfg["causal"]), cfg["layout"])


def _ring_ref(rc, q, k, v, causal, layout):
    W = rc.world
    pos_of = _positions_fn(layout, W, q.shape[0])
    if q.shape[0] * W <= 8192 or not rc.dist.is_cuda:
        # exact restatement: gather everything, mask by global positions
        import torch.distributed as dist

        if W > 1:
            ks = [torch.empty_like(k) for _ in range(W)]
            vs = [torch.empty_like(v) for _ in range(W)]
            dist.all_gather(ks, k.contiguous())
            dist.all_gather(vs, v.contiguous())
        else:
            ks, vs = [k], [v]
        C = q.shape[0] // len(pos_of(0))
        kv_pos = torch.cat([torch.arange(p, p + C, device=q.device) for s in range(W) for p in pos_of(s)])
        q_pos = torch.cat([torch.arange(p, p + C, device=q.device) for p in pos_of(rc.rank)])
        out, _ = attention_positions_ref(q, torch.cat(ks), torch.cat(vs), q_pos, kv_pos, causal, 1.0 / math.sqrt(q.shape[-1]))
        return out.to(q.dtype)
    return cp_attention_reference(q, k, v, pos_of, W, rc.rank, causal)[0]


def _ring_ours(rc, q, k, v, causal, layout):
    from ..ops.attention import RingAttention

    key = ("ring", q.shape, k.shape, layout)
    if key not in rc.cache:
        rc.cache[key] = RingAttention(rc.comm.group(), q.shape[0], q.shape[1], k.shape[1], q.shape[2], layout=layout)
    return rc.cache[key](q, k, v, causal=causal)[0]


def _ring_cost(cfg, W):
    S = cfg["rows"] * W
    return Cost(flops=4.0 * S * S * cfg["d"] * cfg["hq"] * (0.5 if cfg["causal"] else 1.0) / W,
                nvlink_bytes=2.0 * (W - 1) * cfg["rows"] * cfg["hkv"] * cfg["d"] * 2)


register(OpSpec(name="ring_attention", problem_ids=(54,), group="attention",
                configs={"default": {"rows": 1024, "hq": 8, "hkv": 8, "d": 64, "causal": 1, "layout": "zigzag"},
                         "small": {"rows": 256, "hq": 4, "hkv": 2, "d": 128, "causal": 1, "layout": "zigzag"},
                         "contiguous": {"rows": 512, "hq": 8, "hkv": 2, "d": 128, "causal": 0, "layout": "contiguous"},
                         "cp131k": {"rows": 16384, "hq": 32, "hkv": 8, "d": 128, "causal": 1, "layout": "zigzag"}},
                make_inputs=_ring_inputs, reference=_ring_ref, ours=_ring_ours, atol=2e-2, rtol=2e-2, ours_needs_cuda=True,
                cost=_ring_cost, doc="zigzag context-parallel causal attention, KV exchange inside the attention kernel"))
