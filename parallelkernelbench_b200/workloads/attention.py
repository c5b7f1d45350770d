"""Attention workloads: single-device flash attention and context-parallel (ring) attention.

Reference workloads covered: reference/54_ring_attention.py (forward over a context-parallel group),
and the local attention inside reference/39_ulysses_attention_e2e.py / reference/77_magi1_cso_async_attention.py.
"""
from __future__ import annotations

import math

import torch

from ..harness.roofline import Cost
from ..refs.attention import attention_positions_ref, cp_attention_fwd_bwd_reference, cp_attention_reference
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


def _ring_heap_gib(cfg, W, backward: bool) -> float:
    """Gather buffers for K and V (bf16) and, for the backward, fp32 partial dK / dV for every KV row of the group."""
    per_row = cfg["hkv"] * cfg["d"]
    b = 2 * W * cfg["rows"] * per_row * 2 + (2 * W * cfg["rows"] * per_row * 4 if backward else 0)
    return max(1.0, math.ceil(1.5 * b / (1 << 30) + 0.25))


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
                cost=_ring_cost, heap_gib=lambda cfg, W: _ring_heap_gib(cfg, W, False),
                doc="zigzag context-parallel causal attention, KV exchange inside the attention kernel"))


# ---- context-parallel attention, forward and backward -----------------------------------------------
def _ringfb_inputs(rc: RunCtx, cfg):
    rows, Hq, Hkv, D = cfg["rows"], cfg["hq"], cfg["hkv"], cfg["d"]
    return (rc.randn(rows, Hq, D), rc.randn(rows, Hkv, D, salt=1), rc.randn(rows, Hkv, D, salt=2), rc.randn(rows, Hq, D, salt=3),
            bool(cfg["causal"]), cfg["layout"])


def _ringfb_ref(rc, q, k, v, dout, causal, layout):
    W = rc.world
    exact = q.shape[0] * W <= 4096 or not rc.dist.is_cuda
    return cp_attention_fwd_bwd_reference(q, k, v, dout, _positions_fn(layout, W, q.shape[0]), W, rc.rank, causal, exact=exact)


def _ringfb_ours(rc, q, k, v, dout, causal, layout):
    from ..ops.attention import RingAttention

    key = ("ring", q.shape, k.shape, layout)
    if key not in rc.cache:
        rc.cache[key] = RingAttention(rc.comm.group(), q.shape[0], q.shape[1], k.shape[1], q.shape[2], layout=layout)
    ring = rc.cache[key]
    out, lse = ring(q, k, v, causal=causal)
    dq, dk, dv = ring.backward(q, k, v, out, lse, dout, causal=causal)
    return out, dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def _ringfb_cost(cfg, W):
    S = cfg["rows"] * W
    fwd = 4.0 * S * S * cfg["d"] * cfg["hq"] * (0.5 if cfg["causal"] else 1.0) / W
    return Cost(flops=3.5 * fwd, nvlink_bytes=(2.0 * 2 + 2.0 * 4) * (W - 1) * cfg["rows"] * cfg["hkv"] * cfg["d"])


register(OpSpec(name="ring_attention_fwd_bwd", problem_ids=(54, 57), group="attention",
                configs={"default": {"rows": 512, "hq": 8, "hkv": 2, "d": 128, "causal": 1, "layout": "zigzag"},
                         "small": {"rows": 256, "hq": 4, "hkv": 2, "d": 64, "causal": 1, "layout": "zigzag"},
                         "cp131k": {"rows": 16384, "hq": 32, "hkv": 8, "d": 128, "causal": 1, "layout": "zigzag"}},
                make_inputs=_ringfb_inputs, reference=_ringfb_ref, ours=_ringfb_ours, atol=5e-2, rtol=5e-2, ours_needs_cuda=True,
                cost=_ringfb_cost, heap_gib=lambda cfg, W: _ring_heap_gib(cfg, W, True),
                doc="zigzag context-parallel causal attention, forward and backward (GQA)"))


# =================================================================================================
# attention blocks on 2-D meshes: TP x CP (55), CP x PP (56), CP x DP backward (57)
# =================================================================================================
def _mesh(rc: RunCtx, name: str, inner_pref: int = 2):
    """inner = the small dimension (TP / PP / DP, size min(2, W)), outer = the context-parallel ring."""
    from ..parallel.mesh import Mesh2D, factor_two_level

    key = ("mesh", name)
    if key not in rc.cache:
        _, inner = factor_two_level(rc.world, inner_pref)
        rc.cache[key] = Mesh2D.build(rc.world, inner, rc.rank, inner_name=name, outer_name="cp")
    return rc.cache[key]


def _cp_gather(rc, t, m, ours: bool):
    """All-gather over the context-parallel (outer) group; returns [cp, *t.shape]."""
    cp = m.outer
    if cp == 1:
        return t.unsqueeze(0)
    if ours:
        return rc.comm.all_gather(t.contiguous(), group=m.outer_ranks)
    out = torch.empty((cp, *t.shape), dtype=t.dtype, device=t.device)
    dist_mod().all_gather_into_tensor(out.view(-1, *t.shape[1:]), t.contiguous(), group=m.outer_group)
    return out


def dist_mod():
    import torch.distributed as dist

    return dist


def _cp_attention(rc, q, k, v, m, causal, scale, ours: bool):
    """q, k, v: [B, S_local, H, D] with the sequence sharded contiguously over the outer group."""
    B, S, H, D = q.shape
    cp, r = m.outer, m.outer_rank
    if ours and rc.dist.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and cp > 1 and S % 128 == 0:
        from ..ops.attention import RingAttention

        # batch folded into the head dimension: sequence b of head h becomes head b*H + h of one long sequence
        fold = lambda t: t.permute(1, 0, 2, 3).reshape(S, B * t.shape[2], D).contiguous()  # noqa: E731
        key = ("ring2d", m.inner_name, S, B * H, D)
        if key not in rc.cache:
            rc.cache[key] = RingAttention(rc.comm.group(m.outer_ranks), S, B * H, B * k.shape[2], D, layout="contiguous")
        o = rc.cache[key](fold(q), fold(k), fold(v), causal=causal, scale=scale)[0]
        return o.view(S, B, H, D).permute(1, 0, 2, 3).contiguous()
    kg = _cp_gather(rc, k, m, ours).permute(1, 0, 2, 3, 4).reshape(B, cp * S, k.shape[2], D)
    vg = _cp_gather(rc, v, m, ours).permute(1, 0, 2, 3, 4).reshape(B, cp * S, v.shape[2], D)
    if ours and rc.dist.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128):
        from ..ops.attention import flash_attn_fwd

        return flash_attn_fwd(q.contiguous(), kg.contiguous(), vg.contiguous(), causal=causal, scale=scale, q_segments=[(S, r * S)],
                              return_lse=False)[0]
    q_pos = torch.arange(r * S, (r + 1) * S, device=q.device)
    kv_pos = torch.arange(cp * S, device=q.device)
    return torch.stack([attention_positions_ref(q[b], kg[b], vg[b], q_pos, kv_pos, causal, scale)[0] for b in range(B)]).to(q.dtype)


def _lin(rc, a, w, ours: bool):
    if ours and rc.dist.is_cuda and a.dtype == torch.bfloat16 and a.shape[-1] % 8 == 0:
        from ..ops import gemm_bf16

        return gemm_bf16(a.reshape(-1, a.shape[-1]).contiguous(), w.contiguous()).view(*a.shape[:-1], w.shape[0])
    return torch.nn.functional.linear(a, w)


def _attn_block(rc, hidden, w_qkv, w_o, heads_local, m, causal, ours):
    B, S, _ = hidden.shape
    D = w_qkv.shape[0] // 3 // heads_local
    qkv = _lin(rc, hidden, w_qkv, ours).view(B, S, 3, heads_local, D)
    q, k, v = (qkv[:, :, i].contiguous() for i in range(3))
    ctx = _cp_attention(rc, q, k, v, m, causal, D ** -0.5, ours)
    return _lin(rc, ctx.reshape(B, S, heads_local * D), w_o, ours)


# ---- 55: heads sharded over TP, sequence over CP ---------------------------------------------------
def _p55_inputs(rc: RunCtx, cfg):
    m = _mesh(rc, "tp")
    H, D = cfg["heads"], cfg["d"]
    hid, hl = H * D, H // m.inner
    g_cp = torch.Generator(device=rc.device).manual_seed(4200 + m.outer_rank + 1000003 * rc.trial)
    g_tp = torch.Generator(device=rc.device).manual_seed(14200 + m.inner_rank + 1000003 * rc.trial)
    hidden = torch.randn(cfg["b"], cfg["s_local"], hid, device=rc.device, generator=g_cp).to(rc.dtype)   # same on both TP ranks
    w_qkv = (torch.randn(3 * hl * D, hid, device=rc.device, generator=g_tp) * 0.02).to(rc.dtype)
    w_o = (torch.randn(hid, hl * D, device=rc.device, generator=g_tp) * 0.02).to(rc.dtype)
    return (hidden, w_qkv, w_o, H, bool(cfg["causal"]))


def _p55(rc, hidden, w_qkv, w_o, H, causal, ours):
    m = _mesh(rc, "tp")
    out = _attn_block(rc, hidden, w_qkv, w_o, H // m.inner, m, causal, ours)
    if m.inner > 1:
        if ours:
            out = rc.comm.all_reduce(out, group=m.inner_ranks)
        else:
            dist_mod().all_reduce(out, group=m.inner_group)
    return out


_BLOCK_CFG = {"default": {"b": 16, "s_local": 4, "heads": 8, "d": 64, "causal": 1},
              "small": {"b": 2, "s_local": 8, "heads": 4, "d": 16, "causal": 1},
              "large": {"b": 1, "s_local": 4096, "heads": 32, "d": 128, "causal": 1}}
register(OpSpec(name="ring_attention_tp", problem_ids=(55,), group="attention", configs=_BLOCK_CFG, make_inputs=_p55_inputs,
                reference=lambda rc, *a: _p55(rc, *a, ours=False), ours=lambda rc, *a: _p55(rc, *a, ours=True), atol=3e-2, rtol=3e-2))


# ---- 56: two pipeline stages, context parallel inside each -----------------------------------------
def _p56_inputs(rc: RunCtx, cfg):
    m = _mesh(rc, "pp")
    H, D = cfg["heads"], cfg["d"]
    hid = H * D
    g_cp = torch.Generator(device=rc.device).manual_seed(5200 + m.outer_rank + 1000003 * rc.trial)
    g_pp = torch.Generator(device=rc.device).manual_seed(25200 + m.inner_rank + 1000003 * rc.trial)
    hidden = torch.randn(cfg["b"], cfg["s_local"], hid, device=rc.device, generator=g_cp).to(rc.dtype)
    w_qkv = (torch.randn(3 * hid, hid, device=rc.device, generator=g_pp) * 0.02).to(rc.dtype)
    w_o = (torch.randn(hid, hid, device=rc.device, generator=g_pp) * 0.02).to(rc.dtype)
    return (hidden, w_qkv, w_o, H, bool(cfg["causal"]))


def _p56(rc, hidden, w_qkv, w_o, H, causal, ours):
    """Stage hand-off stays on the process group's point-to-point path in both implementations."""
    m = _mesh(rc, "pp")
    dist = dist_mod()
    stage, n_stage = m.inner_rank, m.inner
    x = hidden
    if stage > 0:
        x = torch.empty_like(hidden)
        dist.recv(x, src=m.inner_ranks[stage - 1])
    y = _attn_block(rc, x, w_qkv, w_o, H, m, causal, ours)
    if stage + 1 < n_stage:
        dist.send(y.contiguous(), dst=m.inner_ranks[stage + 1])
    return y


register(OpSpec(name="ring_attention_pp", problem_ids=(56,), group="attention", configs=_BLOCK_CFG, make_inputs=_p56_inputs,
                reference=lambda rc, *a: _p56(rc, *a, ours=False), ours=lambda rc, *a: _p56(rc, *a, ours=True), atol=3e-2, rtol=3e-2))


# ---- 57: context-parallel attention backward, gradients averaged over DP ---------------------------
def _p57_inputs(rc: RunCtx, cfg):
    """Forward outputs (out, lse) are those of the whole context-parallel sequence, so the result is the true gradient."""
    m = _mesh(rc, "dp")
    S, Hq, Hkv, D = cfg["s_local"], cfg["hq"], cfg["hkv"], cfg["d"]
    causal = bool(cfg["causal"])
    q, k, v, dout = rc.randn(S, Hq, D), rc.randn(S, Hkv, D, salt=1), rc.randn(S, Hkv, D, salt=2), rc.randn(S, Hq, D, salt=3)
    kg = _cp_gather(rc, k, m, False).reshape(-1, Hkv, D)
    vg = _cp_gather(rc, v, m, False).reshape(-1, Hkv, D)
    q_pos = torch.arange(m.outer_rank * S, (m.outer_rank + 1) * S, device=rc.device)
    kv_pos = torch.arange(m.outer * S, device=rc.device)
    out, lse = attention_positions_ref(q, kg, vg, q_pos, kv_pos, causal, D ** -0.5)
    return (dout, q, k, v, out.to(rc.dtype), lse, causal)


def _p57(rc, dout, q, k, v, out, lse, causal, ours):
    from ..refs.attention import attention_bwd_positions_ref

    m = _mesh(rc, "dp")
    S, Hkv, D = k.shape
    cp, r = m.outer, m.outer_rank
    kg = _cp_gather(rc, k, m, ours).reshape(-1, Hkv, D)
    vg = _cp_gather(rc, v, m, ours).reshape(-1, Hkv, D)
    q_pos = torch.arange(r * S, (r + 1) * S, device=q.device)
    kv_pos = torch.arange(cp * S, device=q.device)
    if ours and rc.dist.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128):
        from ..ops.attention import flash_attn_bwd

        dq, dkf, dvf = flash_attn_bwd(q, kg, vg, out, lse, dout, causal=causal, scale=D ** -0.5, q_pos0=r * S)
    else:
        dq, dkf, dvf = attention_bwd_positions_ref(q, kg, vg, out, lse, dout, q_pos, kv_pos, causal, D ** -0.5)
    dq, dkf, dvf = dq.float(), dkf.float().contiguous(), dvf.float().contiguous()
    if cp > 1:                                                   # every rank holds partial dK/dV for all rows: reduce to the owners
        if ours:
            dk, dv = rc.comm.reduce_scatter(dkf, group=m.outer_ranks), rc.comm.reduce_scatter(dvf, group=m.outer_ranks)
        else:
            dk, dv = torch.empty((S, Hkv, D), device=q.device), torch.empty((S, Hkv, D), device=q.device)
            dist_mod().reduce_scatter_tensor(dk, dkf, group=m.outer_group) if dist_mod().get_backend() != "gloo" else dk.copy_(_gloo_rs(dkf, m))
            dist_mod().reduce_scatter_tensor(dv, dvf, group=m.outer_group) if dist_mod().get_backend() != "gloo" else dv.copy_(_gloo_rs(dvf, m))
    else:
        dk, dv = dkf, dvf
    grads = [dq.contiguous(), dk, dv]
    if m.inner > 1:
        if ours:
            packed = rc.comm.all_reduce(torch.cat([g.reshape(-1) for g in grads]), group=m.inner_ranks, scale=1.0 / m.inner)
            outs, o = [], 0
            for g in grads:
                outs.append(packed[o:o + g.numel()].view(g.shape))
                o += g.numel()
            grads = outs
        else:
            for g in grads:
                dist_mod().all_reduce(g, group=m.inner_group)
                g.div_(m.inner)
    return tuple(g.to(q.dtype) for g in grads)


def _gloo_rs(full, m):
    t = full.clone()
    dist_mod().all_reduce(t, group=m.outer_group)
    S = full.shape[0] // m.outer
    return t[m.outer_rank * S:(m.outer_rank + 1) * S]


register(OpSpec(name="ring_attention_backward_dp", problem_ids=(57,), group="attention",
                configs={"default": {"s_local": 128, "hq": 8, "hkv": 8, "d": 64, "causal": 0},
                         "small": {"s_local": 32, "hq": 4, "hkv": 2, "d": 16, "causal": 1},
                         "large": {"s_local": 4096, "hq": 32, "hkv": 8, "d": 128, "causal": 1}},
                make_inputs=_p57_inputs, reference=lambda rc, *a: _p57(rc, *a, ours=False), ours=lambda rc, *a: _p57(rc, *a, ours=True),
                atol=5e-2, rtol=5e-2))
