"""PyTorch (+NCCL) references for attention.

``attention_positions_ref``  exact fp32 restatement with explicit global positions (small shapes).
``cp_attention_reference``   the timed context-parallel baseline: NCCL all-gather of K and V, then the
                             library flash kernel per Q chunk (past chunks un-masked, own chunk causal),
                             merged by log-sum-exp.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist


def attention_positions_ref(q, k, v, q_pos, kv_pos, causal: bool, scale: float):
    """q [Sq,Hq,D], k/v [Skv,Hkv,D]; ``q_pos``/``kv_pos`` global positions. Returns (out fp32, lse)."""
    Hq, Hkv = q.shape[1], k.shape[1]
    qf = q.float().permute(1, 0, 2)
    kf = k.float().permute(1, 0, 2).repeat_interleave(Hq // Hkv, dim=0)
    vf = v.float().permute(1, 0, 2).repeat_interleave(Hq // Hkv, dim=0)
    s = torch.einsum("hqd,hkd->hqk", qf, kf) * scale
    if causal:
        s = s.masked_fill((kv_pos[None, :] > q_pos[:, None])[None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.nan_to_num(torch.softmax(s, dim=-1))
    return torch.einsum("hqk,hkd->hqd", p, vf).permute(1, 0, 2), lse


def _flash(q, k, v, causal, scale):
    """Library flash attention on [S,H,D] tensors with GQA; returns (out [S,H,D], lse [H,S])."""
    Hq, Hkv = q.shape[1], k.shape[1]
    qt = q.permute(1, 0, 2).unsqueeze(0)
    kt = k.permute(1, 0, 2).unsqueeze(0).repeat_interleave(Hq // Hkv, dim=1)
    vt = v.permute(1, 0, 2).unsqueeze(0).repeat_interleave(Hq // Hkv, dim=1)
    res = torch.ops.aten._scaled_dot_product_flash_attention(qt, kt, vt, 0.0, causal, False, scale=scale)
    return res[0][0].permute(1, 0, 2), res[1][0]


def _merge(o1, l1, o2, l2):
    lse = torch.logaddexp(l1, l2)
    w1 = torch.exp(l1 - lse).t().unsqueeze(-1)
    w2 = torch.exp(l2 - lse).t().unsqueeze(-1)
    return (o1.float() * w1 + o2.float() * w2), lse


def cp_attention_reference(q, k, v, positions_of, world: int, rank: int, causal: bool, scale: float | None = None, group=None):
    """``q``/``k``/``v``: this rank's rows [rows, H, D] made of equal chunks whose global start positions
    are ``positions_of(rank)``. Returns (out [rows, Hq, D] in q.dtype, lse [Hq, rows])."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    rows = q.shape[0]
    if world > 1:
        kg = torch.empty((world * rows, *k.shape[1:]), dtype=k.dtype, device=k.device)
        vg = torch.empty_like(kg)
        dist.all_gather_into_tensor(kg, k.contiguous(), group=group)
        dist.all_gather_into_tensor(vg, v.contiguous(), group=group)
    else:
        kg, vg = k, v
    nseg = len(positions_of(0))
    C = rows // nseg
    # global order of the gathered chunks
    chunks = sorted((pos, src * rows + i * C) for src in range(world) for i, pos in enumerate(positions_of(src)))
    kfull = torch.cat([kg[row0:row0 + C] for _, row0 in chunks])
    vfull = torch.cat([vg[row0:row0 + C] for _, row0 in chunks])
    outs, lses = [], []
    for i, pos in enumerate(positions_of(rank)):
        qc = q[i * C:(i + 1) * C]
        if not causal:
            o, l = _flash(qc, kfull, vfull, False, scale)
        else:
            o, l = _flash(qc, kfull[pos:pos + C], vfull[pos:pos + C], True, scale)
            if pos > 0:
                o0, l0 = _flash(qc, kfull[:pos], vfull[:pos], False, scale)
                o, l = _merge(o0, l0, o, l)
        outs.append(o.to(q.dtype))
        lses.append(l)
    return torch.cat(outs), torch.cat(lses, dim=1)


def attention_bwd_positions_ref(q, k, v, out, lse, dout, q_pos, kv_pos, causal: bool, scale: float):
    """Explicit attention backward in fp32 from a saved forward (``out`` [Sq,Hq,D], ``lse`` [Hq,Sq]).

    P = exp(S - lse); dV = P^T dO; dP = dO V^T; dS = P * (dP - rowsum(dO * O)); dQ = dS K * scale; dK = dS^T Q * scale.
    GQA: the gradients of the query heads that share a KV head are summed. Returns (dq, dk, dv) in fp32.
    """
    Hq, Hkv = q.shape[1], k.shape[1]
    rep = Hq // Hkv
    qf, of, dof = (t.float().permute(1, 0, 2) for t in (q, out, dout))
    kf = k.float().permute(1, 0, 2).repeat_interleave(rep, dim=0)
    vf = v.float().permute(1, 0, 2).repeat_interleave(rep, dim=0)
    s = torch.einsum("hqd,hkd->hqk", qf, kf) * scale
    if causal:
        s = s.masked_fill((kv_pos[None, :] > q_pos[:, None])[None], float("-inf"))
    p = torch.exp(s - lse.float()[:, :, None])
    dv = torch.einsum("hqk,hqd->hkd", p, dof)
    dp = torch.einsum("hqd,hkd->hqk", dof, vf)
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta)
    dq = torch.einsum("hqk,hkd->hqd", ds, kf) * scale
    dk = torch.einsum("hqk,hqd->hkd", ds, qf) * scale
    Skv, D = k.shape[0], k.shape[2]
    dk = dk.reshape(Hkv, rep, Skv, D).sum(1)
    dv = dv.reshape(Hkv, rep, Skv, D).sum(1)
    return dq.permute(1, 0, 2), dk.permute(1, 0, 2), dv.permute(1, 0, 2)


def cp_attention_fwd_bwd_reference(q, k, v, dout, positions_of, world: int, rank: int, causal: bool, scale: float | None = None,
                                   group=None, exact: bool = False):
    """Forward and backward of context-parallel attention the PyTorch + process-group way: all-gather K and V, run the
    library flash kernel per query chunk (or the exact fp32 restatement when ``exact``), let autograd produce dQ and the
    gradients of the gathered K / V, and reduce-scatter those to their owners. Returns (out, dq, dk, dv) in q.dtype."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    rows = q.shape[0]
    with torch.enable_grad():
        ql = q.detach().clone().requires_grad_()
        if world > 1:
            kg = torch.empty((world * rows, *k.shape[1:]), dtype=k.dtype, device=k.device)
            vg = torch.empty_like(kg)
            dist.all_gather_into_tensor(kg, k.contiguous(), group=group)
            dist.all_gather_into_tensor(vg, v.contiguous(), group=group)
        else:
            kg, vg = k.detach().clone(), v.detach().clone()
        kg.requires_grad_()
        vg.requires_grad_()
        nseg = len(positions_of(0))
        C = rows // nseg
        chunks = sorted((pos, src * rows + i * C) for src in range(world) for i, pos in enumerate(positions_of(src)))
        kfull = torch.cat([kg[row0:row0 + C] for _, row0 in chunks])
        vfull = torch.cat([vg[row0:row0 + C] for _, row0 in chunks])
        outs = []
        for i, pos in enumerate(positions_of(rank)):
            qc = ql[i * C:(i + 1) * C]
            if exact:
                q_pos = torch.arange(pos, pos + C, device=q.device)
                kv_pos = torch.arange(kfull.shape[0], device=q.device)
                o = attention_positions_ref(qc, kfull, vfull, q_pos, kv_pos, causal, scale)[0]
            elif not causal:
                o = _flash(qc, kfull, vfull, False, scale)[0]
            else:
                o, l = _flash(qc, kfull[pos:pos + C], vfull[pos:pos + C], True, scale)
                if pos > 0:
                    o0, l0 = _flash(qc, kfull[:pos], vfull[:pos], False, scale)
                    o, _ = _merge(o0, l0, o, l)
            outs.append(o)
        out = torch.cat(outs)
        out.backward(dout.to(out.dtype))
    dkg, dvg = kg.grad.float(), vg.grad.float()
    if world > 1:
        if dist.get_backend(group) == "gloo":
            dist.all_reduce(dkg, group=group)
            dist.all_reduce(dvg, group=group)
            dk, dv = dkg[rank * rows:(rank + 1) * rows], dvg[rank * rows:(rank + 1) * rows]
        else:
            dk, dv = torch.empty((rows, *k.shape[1:]), device=k.device), torch.empty((rows, *k.shape[1:]), device=k.device)
            dist.reduce_scatter_tensor(dk, dkg, group=group)
            dist.reduce_scatter_tensor(dv, dvg, group=group)
    else:
        dk, dv = dkg, dvg
    return out.detach().to(q.dtype), ql.grad.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)
