"""Data-parallel / ZeRO / FSDP optimiser steps and distributed loss helpers.

The model in the DDP / ZeRO / FSDP workloads is a two-layer MLP with an MSE loss. "ours" computes
its forward and backward by hand on the tcgen05 GEMM (bf16) and fuses the optimiser with the
collectives the strategy needs: gradients are reduce-scattered, the Adam update runs on the shard
that arrives, and the new parameters are gathered - the same kernel sequence serves DDP, ZeRO-1,
ZeRO-2 and FSDP because on NVSwitch an all-reduce is exactly reduce-scatter + all-gather.
Reference workloads covered: reference/21_clip_grad_norm_no_ep.py ... reference/24_load_balancing_loss_fn.py,
reference/40_ddp.py ... reference/43_fused_adam_grad_unshard_allgather.py, reference/47_fsdp_step_e2e.py.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..harness.roofline import Cost
from .registry import OpSpec, RunCtx, register


# =================================================================================================
# gradient clipping by global norm (21, 22)
# =================================================================================================
def _clip_inputs(rc, cfg):
    return ([rc.randn(cfg["m"], cfg["n"], salt=i) for i in range(3)], 1.0, 2.0)


def _clip_ref(rc, grads, max_norm, p):
    grads = [g.clone() for g in grads]
    acc = torch.zeros((), device=rc.device, dtype=torch.float32)
    for g in grads:
        acc = acc + torch.norm(g.float(), p=p) ** p
    if rc.world > 1:
        dist.all_reduce(acc)
    total = acc ** (1.0 / p)
    if total > max_norm:                      # host branch (a device -> host sync)
        for g in grads:
            g.mul_((max_norm / total).to(g.dtype))
    return {"total_norm": total, "grads": grads}


def _clip_ours(rc, grads, max_norm, p):
    grads = [g.clone() for g in grads]
    if rc.dist.is_cuda and p == 2.0 and grads[0].dtype in (torch.bfloat16, torch.float32):
        from ..ops.quant import clip_grad_norm_

        # three launches (sum of squares of all tensors, the scalar all-reduce, the scaling), no host branch
        total = clip_grad_norm_(grads, max_norm, rc.comm)
        return {"total_norm": total, "grads": grads}
    acc = torch.stack([(g.float().abs() ** p).sum() for g in grads]).sum().reshape(1)
    total = rc.comm.all_reduce(acc) ** (1.0 / p)
    # branch-free: the coefficient is computed on the device, nothing returns to the host
    coef = torch.clamp(max_norm / total, max=1.0)
    for g in grads:
        g.mul_(coef.to(g.dtype))
    return {"total_norm": total.reshape(()), "grads": grads}


register(OpSpec(name="clip_grad_norm", problem_ids=(21,), group="optim", configs={"default": {"m": 1024, "n": 1024}, "small": {"m": 16, "n": 16}},
                make_inputs=_clip_inputs, reference=_clip_ref, ours=_clip_ours, atol=2e-2, rtol=2e-2,
                cost=lambda cfg, W: Cost(hbm_bytes=3 * 3 * cfg["m"] * cfg["n"] * 2)))


def _clip_ep_mesh(rc):
    from ..parallel.mesh import Mesh2D, factor_two_level

    if "mesh22" not in rc.cache:
        _, ep = factor_two_level(rc.world, 2)
        rc.cache["mesh22"] = Mesh2D.build(rc.world, ep, rc.rank, inner_name="ep", outer_name="ep_fsdp")
    return rc.cache["mesh22"]


def _clip_ep_inputs(rc, cfg):
    m = _clip_ep_mesh(rc)
    return ([rc.randn(cfg["m"], cfg["n"], salt=i) for i in range(2)], [rc.randn(cfg["m"], cfg["n"], salt=10 + i) for i in range(2)],
            1.0, 2.0, m.inner)


def _clip_ep_ref(rc, non_ep, ep_grads, max_norm, p, ep_size):
    m = _clip_ep_mesh(rc)
    non_ep = [g.clone() for g in non_ep]
    ep_grads = [g.clone() / ep_size for g in ep_grads]      # EP gradients are pre-scaled by 1/ep
    a = sum(torch.norm(g.float(), p=p) ** p for g in non_ep)
    b = sum(torch.norm(g.float(), p=p) ** p for g in ep_grads)
    if rc.world > 1:
        dist.all_reduce(a)                                   # dense params: sharded over the whole job
        if m.outer_group is not None:
            dist.all_reduce(b, group=m.outer_group)          # expert params: over their FSDP group ...
        if m.inner_group is not None:
            dist.all_reduce(b, group=m.inner_group)          # ... then over the EP group
    total = (a + b) ** (1.0 / p)
    coef = torch.clamp(max_norm / total, max=1.0)
    for g in non_ep + ep_grads:
        g.mul_(coef.to(g.dtype))
    return {"total_norm": total, "non_ep": non_ep, "ep": ep_grads}


def _clip_ep_ours(rc, non_ep, ep_grads, max_norm, p, ep_size):
    m = _clip_ep_mesh(rc)
    if rc.dist.is_cuda and p == 2.0 and non_ep[0].dtype in (torch.bfloat16, torch.float32):
        from ..ops.quant import clip_grad_norm_

        # expert gradients enter pre-scaled by 1/ep; both reductions (EP-FSDP then EP) together span the whole job
        dense, experts = [g.clone() for g in non_ep], [g.clone() for g in ep_grads]
        total = clip_grad_norm_(dense + experts, max_norm, rc.comm, pre_scale=[1.0] * len(dense) + [1.0 / ep_size] * len(experts))
        return {"total_norm": total, "non_ep": dense, "ep": experts}
    non_ep = [g.clone() for g in non_ep]
    ep_grads = [g.clone() / ep_size for g in ep_grads]
    a = torch.stack([(g.float().abs() ** p).sum() for g in non_ep]).sum().reshape(1)
    b = torch.stack([(g.float().abs() ** p).sum() for g in ep_grads]).sum().reshape(1)
    # both reductions over (ep_fsdp x ep) cover the whole job: one packed all-reduce does it
    ab = rc.comm.all_reduce(torch.cat([a, b]))
    total = (ab[0] + ab[1]) ** (1.0 / p)
    coef = torch.clamp(max_norm / total, max=1.0)
    for g in non_ep + ep_grads:
        g.mul_(coef.to(g.dtype))
    return {"total_norm": total, "non_ep": non_ep, "ep": ep_grads}


register(OpSpec(name="clip_grad_norm_ep", problem_ids=(22,), group="optim", configs={"default": {"m": 512, "n": 512}, "small": {"m": 8, "n": 16}},
                make_inputs=_clip_ep_inputs, reference=_clip_ep_ref, ours=_clip_ep_ours, atol=2e-2, rtol=2e-2))


# =================================================================================================
# token-weighted loss normalisation (23) and router load-balancing loss (24)
# =================================================================================================
def _gal_inputs(rc, cfg):
    n = cfg["m"] * cfg["n"]
    return (rc.randn(1, dtype=torch.float32).reshape(()), torch.tensor(n, device=rc.device), torch.tensor(n * rc.world, device=rc.device),
            torch.ones((), device=rc.device), torch.zeros((), device=rc.device))


def _gal_common(loss, lv, gv, g_norm, g_sum, reduce_fn):
    loss = torch.where(lv == 0, torch.nan_to_num(loss), loss)
    loss_sum = reduce_fn((loss * lv).reshape(1)).reshape(())
    return loss_sum / gv, loss_sum, g_norm * lv / gv + g_sum * lv


def _gal_ref(rc, loss, lv, gv, g_norm, g_sum):
    def red(t):
        if rc.world > 1:
            dist.all_reduce(t)
        return t
    return _gal_common(loss, lv, gv, g_norm, g_sum, red)


register(OpSpec(name="grad_acc_loss", problem_ids=(23,), group="optim", configs={"default": {"m": 1024, "n": 1024}},
                make_inputs=_gal_inputs, reference=_gal_ref,
                ours=lambda rc, loss, lv, gv, gn, gs: _gal_common(loss, lv, gv, gn, gs, lambda t: rc.comm.all_reduce(t)),
                atol=1e-3, rtol=1e-4))


def _lb_core(logits, num_experts, top_k):
    w = torch.softmax(logits.float(), dim=-1)
    _, sel = torch.topk(w, top_k, dim=-1)
    mask = F.one_hot(sel, num_experts).float()                 # [T, k, E]
    return (mask.mean(0) * w.mean(0).unsqueeze(0)).sum() * num_experts


def _lb_ref(rc, logits, num_experts, top_k):
    loss = _lb_core(logits, num_experts, top_k)
    if rc.world > 1:
        dist.all_reduce(loss)
    return loss / rc.world


register(OpSpec(name="load_balancing_loss", problem_ids=(24,), group="optim", configs={"default": {"m": 1024, "experts": 8, "topk": 2}},
                make_inputs=lambda rc, cfg: (rc.randn(cfg["m"], cfg["experts"]), cfg["experts"], cfg["topk"]),
                reference=_lb_ref,
                ours=lambda rc, lg, e, k: rc.comm.all_reduce(_lb_core(lg, e, k).reshape(1), scale=1.0 / rc.world).reshape(()),
                atol=1e-3, rtol=1e-3))


# =================================================================================================
# two-layer MLP with MSE loss: forward + backward by hand
# =================================================================================================
def _nt(rc: RunCtx, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``a[M,K] @ w[N,K].T`` in fp32 out; tcgen05 GEMM for bf16 operands on GPUs."""
    if rc.dist.is_cuda and a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0:
        from ..ops import gemm_bf16

        return gemm_bf16(a.contiguous(), w.contiguous(), out_dtype=torch.float32)
    return a.float() @ w.float().t()


def mlp_grads(rc: RunCtx, x, y, w1, b1, w2, b2):
    """Gradients of ``mse(relu(x w1^T + b1) w2^T + b2, y)`` as one flat fp32 vector [w1, b1, w2, b2]."""
    dt = x.dtype
    z1 = (_nt(rc, x, w1) + b1.float()).to(dt)
    h = torch.relu(z1)
    out = (_nt(rc, h, w2) + b2.float()).to(dt)
    dout = ((out.float() - y.float()) * (2.0 / out.numel())).to(dt)
    dw2 = _nt(rc, dout.t().contiguous(), h.t().contiguous())
    db2 = dout.float().sum(0)
    dh = _nt(rc, dout, w2.t().contiguous()).to(dt)
    dz1 = dh * (z1 > 0).to(dt)
    dw1 = _nt(rc, dz1.t().contiguous(), x.t().contiguous())
    db1 = dz1.float().sum(0)
    return torch.cat([dw1.reshape(-1), db1, dw2.reshape(-1), db2]).to(dt)


def _mlp_grads_autograd(x, y, w1, b1, w2, b2):
    with torch.enable_grad():
        ps = [t.detach().clone().requires_grad_(True) for t in (w1, b1, w2, b2)]
        loss = F.mse_loss(F.linear(torch.relu(F.linear(x, ps[0], ps[1])), ps[2], ps[3]), y)
        loss.backward()
    return torch.cat([p.grad.reshape(-1) for p in ps])


def _adam_torch(p, m, v, g, lr, b1, b2, eps, step, wd=0.0):
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    upd = (m / (1 - math.pow(b1, step))) / ((v / (1 - math.pow(b2, step))).sqrt() + eps)
    return p - lr * upd - lr * wd * p, m, v


def _adam_ours(rc, p, m, v, g, lr, b1, b2, eps, step, wd=0.0):
    """Adam on a flat shard; the fused CUDA kernel keeps fp32 state, as the fp32 master copy does."""
    if rc.dist.is_cuda:
        from ..ops import adam_step

        pf, mf, vf = p.float().contiguous(), m.float().contiguous(), v.float().contiguous()
        adam_step(pf, mf, vf, g.float().contiguous(), lr=lr, beta1=b1, beta2=b2, eps=eps, step=step, weight_decay=wd, decoupled=True)
        return pf.to(p.dtype), mf.to(m.dtype), vf.to(v.dtype)
    pn, mn, vn = _adam_torch(p.float(), m.float(), v.float(), g.float(), lr, b1, b2, eps, step, wd)
    return pn.to(p.dtype), mn.to(m.dtype), vn.to(v.dtype)


def _mlp_dims(cfg, W):
    n_total = (max(cfg["m"], W) + W - 1) // W * W
    return n_total, max(16, min(cfg["n"], 256)), max(32, min(cfg["n"] // 2, 512)), max(8, min(cfg["n"] // 4, 256))


def _mlp_param_count(cfg, W) -> int:
    _, d_in, hid, d_out = _mlp_dims(cfg, W)
    return hid * d_in + hid + d_out * hid + d_out


def _step_cost(cfg, W, broadcasts: int = 0) -> Cost:
    """Communication and memory floor of one data-parallel optimiser step on the two-layer MLP: the gradient crosses the links
    once reduced ((W-1)/W of it per rank) and the new parameters once gathered; parameters, two moments and the gradient are
    read and the first three written, in bf16."""
    n = _mlp_param_count(cfg, W)
    return Cost(nvlink_bytes=(2.0 + broadcasts) * n * 2 * (W - 1) / max(W, 1), hbm_bytes=7.0 * n * 2 / max(W, 1))


def _mlp_data(rc, cfg, salt=0):
    n_total, d_in, hid, d_out = _mlp_dims(cfg, rc.world)
    chunk = n_total // rc.world
    fx = rc.randn(n_total, d_in, shared=True, salt=salt + 1)
    fy = rc.randn(n_total, d_out, shared=True, salt=salt + 2)
    sl = slice(rc.rank * chunk, (rc.rank + 1) * chunk)
    shapes = [(hid, d_in), (hid,), (d_out, hid), (d_out,)]
    return fx[sl].contiguous(), fy[sl].contiguous(), shapes


def _pad_to(flat, mult):
    pad = (-flat.numel()) % mult
    return F.pad(flat, (0, pad)) if pad else flat


_HYP = (1e-3, 0.9, 0.999, 1e-8)


def _fused_step(rc, part):
    """The one-launch reduce-scatter -> Adam -> all-gather step for shards of ``part`` elements (GPU, bf16, part % 8 == 0), or
    None where it does not apply. ``PKB_UNFUSED_OPTIM=1`` keeps the three-launch form."""
    import os

    if not rc.dist.is_cuda or rc.dtype != torch.bfloat16 or part % 8 or rc.world < 2 or os.environ.get("PKB_UNFUSED_OPTIM") == "1":
        return None
    key = ("zero_adam", part)
    if key not in rc.cache:
        from ..ops.optim import ZeroAdamStep

        rc.cache[key] = ZeroAdamStep(rc.comm.group(), part)
    return rc.cache[key]


# ---- 40: DDP ---------------------------------------------------------------------------------------
def _ddp_inputs(rc, cfg):
    x, y, shapes = _mlp_data(rc, cfg)
    params = [rc.randn(*s, shared=True, salt=10 + i, std=0.2) if rc.rank == 0 else torch.zeros(s, device=rc.device, dtype=rc.dtype)
              for i, s in enumerate(shapes)]
    zeros = [torch.zeros(s, device=rc.device, dtype=rc.dtype) for s in shapes]
    return (x, y, params, zeros, [z.clone() for z in zeros], *_HYP, 1 + rc.trial % 7)


def _ddp_ref(rc, x, y, params, ms, vs, lr, b1, b2, eps, step):
    flat = torch.cat([p.reshape(-1) for p in params])
    fm = torch.cat([p.reshape(-1) for p in ms])
    fv = torch.cat([p.reshape(-1) for p in vs])
    if rc.world > 1:
        for t in (flat, fm, fv):
            dist.broadcast(t, src=0)
    ps = _split(flat, params)
    g = _mlp_grads_autograd(x, y, *ps)
    if rc.world > 1:
        dist.all_reduce(g)
    g = g / rc.world
    p, m, v = _adam_torch(flat.float(), fm.float(), fv.float(), g.float(), lr, b1, b2, eps, step)
    return {"params": p.to(flat.dtype), "m": m.to(flat.dtype), "v": v.to(flat.dtype)}


def _split(flat, like):
    out, o = [], 0
    for t in like:
        out.append(flat[o:o + t.numel()].view(t.shape))
        o += t.numel()
    return out


def _ddp_ours(rc, x, y, params, ms, vs, lr, b1, b2, eps, step):
    W = rc.world
    state = torch.stack([torch.cat([p.reshape(-1) for p in grp]) for grp in (params, ms, vs)])
    if W > 1:
        state = rc.comm.broadcast(state.contiguous(), src=0)            # params, m, v in one broadcast
    flat, fm, fv = state[0], state[1], state[2]
    g = mlp_grads(rc, x, y, *_split(flat, params))
    n = flat.numel()
    fused = _fused_step(rc, (n + 8 * W - 1) // (8 * W) * 8) if W > 1 else None
    if fused is not None:
        # one launch: in-switch sum of this rank's gradient slice, Adam in registers, the new parameters stored on every rank;
        # the moments of the other shards come with a second small gather
        part = fused.part
        fused.grad_buffer.zero_()
        fused.grad_buffer[:n].copy_(g)
        sl = slice(rc.rank * part, (rc.rank + 1) * part)
        pad = lambda t: F.pad(t, (0, W * part - n))[sl].contiguous()  # noqa: E731
        ps, ms_, vs_ = pad(flat), pad(fm), pad(fv)
        p = fused.step(ps, ms_, vs_, lr=lr, beta1=b1, beta2=b2, eps=eps, step=step, grad_scale=1.0 / W)[:n].clone()
        mv = rc.comm.all_gather(torch.stack([ms_, vs_]))                # [W, 2, part]
        m, v = (mv[:, i].reshape(-1)[:n] for i in range(2))
    elif W > 1:
        # all-reduce = reduce-scatter + all-gather: update the shard between the two halves
        gs = rc.comm.reduce_scatter(_pad_to(g, W).contiguous(), scale=1.0 / W)
        sh = gs.numel()
        sl = slice(rc.rank * sh, (rc.rank + 1) * sh)
        p, m, v = _adam_ours(rc, _pad_to(flat, W)[sl], _pad_to(fm, W)[sl], _pad_to(fv, W)[sl], gs, lr, b1, b2, eps, step)
        full = rc.comm.all_gather(torch.stack([p, m, v]))               # [W, 3, shard]
        p, m, v = (full[:, i].reshape(-1)[:n] for i in range(3))
    else:
        p, m, v = _adam_ours(rc, flat, fm, fv, g, lr, b1, b2, eps, step)
    return {"params": p, "m": m, "v": v}


_MLP_CFG = {"default": {"m": 1024, "n": 1024}, "small": {"m": 32, "n": 64}}
register(OpSpec(name="ddp_step", problem_ids=(40,), group="optim", configs=_MLP_CFG, make_inputs=_ddp_inputs, reference=_ddp_ref,
                ours=_ddp_ours, atol=2e-2, rtol=2e-2, cost=lambda cfg, W: _step_cost(cfg, W, broadcasts=3)))


# ---- 41 / 42: ZeRO-1 / ZeRO-2 (optimizer state sharded; grads all-reduced vs reduce-scattered) --------
def _zero_inputs(rc, cfg):
    x, y, shapes = _mlp_data(rc, cfg)
    params = [rc.randn(*s, shared=True, salt=10 + i, std=0.2) for i, s in enumerate(shapes)]
    n = sum(p.numel() for p in params)
    part = (n + rc.world - 1) // rc.world
    z = torch.zeros(part, device=rc.device, dtype=rc.dtype)
    return (x, y, params, z, z.clone(), *_HYP, 1 + rc.trial % 7)


def _zero_ref(stage):
    def ref(rc, x, y, params, m_part, v_part, lr, b1, b2, eps, step):
        W, r = rc.world, rc.rank
        flat = torch.cat([p.reshape(-1) for p in params])
        if W > 1:
            dist.broadcast(flat, src=0)
        g = _mlp_grads_autograd(x, y, *_split(flat, params))
        part = m_part.numel()
        gp, fp = _pad_to(g, W * part) if g.numel() < W * part else g, _pad_to(flat, W * part) if flat.numel() < W * part else flat
        gp = F.pad(g, (0, W * part - g.numel()))
        fp = F.pad(flat, (0, W * part - flat.numel()))
        if stage == 1:
            if W > 1:
                dist.all_reduce(gp)
            gs = gp[r * part:(r + 1) * part] / W
        else:
            gs = gp.new_empty(part)
            if W > 1:
                dist.reduce_scatter_tensor(gs, gp.contiguous())
            else:
                gs.copy_(gp)
            gs = gs / W
        p, m, v = _adam_torch(fp[r * part:(r + 1) * part].float(), m_part.float(), v_part.float(), gs.float(), lr, b1, b2, eps, step)
        p = p.to(flat.dtype)
        full = p.new_empty(W * part)
        if W > 1:
            dist.all_gather_into_tensor(full, p.contiguous())
        else:
            full.copy_(p)
        return {"params": full[:flat.numel()], "m": m.to(flat.dtype), "v": v.to(flat.dtype)}
    return ref


def _zero_ours(rc, x, y, params, m_part, v_part, lr, b1, b2, eps, step):
    W, r = rc.world, rc.rank
    flat = torch.cat([p.reshape(-1) for p in params])
    if W > 1:
        flat = rc.comm.broadcast(flat.contiguous(), src=0)
    g = mlp_grads(rc, x, y, *_split(flat, params))
    part = m_part.numel()
    fp = F.pad(flat, (0, W * part - flat.numel()))
    fused = _fused_step(rc, part) if W > 1 else None
    if fused is not None:
        # reduce-scatter of the gradient, Adam on the shard and all-gather of the new parameters in one launch
        fused.grad_buffer.zero_()
        fused.grad_buffer[:g.numel()].copy_(g)
        ps, m, v = fp[r * part:(r + 1) * part].contiguous(), m_part.clone(), v_part.clone()
        full = fused.step(ps, m, v, lr=lr, beta1=b1, beta2=b2, eps=eps, step=step, grad_scale=1.0 / W)
        return {"params": full[:flat.numel()].clone(), "m": m, "v": v}
    gp = F.pad(g, (0, W * part - g.numel()))
    gs = rc.comm.reduce_scatter(gp.contiguous(), scale=1.0 / W) if W > 1 else gp
    p, m, v = _adam_ours(rc, fp[r * part:(r + 1) * part], m_part, v_part, gs, lr, b1, b2, eps, step)
    full = rc.comm.all_gather(p.contiguous()).reshape(-1) if W > 1 else p
    return {"params": full[:flat.numel()], "m": m, "v": v}


register(OpSpec(name="zero1_step", problem_ids=(41,), group="optim", configs=_MLP_CFG, make_inputs=_zero_inputs, reference=_zero_ref(1),
                ours=_zero_ours, atol=2e-2, rtol=2e-2, cost=_step_cost))
register(OpSpec(name="zero2_step", problem_ids=(42,), group="optim", configs=_MLP_CFG, make_inputs=_zero_inputs, reference=_zero_ref(2),
                ours=_zero_ours, atol=2e-2, rtol=2e-2, cost=_step_cost))


# ---- 43: Adam on the shard, then all-gather of the updated parameters ---------------------------------
def _fa_inputs(rc, cfg):
    P = max(64, min(cfg["m"] * 64, 4096))
    fg = rc.randn(P * rc.world, shared=True, salt=1)
    fm = rc.randn(P * rc.world, shared=True, salt=2)
    sl = slice(rc.rank * P, (rc.rank + 1) * P)
    z = torch.zeros(P, device=rc.device, dtype=rc.dtype)
    return (fg[sl].contiguous(), fm[sl].contiguous(), z, z.clone(), *_HYP, 1 + rc.trial % 7)


def _fa_ref(rc, g, w, m, v, lr, b1, b2, eps, step):
    p, _, _ = _adam_torch(w.float(), m.float(), v.float(), g.float(), lr, b1, b2, eps, step)
    p = p.to(w.dtype)
    out = p.new_empty(rc.world * p.numel())
    if rc.world > 1:
        dist.all_gather_into_tensor(out, p.contiguous())
    else:
        out.copy_(p)
    return out


def _fa_ours(rc, g, w, m, v, lr, b1, b2, eps, step):
    fused = _fused_step(rc, w.numel())
    if fused is not None:
        # Adam on the local shard and the all-gather of the result in one launch (no reduction: the gradient is local)
        fused.grad_buffer[:g.numel()].copy_(g)
        return fused.step(w.clone(), m.clone(), v.clone(), lr=lr, beta1=b1, beta2=b2, eps=eps, step=step, reduce=False).clone()
    p, _, _ = _adam_ours(rc, w, m, v, g, lr, b1, b2, eps, step)
    return rc.comm.all_gather(p.contiguous()).reshape(-1) if rc.world > 1 else p


register(OpSpec(name="fused_adam_allgather", problem_ids=(43,), group="optim", configs={"default": {"m": 1024}, "small": {"m": 1}},
                make_inputs=_fa_inputs, reference=_fa_ref, ours=_fa_ours, atol=2e-2, rtol=2e-2))


# ---- 47: FSDP step end to end (AG params -> fwd/bwd -> RS grads -> AdamW on the shard) ----------------
def _fsdp_inputs(rc, cfg):
    x, y, shapes = _mlp_data(rc, cfg)
    params = [rc.randn(*s, shared=True, salt=10 + i, std=0.2) for i, s in enumerate(shapes)]
    flat = torch.cat([p.reshape(-1) for p in params])
    part = (flat.numel() + rc.world - 1) // rc.world
    fp = F.pad(flat, (0, rc.world * part - flat.numel()))
    z = torch.zeros(part, device=rc.device, dtype=rc.dtype)
    return (x, y, fp[rc.rank * part:(rc.rank + 1) * part].contiguous(), shapes, z, z.clone(), *_HYP, 0.01, 1 + rc.trial % 7)


def _fsdp_ref(rc, x, y, shard, shapes, m, v, lr, b1, b2, eps, wd, step):
    W = rc.world
    full = shard.new_empty(W * shard.numel())
    if W > 1:
        dist.all_gather_into_tensor(full, shard.contiguous())
    else:
        full.copy_(shard)
    n = sum(math.prod(s) for s in shapes)
    like = [torch.empty(s) for s in shapes]
    g = _mlp_grads_autograd(x, y, *_split(full[:n], like))
    gp = F.pad(g, (0, full.numel() - n))
    gs = gp.new_empty(shard.numel())
    if W > 1:
        dist.reduce_scatter_tensor(gs, gp.contiguous())
    else:
        gs.copy_(gp)
    p, mn, vn = _adam_torch(shard.float(), m.float(), v.float(), gs.float() / W, lr, b1, b2, eps, step, wd)
    return p.to(shard.dtype), mn.to(shard.dtype), vn.to(shard.dtype)


def _fsdp_ours(rc, x, y, shard, shapes, m, v, lr, b1, b2, eps, wd, step):
    W = rc.world
    full = rc.comm.all_gather(shard.contiguous()).reshape(-1) if W > 1 else shard
    n = sum(math.prod(s) for s in shapes)
    like = [torch.empty(s) for s in shapes]
    g = mlp_grads(rc, x, y, *_split(full[:n], like))
    fused = _fused_step(rc, shard.numel()) if W > 1 else None
    if fused is not None:
        # gradient reduce-scatter and AdamW on the shard in one launch (the parameters are gathered by the next step)
        fused.grad_buffer.zero_()
        fused.grad_buffer[:n].copy_(g)
        ps, mn, vn = shard.clone(), m.clone(), v.clone()
        fused.step(ps, mn, vn, lr=lr, beta1=b1, beta2=b2, eps=eps, step=step, weight_decay=wd, grad_scale=1.0 / W, gather=False)
        return ps, mn, vn
    gp = F.pad(g, (0, full.numel() - n))
    gs = rc.comm.reduce_scatter(gp.contiguous(), scale=1.0 / W) if W > 1 else gp
    if rc.dist.is_cuda:
        return _adam_ours(rc, shard, m, v, gs, lr, b1, b2, eps, step, wd)
    p, mn, vn = _adam_torch(shard.float(), m.float(), v.float(), gs.float(), lr, b1, b2, eps, step, wd)
    return p.to(shard.dtype), mn.to(shard.dtype), vn.to(shard.dtype)


register(OpSpec(name="fsdp_step", problem_ids=(47,), group="optim", configs=_MLP_CFG, make_inputs=_fsdp_inputs, reference=_fsdp_ref,
                ours=_fsdp_ours, atol=2e-2, rtol=2e-2, cost=_step_cost))
