"""Bare collectives and the no-GPU plumbing configuration.

Inputs are constant ``rank + 1`` patterns by default (sums are exactly representable, so results are
compared bitwise-tight) with a ``random=1`` override for accumulation-order coverage; shapes default
to 1024 x 1024 like the reference's collective problems (reference: reference/1_allreduce.py ...
reference/8_alltoall.py, inputs: utils/input_output_tensors.py:297-314).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..harness.roofline import Cost
from .registry import OpSpec, RunCtx, register

_CFG = {"default": {"m": 1024, "n": 1024}, "small": {"m": 8, "n": 128}, "large": {"m": 8192, "n": 8192}}


def _esize(rc):
    return torch.empty((), dtype=rc.dtype).element_size()


def _fill(rc: RunCtx, cfg: dict, *lead):
    shape = (*lead, cfg["m"], cfg["n"])
    if cfg.get("random"):
        return rc.randn(*shape)
    return torch.full(shape, float(rc.rank + 1), device=rc.device, dtype=rc.dtype)


# ---- all-reduce ------------------------------------------------------------------------------
def _ar_ref(rc, x):
    y = x.clone()
    if rc.world > 1:
        dist.all_reduce(y)
    return y


register(OpSpec(
    name="allreduce", problem_ids=(1,), group="collectives", configs=_CFG,
    make_inputs=lambda rc, cfg: (_fill(rc, cfg),),
    reference=_ar_ref,
    ours=lambda rc, x: rc.comm.all_reduce(x),
    cost=lambda cfg, W: Cost(nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (W - 1) / max(W, 1) * (1 if W > 1 else 0),
                             hbm_bytes=2 * cfg["m"] * cfg["n"] * 2),
    doc="sum all-reduce: one-shot P2P below 512 KiB, NVLS multimem above, two-shot without multicast"))


# ---- all-gather ------------------------------------------------------------------------------
def _ag_ref(rc, x):
    out = torch.empty((rc.world, *x.shape), dtype=x.dtype, device=x.device)
    if rc.world > 1:
        dist.all_gather_into_tensor(out.view(rc.world * x.shape[0], *x.shape[1:]), x)
    else:
        out[0] = x
    return out


register(OpSpec(
    name="allgather", problem_ids=(2, 34), group="collectives", configs=_CFG,
    make_inputs=lambda rc, cfg: (_fill(rc, cfg),),
    reference=_ag_ref,
    ours=lambda rc, x: rc.comm.all_gather(x),
    cost=lambda cfg, W: Cost(nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (W - 1), hbm_bytes=(W + 1) * cfg["m"] * cfg["n"] * 2)))


# ---- broadcast / reduce / scatter / gather -----------------------------------------------------
def _bc_ref(rc, x, src):
    y = x.clone()
    if rc.world > 1:
        dist.broadcast(y, src=src)
    return y


register(OpSpec(
    name="broadcast", problem_ids=(3,), group="collectives", configs=_CFG,
    make_inputs=lambda rc, cfg: (_fill(rc, cfg), 0),
    reference=_bc_ref,
    ours=lambda rc, x, src: rc.comm.broadcast(x, src=src),
    cost=lambda cfg, W: Cost(nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (1 if W > 1 else 0))))


def _reduce_ref(rc, x, dst):
    # non-root ranks return their input unchanged (NCCL leaves their buffer unspecified)
    y = x.clone()
    if rc.world > 1:
        dist.reduce(y, dst=dst)
    return y if rc.rank == dst else x


register(OpSpec(
    name="reduce", problem_ids=(4,), group="collectives", configs=_CFG,
    make_inputs=lambda rc, cfg: (_fill(rc, cfg), 0),
    reference=_reduce_ref,
    ours=lambda rc, x, dst: rc.comm.reduce(x, dst=dst),
    cost=lambda cfg, W: Cost(nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (W - 1))))


def _scatter_ref(rc, x, src):
    out = torch.empty_like(x[0])
    if rc.world > 1:
        dist.scatter(out, [c.contiguous() for c in x.unbind(0)] if rc.rank == src else None, src=src)
    else:
        out.copy_(x[0])
    return out


register(OpSpec(
    name="scatter", problem_ids=(5,), group="collectives", configs=_CFG,
    make_inputs=lambda rc, cfg: (_fill(rc, cfg, rc.world) + torch.arange(rc.world, device=rc.device, dtype=rc.dtype).view(-1, 1, 1), 0),
    reference=_scatter_ref,
    ours=lambda rc, x, src: rc.comm.scatter(x, src=src),
    cost=lambda cfg, W: Cost(nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (W - 1))))


def _gather_ref(rc, x, dst):
    if rc.world == 1:
        return x.unsqueeze(0).clone()
    lst = [torch.empty_like(x) for _ in range(rc.world)] if rc.rank == dst else None
    dist.gather(x, lst, dst=dst)
    return torch.stack(lst) if rc.rank == dst else x


register(OpSpec(
    name="gather", problem_ids=(6,), group="collectives", configs=_CFG,
    make_inputs=lambda rc, cfg: (_fill(rc, cfg), 0),
    reference=_gather_ref,
    ours=lambda rc, x, dst: rc.comm.gather(x, dst=dst),
    cost=lambda cfg, W: Cost(nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (W - 1))))


# ---- reduce-scatter / all-to-all ---------------------------------------------------------------
def _rs_ref(rc, x):
    out = torch.empty((x.shape[0] // rc.world, *x.shape[1:]), dtype=x.dtype, device=x.device)
    if rc.world > 1:
        dist.reduce_scatter_tensor(out, x)
    else:
        out.copy_(x)
    return out


register(OpSpec(
    name="reducescatter", problem_ids=(7,), group="collectives", configs=_CFG,
    make_inputs=lambda rc, cfg: (_fill(rc, cfg, rc.world).reshape(rc.world * cfg["m"], cfg["n"]),),
    reference=_rs_ref,
    ours=lambda rc, x: rc.comm.reduce_scatter(x),
    cost=lambda cfg, W: Cost(nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (W - 1))))


def _a2a_ref(rc, x):
    out = torch.empty_like(x)
    if rc.world > 1:
        dist.all_to_all_single(out, x)
    else:
        out.copy_(x)
    return out


def _a2a_inputs(rc, cfg):
    # chunk d of rank r carries the value 10 r + d, so a misrouted chunk is recognisable
    x = torch.empty((rc.world, cfg["m"], cfg["n"]), device=rc.device, dtype=rc.dtype)
    for d in range(rc.world):
        x[d] = float(10 * rc.rank + d)
    return (x,)


register(OpSpec(
    name="alltoall", problem_ids=(8,), group="collectives", configs=_CFG,
    make_inputs=_a2a_inputs, reference=_a2a_ref,
    ours=lambda rc, x: rc.comm.all_to_all(x),
    cost=lambda cfg, W: Cost(nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (W - 1))))


# ---- the no-GPU plumbing configuration: AR -> AG -> RS on fp32 (4096,) -------------------------
def _plumbing_inputs(rc, cfg):
    g = torch.Generator(device=rc.device).manual_seed(rc.rank)
    return (torch.randn(cfg["n"], device=rc.device, dtype=torch.float32, generator=g),)


def _plumbing_ref(rc, x):
    ar = x.clone()
    dist.all_reduce(ar)
    ag = torch.empty(rc.world * x.numel(), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(ag, ar)
    rs = torch.empty(ag.numel() // rc.world, dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(rs, ag)
    return {"allreduce": ar, "allgather": ag, "reducescatter": rs}


def _plumbing_ours(rc, x):
    ar = rc.comm.all_reduce(x)
    ag = rc.comm.all_gather(ar).reshape(-1)
    rs = rc.comm.reduce_scatter(ag)
    return {"allreduce": ar, "allgather": ag, "reducescatter": rs}


register(OpSpec(
    name="plumbing", problem_ids=(1, 2, 7), group="collectives", configs={"default": {"n": 4096}},
    make_inputs=_plumbing_inputs, reference=_plumbing_ref, ours=_plumbing_ours, atol=1e-5, rtol=1e-5,
    doc="sum all-reduce, then all-gather, then reduce-scatter (chunk n*W/W) of an fp32 vector seeded by rank"))
