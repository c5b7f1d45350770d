"""Expert-parallel MoE workloads: token-count exchange, variable all-to-all, the full layer.

Reference workloads covered: reference/26_moe_token_preprocess.py, reference/27_moe_all2all_primitive.py,
reference/28_moe_pre_all2all.py, reference/29_moe_post_all2all.py, reference/30_moe_epgroupgemm_lora_backward.py,
reference/31_fused_moe_fwd.py, reference/32_fused_moe_fwd_lora.py, reference/49_moe_ep_balanced.py,
reference/50_moe_ep_wide.py, reference/51_moe_ep_narrow.py. Every expert has its own weights here
(the reference applies one shared weight triple to all experts).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..harness.roofline import Cost
from ..refs.moe import moe_reference
from ..utils.ragged import Ragged, compact_padded, permute_segments_padded
from .registry import OpSpec, RunCtx, register


# ---- 26: per-expert token counts and the split sizes derived from them ----------------------------
def _cnt_inputs(rc, cfg):
    E = max(cfg["experts"], rc.world) // rc.world * rc.world
    return (rc.randint(0, E, (cfg["tokens"], cfg["topk"]), dtype=torch.int32), E)


def _cnt_ref(rc, sel, E):
    W, r = rc.world, rc.rank
    el = E // W
    counts = torch.bincount(sel.reshape(-1).long(), minlength=E).to(torch.int32)
    allc = torch.empty(W, E, dtype=torch.int32, device=sel.device)
    if W > 1:
        dist.all_gather_into_tensor(allc.view(-1), counts)
    else:
        allc[0] = counts
    return {"input_splits": counts.view(W, el).sum(1), "output_splits": allc[:, r * el:(r + 1) * el].sum(1),
            "tokens_per_local_expert": allc[:, r * el:(r + 1) * el].sum(0)}


def _cnt_ours(rc, sel, E):
    W, r = rc.world, rc.rank
    el = E // W
    if rc.dist.is_cuda:
        from .. import _native as nv

        counts = torch.empty(E, dtype=torch.int32, device=sel.device)
        flat = sel.reshape(-1).contiguous()
        nv.check(nv.cuda_lib().pkb_moe_histogram(nv.ptr(flat), nv.c_ll(flat.numel()), E, nv.ptr(counts), nv.current_stream()))
        nv.count_launch()
    else:
        counts = torch.bincount(sel.reshape(-1).long(), minlength=E).to(torch.int32)
    allc = rc.comm.all_gather(counts) if W > 1 else counts.unsqueeze(0)
    return {"input_splits": counts.view(W, el).sum(1), "output_splits": allc[:, r * el:(r + 1) * el].sum(1),
            "tokens_per_local_expert": allc[:, r * el:(r + 1) * el].sum(0)}


register(OpSpec(name="moe_token_counts", problem_ids=(26,), group="moe", configs={"default": {"tokens": 1024, "topk": 2, "experts": 8}},
                make_inputs=_cnt_inputs, reference=_cnt_ref, ours=_cnt_ours, atol=0, rtol=0))


# ---- 27: variable all-to-all with device-resident split sizes ---------------------------------------
def _a2av_inputs(rc, cfg):
    W = rc.world
    base = cfg["rows"] // W
    counts = torch.tensor([max(0, base + ((rc.rank * 3 + d * 5) % 7) - 3) for d in range(W)], device=rc.device, dtype=torch.int64)
    return (rc.randn(int(counts.sum()), cfg["cols"]), counts, cfg["rows"] + 8 * W)


def _a2av_ref(rc, x, counts, cap):
    W = rc.world
    if W == 1:
        return {"rows": x, "count": counts.sum().reshape(1)}
    allc = torch.empty(W, W, dtype=torch.int64, device=x.device)
    dist.all_gather_into_tensor(allc.view(-1), counts)
    recv = allc[:, rc.rank].tolist()                       # host sync, as in the reference
    out = x.new_empty((sum(recv), x.shape[1]))
    dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=counts.tolist())
    return {"rows": out, "count": torch.tensor([sum(recv)], device=x.device)}


def _a2av_ours(rc, x, counts, cap):
    out, _recv, total = rc.comm.all_to_all_v(x.contiguous(), counts, cap)
    return {"rows": Ragged(out, total), "count": total.reshape(1).to(torch.int64)}    # the length never leaves the device


register(OpSpec(name="alltoall_v", problem_ids=(27,), group="moe", configs={"default": {"rows": 1024, "cols": 1024}, "small": {"rows": 64, "cols": 8}},
                make_inputs=_a2av_inputs, reference=_a2av_ref, ours=_a2av_ours, atol=0, rtol=0,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["rows"] * cfg["cols"] * 2.0 * (W - 1) / max(W, 1))))   # rows leave once


# ---- 30: all-reduce of three small LoRA gradients ----------------------------------------------------
def _lora_inputs(rc, cfg):
    return (rc.randn(8, cfg["n"]), rc.randn(8, cfg["n"], salt=1), rc.randn(cfg["n"], 8, salt=2))


def _lora_ref(rc, a, b, c):
    outs = [t.clone() for t in (a, b, c)]
    if rc.world > 1:
        for t in outs:
            dist.all_reduce(t)
    return tuple(outs)


def _lora_ours(rc, a, b, c):
    flat = rc.comm.all_reduce(torch.cat([a.reshape(-1), b.reshape(-1), c.reshape(-1)]))   # one packed launch
    na, nb = a.numel(), b.numel()
    return flat[:na].view(a.shape), flat[na:na + nb].view(b.shape), flat[na + nb:].view(c.shape)


register(OpSpec(name="lora_grad_allreduce", problem_ids=(30,), group="moe", configs={"default": {"n": 1024}},
                make_inputs=_lora_inputs, reference=_lora_ref, ours=_lora_ours, atol=5e-2, rtol=2e-2))


# ---- the MoE layer -----------------------------------------------------------------------------------
def _experts_for(cfg, W):
    mode = cfg.get("experts_mode", "fixed")
    if mode == "balanced":
        return W
    if mode == "wide":
        return 2 * W
    if mode == "narrow":
        return max(1, W // 2)
    return max(cfg["experts"], W) // W * W


def _ep_members(rc, E):
    """Narrow EP: fewer experts than ranks -> EP groups of E consecutive ranks, replicated W/E times."""
    W = rc.world
    if E >= W:
        return list(range(W))
    g = rc.rank // E
    return list(range(g * E, (g + 1) * E))


def _moe_inputs(rc: RunCtx, cfg):
    W = rc.world
    E = _experts_for(cfg, W)
    members = _ep_members(rc, E)
    ew = len(members)
    el = E // ew
    H, I, T = cfg["hidden"], cfg["inter"], cfg["tokens"]
    std = cfg.get("std", 0.05)
    x = rc.randn(T, H)
    w_router = rc.randn(E, H, shared=True, salt=1, std=std)
    b_router = rc.randn(E, shared=True, salt=2, std=0.1)
    er = members.index(rc.rank)
    g = torch.Generator(device=rc.device).manual_seed(900 + er + 31 * rc.trial)   # same experts in every replica group
    mk = lambda *s: (torch.randn(*s, device=rc.device, generator=g) * std).to(rc.dtype)  # noqa: E731
    wg, wu, wd = mk(el, I, H), mk(el, I, H), mk(el, H, I)
    lora = None
    if cfg.get("lora_rank"):
        r = cfg["lora_rank"]
        lora = [mk(el, r, H), mk(el, I, r), mk(el, r, H), mk(el, I, r), mk(el, r, I), mk(el, H, r)]
    # precision mode: 0 = bf16 on the wire, 1 = e4m3 + 1x128 scales on the wire, 2 = additionally e4m3 experts
    # (128 x 128 block-scaled weights, re-quantised hidden activations)
    fp8 = 2 if cfg.get("fp8_experts") else int(bool(cfg.get("fp8", False)))
    return (x, w_router, b_router, wg, wu, wd, E, cfg["topk"], members, fp8, lora)


def _merge_lora(wg, wu, wd, lora):
    if lora is None:
        return wg, wu, wd
    ga, gb, ua, ub, da, db = lora
    f = lambda w, a, b: (w.float() + torch.bmm(b.float(), a.float())).to(w.dtype)  # noqa: E731
    return f(wg, ga, gb), f(wu, ua, ub), f(wd, da, db)


def _pg_for(rc, members):
    if len(members) == rc.world:
        return None
    key = ("pg", tuple(members))
    if key not in rc.cache:
        # new_group is collective over the whole job: create every replica's group in the same order
        E = len(members)
        for g0 in range(0, rc.world, E):
            pg = dist.new_group(list(range(g0, g0 + E)))
            if g0 == members[0]:
                rc.cache[key] = pg
    return rc.cache[key]


def _moe_ref(rc, x, w_router, b_router, wg, wu, wd, E, k, members, fp8, lora):
    wg, wu, wd = _merge_lora(wg, wu, wd, lora)
    return moe_reference(x, w_router, b_router, wg, wu, wd, E, k, group=_pg_for(rc, members), fp8_dispatch=fp8 >= 1,
                         fp8_experts=fp8 >= 2)


def _moe_ours(rc, x, w_router, b_router, wg, wu, wd, E, k, members, fp8, lora):
    wg, wu, wd = _merge_lora(wg, wu, wd, lora)
    if not rc.dist.is_cuda:
        raise RuntimeError("the MoE layer kernels need a GPU")
    from ..models.moe_layer import EPMoELayer, MoEConfig

    key = ("moe_layer", x.shape, wg.data_ptr(), fp8)
    if key not in rc.cache:
        cfg = MoEConfig(hidden=x.shape[1], inter=wg.shape[1], num_experts=E, top_k=k, tokens_per_rank=x.shape[0],
                        capacity_factor=float(len(members)) if x.shape[0] * k <= 8192 else 2.0, fp8_dispatch=fp8 >= 1,
                        fp8_experts=fp8 >= 2, fused_router=os.environ.get("PKB_FUSED_ROUTER", "1") != "0" and E <= 256,
                        push_combine=os.environ.get("PKB_PUSH_COMBINE") == "1")
        rc.cache[key] = EPMoELayer(rc.comm.group(members), rc.comm, cfg, w_router, wg, wu, wd, router_bias=b_router)
    return rc.cache[key](x)


def _moe_cost(cfg, W):
    T, H, I, k = cfg["tokens"], cfg["hidden"], cfg["inter"], cfg["topk"]
    payload = H * (1 + 4 / 128) if (cfg.get("fp8") or cfg.get("fp8_experts")) else 2 * H
    return Cost(flops=6.0 * T * k * H * I, nvlink_bytes=T * k * (W - 1) / max(W, 1) * max(payload, 2 * H),
                hbm_bytes=3.0 * 2 * H * I * max(cfg.get("experts", 8), W) / W)


_MOE_CFG = {
    "default": {"tokens": 1024, "hidden": 1024, "inter": 128, "experts": 8, "topk": 2},
    "small": {"tokens": 64, "hidden": 128, "inter": 64, "experts": 8, "topk": 2},
    "balanced": {"tokens": 1024, "hidden": 1024, "inter": 128, "experts_mode": "balanced", "experts": 8, "topk": 1},
    "wide": {"tokens": 1024, "hidden": 1024, "inter": 128, "experts_mode": "wide", "experts": 8, "topk": 2},
    "narrow": {"tokens": 1024, "hidden": 1024, "inter": 128, "experts_mode": "narrow", "experts": 8, "topk": 1},
    "fp8": {"tokens": 1024, "hidden": 1024, "inter": 128, "experts": 8, "topk": 2, "fp8": True},
    "lora": {"tokens": 1024, "hidden": 1024, "inter": 128, "experts": 8, "topk": 2, "lora_rank": 8},
    "deepseek": {"tokens": 8192, "hidden": 7168, "inter": 2048, "experts": 256, "topk": 8, "fp8": True, "std": 0.02},
    # e4m3 experts: the hidden activations are re-quantised after the SwiGLU, and a bf16-rounding difference in the value being
    # quantised flips single e4m3 codes (a 6-12 % step of that element), hence the wider absolute gate of these two configs
    "fp8_experts": {"tokens": 1024, "hidden": 1024, "inter": 128, "experts": 8, "topk": 2, "fp8_experts": True, "atol": 0.25},
    "deepseek_fp8_experts": {"tokens": 8192, "hidden": 7168, "inter": 2048, "experts": 256, "topk": 8, "fp8_experts": True,
                             "std": 0.02, "atol": 0.25},
}
register(OpSpec(name="moe_layer", problem_ids=(28, 29, 31, 32, 49, 50, 51), group="moe", configs=_MOE_CFG, make_inputs=_moe_inputs,
                reference=_moe_ref, ours=_moe_ours, atol=1e-1, rtol=3e-2, cost=_moe_cost, ours_needs_cuda=True,
                # receive buffers (capacity factor 2 over tokens * topk rows of `hidden` bytes + scales) and expert outputs in bf16
                heap_gib=lambda cfg, W: max(1.0, float(-(-int(2.0 * cfg["tokens"] * cfg["topk"] * cfg["hidden"] * 5.0) // (1 << 30)) + 1)),
                doc="router -> fp8/bf16 dispatch (P2P push) -> grouped SwiGLU experts -> combine (P2P pull)"))
