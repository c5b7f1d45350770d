"""Sequence-parallel (Ulysses) workloads: sequence <-> head exchanges and the attention block built on them.

Reference workloads covered: reference/33_ulysses_all_to_all_tensor_primitive.py,
reference/35_ulysses_all_gather_variable_primitive.py, reference/36_ulysses_gather_seq_scatter_heads.py,
reference/37_ulysses_gather_heads_scatter_seq.py, reference/38_ulysses_gather_seq_scatter_heads_qkv.py,
reference/39_ulysses_attention_e2e.py. The reference implements every exchange as chunk -> list all-to-all -> cat
(three passes over the data plus the transfer); ours is one launch whose peer loads land the data in its final layout.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..harness.roofline import Cost
from ..utils.ragged import Ragged, compact_padded, permute_segments_padded
from .registry import OpSpec, RunCtx, register


def _a2a_ref(x: torch.Tensor, scatter_dim: int, gather_dim: int, W: int) -> torch.Tensor:
    if W == 1:
        return x.contiguous()
    ins = [t.contiguous() for t in torch.tensor_split(x, W, scatter_dim)]
    outs = [torch.empty_like(ins[0]) for _ in range(W)]
    dist.all_to_all(outs, ins) if dist.get_backend() != "gloo" else _gloo_all_to_all(outs, ins)
    return torch.cat(outs, dim=gather_dim).contiguous()


def _gloo_all_to_all(outs, ins):
    """gloo has no all_to_all: W broadcasts of the stacked chunks, each rank keeps its column."""
    W, r = dist.get_world_size(), dist.get_rank()
    stacked = torch.stack(ins)
    for src in range(W):
        buf = stacked.clone() if src == r else torch.empty_like(stacked)
        dist.broadcast(buf, src)
        outs[src].copy_(buf[r])


def _pad_to(x: torch.Tensor, dim: int, W: int) -> torch.Tensor:
    rem = x.shape[dim] % W
    if rem == 0:
        return x
    shape = list(x.shape)
    shape[dim] = W - rem
    return torch.cat([x, torch.zeros(shape, dtype=x.dtype, device=x.device)], dim=dim)


# ---- 33: all-to-all tensor primitive (split dim 0, concatenate dim 1) ----------------------------
def _p33_inputs(rc: RunCtx, cfg):
    return (rc.randn(cfg["m"], cfg["n"]), 0, 1)


register(OpSpec(name="ulysses_all_to_all", problem_ids=(33,), group="ulysses",
                configs={"default": {"m": 1024, "n": 1024}, "small": {"m": 32, "n": 16}},
                make_inputs=_p33_inputs,
                reference=lambda rc, x, sd, gd: _a2a_ref(x, sd, gd, rc.world),
                ours=lambda rc, x, sd, gd: rc.comm.all_to_all_permute(x, sd, gd), atol=0.0, rtol=0.0,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (W - 1) / max(W, 1))))


# ---- 35: variable-size all-gather -----------------------------------------------------------------
def _p35_inputs(rc: RunCtx, cfg):
    rows = cfg["m"] - (rc.rank * cfg.get("shrink", 0))          # ranks may hold different numbers of rows
    return (rc.randn(max(rows, 1), cfg["n"]), 0, cfg["m"])      # the last entry: an upper bound of the rows of any rank


def _p35_ref(rc, x, gather_dim, cap=None):
    W = rc.world
    if W == 1:
        return x.contiguous()
    size = torch.tensor(list(x.shape), dtype=torch.int64, device=x.device)
    sizes = [torch.zeros_like(size) for _ in range(W)]
    dist.all_gather(sizes, size)
    parts = [torch.empty(torch.Size(s.tolist()), dtype=x.dtype, device=x.device) for s in sizes]
    if len({tuple(s.tolist()) for s in sizes}) == 1:
        dist.all_gather(parts, x.contiguous())
    else:                                                       # uneven sizes: one broadcast per member
        for src in range(W):
            if src == rc.rank:
                parts[src].copy_(x)
            dist.broadcast(parts[src], src)
    return torch.cat(parts, dim=gather_dim).contiguous()


def _p35_ours(rc, x, gather_dim, cap):
    """The row counts travel as device data next to the payload (padded to the capacity ``cap`` that the configuration
    gives), and the valid rows are brought together by a gather through computed indices, so no size comes back to the host:
    the result is a ``Ragged`` buffer whose length stays on the device."""
    W = rc.world
    if W == 1:
        return x.contiguous()
    xm = x.movedim(gather_dim, 0).contiguous()
    padded = torch.zeros((cap, *xm.shape[1:]), dtype=x.dtype, device=x.device)
    padded[:xm.shape[0]] = xm
    hdr = torch.tensor([xm.shape[0]], dtype=torch.int64, device=x.device)      # host-known shape -> device, no read-back
    counts = rc.comm.all_gather(hdr).view(-1)
    rows, total = compact_padded(rc.comm.all_gather(padded), counts)
    return Ragged(rows.movedim(0, gather_dim), total, dim=gather_dim)


register(OpSpec(name="ulysses_all_gather_variable", problem_ids=(35,), group="ulysses",
                configs={"default": {"m": 1024, "n": 1024, "shrink": 0}, "uneven": {"m": 512, "n": 256, "shrink": 8},
                         "small": {"m": 32, "n": 16, "shrink": 1}},
                make_inputs=_p35_inputs, reference=_p35_ref, ours=_p35_ours, atol=0.0, rtol=0.0,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (W - 1))))


# ---- 36 / 37: gather sequence + scatter heads and its inverse ------------------------------------
def _attn_dims(cfg, W):
    return cfg["b"], cfg["t"], cfg["heads"] * (W if cfg.get("heads_per_rank") else 1), cfg["d"]


def _p36_inputs(rc: RunCtx, cfg):
    B, T, H, D = _attn_dims(cfg, rc.world)
    return (rc.randn(B, T, H, D), 1, 2, int(cfg.get("unpadded", 0)))


def _unpad(x, seq_dim, unpadded, W):
    if unpadded and unpadded % W != 0:
        return x.narrow(seq_dim, 0, unpadded).contiguous()
    return x


register(OpSpec(name="ulysses_gather_seq_scatter_heads", problem_ids=(36,), group="ulysses",
                configs={"default": {"b": 16, "t": 16, "heads": 8, "d": 64}, "small": {"b": 2, "t": 4, "heads": 8, "d": 8},
                         "large": {"b": 1, "t": 4096, "heads": 32, "d": 128}},
                make_inputs=_p36_inputs,
                reference=lambda rc, x, sd, hd, unp: _unpad(_a2a_ref(x, hd, sd, rc.world), sd, unp, rc.world),
                ours=lambda rc, x, sd, hd, unp: _unpad(rc.comm.all_to_all_permute(x, hd, sd), sd, unp, rc.world),
                atol=0.0, rtol=0.0,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["b"] * cfg["t"] * cfg["heads"] * cfg["d"] * 2 * (W - 1) / max(W, 1))))


def _p37_inputs(rc: RunCtx, cfg):
    B, T, H, D = _attn_dims(cfg, rc.world)
    return (rc.randn(B, T, H, D), 1, 2)


register(OpSpec(name="ulysses_gather_heads_scatter_seq", problem_ids=(37,), group="ulysses",
                configs={"default": {"b": 16, "t": 16, "heads": 8, "d": 64}, "small": {"b": 2, "t": 5, "heads": 2, "d": 8},
                         "large": {"b": 1, "t": 32768, "heads": 4, "d": 128}},
                make_inputs=_p37_inputs,
                reference=lambda rc, x, sd, hd: _a2a_ref(_pad_to(x, sd, rc.world), sd, hd, rc.world),
                ours=lambda rc, x, sd, hd: rc.comm.all_to_all_permute(_pad_to(x, sd, rc.world), sd, hd),
                atol=0.0, rtol=0.0,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["b"] * cfg["t"] * cfg["heads"] * cfg["d"] * 2 * (W - 1) / max(W, 1))))


# ---- 38: packed-QKV variant -------------------------------------------------------------------------
def _p38_inputs(rc: RunCtx, cfg):
    B, T, H, D = _attn_dims(cfg, rc.world)
    return (rc.randn(B, T, 3 * H * D), 1)


def _p38(rc, qkv, seq_dim, a2a):
    """[B, T, 3*P] -> view [B, T, 3, P] -> scatter P, gather T -> [B, T*W, 3*P/W] (q, k, v stay interleaved per token)."""
    W = rc.world
    B, T, P3 = qkv.shape
    x = a2a(qkv.view(B, T, 3, P3 // 3), 3, seq_dim)
    return x.reshape(B, T * W, P3 // W)


register(OpSpec(name="ulysses_gather_seq_scatter_heads_qkv", problem_ids=(38,), group="ulysses",
                configs={"default": {"b": 16, "t": 16, "heads": 8, "d": 64}, "small": {"b": 2, "t": 4, "heads": 8, "d": 8}},
                make_inputs=_p38_inputs,
                reference=lambda rc, qkv, sd: _p38(rc, qkv, sd, lambda x, s, g: _a2a_ref(x, s, g, rc.world)),
                ours=lambda rc, qkv, sd: _p38(rc, qkv, sd, lambda x, s, g: rc.comm.all_to_all_permute(x, s, g)),
                atol=0.0, rtol=0.0,
                cost=lambda cfg, W: Cost(nvlink_bytes=3 * cfg["b"] * cfg["t"] * cfg["heads"] * cfg["d"] * 2 * (W - 1) / max(W, 1))))


# ---- 39: attention block end to end -----------------------------------------------------------------
def _p39_inputs(rc: RunCtx, cfg):
    B, S, H, D = cfg["b"], cfg["s_local"], cfg["heads"], cfg["d"]
    hid = H * D
    std = 1.0 / math.sqrt(hid)
    return (rc.randn(B, S, hid), rc.randn(3 * hid, hid, std=std, shared=True, salt=1), rc.randn(hid, hid, std=std, shared=True, salt=2),
            H, bool(cfg["causal"]))


def _sdpa_math(q, k, v, scale, causal):
    """q, k, v: [B, S, H, D] -> [B, S, H, D], fp32 softmax."""
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    if causal:
        S = s.shape[-1]
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=s.device), 1), float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v.float()).to(q.dtype)


def _p39_ref(rc, hidden, w_qkv, w_o, H, causal):
    W = rc.world
    B, S, hid = hidden.shape
    D = hid // H
    qkv = F.linear(hidden, w_qkv).view(B, S, 3, H, D)
    q, k, v = (qkv[:, :, i].contiguous() for i in range(3))
    q, k, v = (_a2a_ref(t, 2, 1, W) for t in (q, k, v))
    o = _sdpa_math(q, k, v, D ** -0.5, causal)
    o = _a2a_ref(o, 1, 2, W)
    return F.linear(o.reshape(B, S, hid), w_o)


def _p39_ours(rc, hidden, w_qkv, w_o, H, causal):
    """QKV projection on the tcgen05 GEMM, ONE exchange for q, k and v together (the reference does two, after a
    stack/reshape copy), flash attention on the local heads, one exchange back, output projection."""
    W = rc.world
    B, S, hid = hidden.shape
    D = hid // H
    cuda = rc.dist.is_cuda and hidden.dtype == torch.bfloat16
    if cuda:
        from ..ops import gemm_bf16
        from ..ops.attention import flash_attn_fwd

        lin = lambda a, w: gemm_bf16(a.reshape(-1, a.shape[-1]), w).view(*a.shape[:-1], w.shape[0])  # noqa: E731
    else:
        lin = F.linear
    qkv = lin(hidden, w_qkv).view(B, S, 3, H, D)
    qkv = rc.comm.all_to_all_permute(qkv, 3, 1)                 # [B, S*W, 3, H/W, D]
    q, k, v = (qkv[:, :, i].contiguous() for i in range(3))
    if cuda and D in (64, 128):
        o = flash_attn_fwd(q, k, v, causal=causal, scale=D ** -0.5, return_lse=False)[0]
    else:
        o = _sdpa_math(q, k, v, D ** -0.5, causal)
    o = rc.comm.all_to_all_permute(o, 1, 2)                     # [B, S, H, D]
    return lin(o.reshape(B, S, hid), w_o)


def _p39_cost(cfg, W):
    B, S, H, D = cfg["b"], cfg["s_local"], cfg["heads"], cfg["d"]
    hid, St = H * D, cfg["s_local"] * W
    flops = 2.0 * B * S * hid * 4 * hid + 4.0 * B * St * St * D * (H / max(W, 1)) * (0.5 if cfg["causal"] else 1.0)
    return Cost(flops=flops, nvlink_bytes=4 * B * S * hid * 2 * (W - 1) / max(W, 1))


register(OpSpec(name="ulysses_attention", problem_ids=(39,), group="ulysses",
                configs={"default": {"b": 16, "s_local": 2, "heads": 8, "d": 64, "causal": 0},
                         "small": {"b": 1, "s_local": 8, "heads": 8, "d": 16, "causal": 1},
                         "large": {"b": 1, "s_local": 4096, "heads": 32, "d": 128, "causal": 1}},
                make_inputs=_p39_inputs, reference=_p39_ref, ours=_p39_ours, atol=3e-2, rtol=3e-2, cost=_p39_cost))
