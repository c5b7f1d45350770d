"""Quantised communication workloads: the bytes on the wire are fp8 / int8 plus scales, dequantised
(and accumulated) where they arrive.

Reference workloads covered: reference/19_blocked_fp8_quantize.py, reference/20_blocked_fp8_dequantize.py,
reference/44_quantized_grad_allreduce.py, reference/52_fp8_reduce_scatter_grads.py,
reference/53_fp8_allgather_params.py.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..harness.roofline import Cost
from .registry import OpSpec, RunCtx, register

FP8_MAX = 448.0


def _q1x128_torch(x: torch.Tensor):
    xb = x.float().reshape(-1, 128)
    s = xb.abs().amax(-1) / FP8_MAX
    s = torch.where(s == 0, torch.ones_like(s), s)
    y = (xb / s.unsqueeze(-1)).to(torch.float8_e4m3fn)
    return y.view(torch.uint8).reshape(x.shape), s.reshape(*x.shape[:-1], x.shape[-1] // 128)


def _quant(rc: RunCtx, x):
    if rc.dist.is_cuda:
        from ..ops import fp8_quantize_1x128

        return fp8_quantize_1x128(x)
    return _q1x128_torch(x)


# ---- 19: 1x128 fp8 quantise, then all-gather of payload and scales -------------------------------
def _q19_ref(rc, x, block):
    y, s = _q1x128_torch(x)
    if rc.world == 1:
        return y.unsqueeze(0), s.unsqueeze(0)
    ys = [torch.empty_like(y) for _ in range(rc.world)]
    ss = [torch.empty_like(s) for _ in range(rc.world)]
    dist.all_gather(ys, y)
    dist.all_gather(ss, s)
    return torch.stack(ys), torch.stack(ss)


def _q19_ours(rc, x, block):
    import os

    if rc.dist.is_cuda and rc.world > 1 and x.dtype == torch.bfloat16 and os.environ.get("PKB_UNFUSED_PUSH") != "1":
        # quantise and gather in one launch: payload and scales go from the quantising thread to every rank's gathered buffers
        from ..ops.fused_push import Fp8QuantAllGather

        key = ("q19", tuple(x.shape))
        if key not in rc.cache:
            rc.cache[key] = Fp8QuantAllGather(rc.comm.group(), tuple(x.shape))
        y, s = rc.cache[key](x)
        return y.clone(), s.clone()
    y, s = _quant(rc, x)
    if rc.world == 1:
        return y.unsqueeze(0), s.unsqueeze(0)
    return rc.comm.all_gather(y), rc.comm.all_gather(s)


def _fp8_payload_close(a, b):
    return (a.view(torch.float8_e4m3fn).float() - b.view(torch.float8_e4m3fn).float()).abs()


register(OpSpec(name="fp8_quantize_allgather", problem_ids=(19,), group="quant",
                configs={"default": {"m": 1024, "n": 1024}, "small": {"m": 8, "n": 256}},
                make_inputs=lambda rc, cfg: (rc.randn(cfg["m"], cfg["n"]), 128),
                reference=_q19_ref, ours=_q19_ours, atol=33.0, rtol=0.0,   # payload bytes compared as integers: <= 1 code apart
                cost=lambda cfg, W: Cost(hbm_bytes=cfg["m"] * cfg["n"] * 3, nvlink_bytes=cfg["m"] * cfg["n"] * (1 + 4 / 128) * (W - 1))))


# ---- 20: fp8 payload + scales exchanged by all-to-all, dequantised to fp32 -----------------------
def _dq20_inputs(rc, cfg):
    x = rc.randn(rc.world, cfg["m"], cfg["n"], dtype=torch.float32)
    y, s = _q1x128_torch(x)
    return (y, s, 128)


def _dq20_ref(rc, y, s, block):
    full = (y.view(torch.float8_e4m3fn).float().reshape(-1, block) * s.reshape(-1, 1)).reshape(y.shape)
    out = torch.empty_like(full)
    if rc.world > 1:
        dist.all_to_all_single(out, full.contiguous())
    else:
        out.copy_(full)
    return out


def _dq20_ours(rc, y, s, block):
    # ship 1 byte per element (+ scales) instead of 4, dequantise after the exchange
    if rc.world > 1:
        y, s = rc.comm.all_to_all(y.contiguous()), rc.comm.all_to_all(s.contiguous())
    if rc.dist.is_cuda:
        from ..ops import fp8_dequantize_1x128

        return fp8_dequantize_1x128(y, s, torch.float32)
    return (y.view(torch.float8_e4m3fn).float().reshape(-1, block) * s.reshape(-1, 1)).reshape(y.shape)


register(OpSpec(name="fp8_dequantize_alltoall", problem_ids=(20,), group="quant",
                configs={"default": {"m": 1024, "n": 1024}, "small": {"m": 4, "n": 256}},
                make_inputs=_dq20_inputs, reference=_dq20_ref, ours=_dq20_ours, atol=1e-5, rtol=1e-5,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["m"] * cfg["n"] * (1 + 4 / 128) * (W - 1))))


# ---- 44: block-int8 gradient all-reduce (mean) -----------------------------------------------------
def _int8_round_trip(x, block):
    n = x.numel()
    flat = x.reshape(-1).float()
    pad = (-n) % block
    if pad:
        flat = torch.nn.functional.pad(flat, (0, pad))
    xv = flat.view(-1, block)
    s = xv.abs().amax(1).clamp(min=1e-8) / 127.0
    q = (xv / s.unsqueeze(1)).round().clamp(-127, 127)
    return (q * s.unsqueeze(1)).reshape(-1)[:n], q.to(torch.int8).reshape(-1)[:n], s


def _q44_ref(rc, g, block):
    rec, _, _ = _int8_round_trip(g, block)
    if rc.world > 1:
        dist.all_reduce(rec)
    return (rec / rc.world).to(g.dtype).reshape(g.shape)


def _q44_ours(rc, g, block):
    W = rc.world
    if rc.dist.is_cuda:
        from ..ops.quant import dequant_sum, int8_quantize_block

        q, s = int8_quantize_block(g, block)
        if W > 1:
            q, s = rc.comm.all_gather(q), rc.comm.all_gather(s)       # 1 byte per element on the wire
        else:
            q, s = q.unsqueeze(0), s.unsqueeze(0)
        return dequant_sum(q.view(torch.uint8), s, "int8_block", block, 1.0 / W, torch.float32).to(g.dtype).reshape(g.shape)
    rec, q, s = _int8_round_trip(g, block)
    if W > 1:
        qa, sa = rc.comm.all_gather(q), rc.comm.all_gather(s)
        n = g.numel()
        pad = (-n) % block
        acc = torch.zeros(n + pad)
        for w in range(W):
            acc += (torch.nn.functional.pad(qa[w].float(), (0, pad)).view(-1, block) * sa[w].unsqueeze(1)).reshape(-1)
        rec = acc[:n]
    return (rec / W).to(g.dtype).reshape(g.shape)


register(OpSpec(name="int8_grad_allreduce", problem_ids=(44,), group="quant",
                configs={"default": {"n": 1 << 20, "block": 128}, "small": {"n": 1000, "block": 128}},
                make_inputs=lambda rc, cfg: (rc.randn(cfg["n"], dtype=torch.float32), cfg["block"]),
                reference=_q44_ref, ours=_q44_ours, atol=1e-4, rtol=1e-4,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["n"] * (1 + 4 / cfg["block"]) * (W - 1))))


# ---- 52 / 53: delayed-scaling fp8 reduce-scatter of gradients / all-gather of parameters ----------
def _delayed_scale(x, hist):
    cur = x.abs().max().to(torch.float32)
    new_hist = torch.roll(hist, shifts=-1, dims=0)
    new_hist[-1] = cur
    return new_hist.max().clamp(min=1e-12).to(torch.float32) / FP8_MAX, new_hist


def _rt(x, scale):
    return ((x.float() / scale).to(torch.float8_e4m3fn).float() * scale).to(x.dtype)


def _fp8rs_inputs(rc, cfg):
    return (rc.randn(rc.world * cfg["shard"]), (rc.rand(16, salt=1) * 4).float())


def _fp8rs_ref(rc, g, hist):
    scale, new_hist = _delayed_scale(g, hist)
    rec = _rt(g, scale)
    out = g.new_empty(g.numel() // rc.world)
    if rc.world > 1:
        dist.reduce_scatter_tensor(out, rec.contiguous())
    else:
        out.copy_(rec)
    return out / rc.world, new_hist


def _fp8rs_ours(rc, g, hist):
    W = rc.world
    scale, new_hist = _delayed_scale(g, hist)
    if rc.dist.is_cuda:
        from ..ops.quant import dequant_sum, fp8_quantize_scaled

        q = fp8_quantize_scaled(g, scale).view(W, -1)
        if W > 1:
            q = rc.comm.all_to_all(q.contiguous())                    # fp8 slices travel, 1 byte per element
            scales = rc.comm.all_gather(scale.reshape(1)).reshape(W)
        else:
            scales = scale.reshape(1)
        return dequant_sum(q, scales, "fp8_tensor", 128, 1.0 / W, torch.float32).to(g.dtype), new_hist
    rec = _rt(g, scale).float().view(W, -1)
    out = rc.comm.reduce_scatter(rec.reshape(-1).contiguous()) if W > 1 else rec.reshape(-1)
    return (out / W).to(g.dtype), new_hist


register(OpSpec(name="fp8_reduce_scatter_grads", problem_ids=(52,), group="quant",
                configs={"default": {"shard": 4096}, "large": {"shard": 1 << 22}},
                make_inputs=_fp8rs_inputs, reference=_fp8rs_ref, ours=_fp8rs_ours, atol=2e-2, rtol=2e-2,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["shard"] * (W - 1))))


def _fp8ag_ref(rc, p, hist):
    scale, new_hist = _delayed_scale(p, hist)
    rec = _rt(p, scale)
    out = p.new_empty(p.numel() * rc.world)
    if rc.world > 1:
        dist.all_gather_into_tensor(out, rec.contiguous())
    else:
        out.copy_(rec)
    return out, new_hist


def _fp8ag_ours(rc, p, hist):
    W = rc.world
    scale, new_hist = _delayed_scale(p, hist)
    if rc.dist.is_cuda:
        from ..ops.quant import dequant_sum, fp8_quantize_scaled

        q = fp8_quantize_scaled(p, scale)
        if W > 1:
            qa = rc.comm.all_gather(q)                                 # fp8 on the wire
            sa = rc.comm.all_gather(scale.reshape(1)).reshape(W)
        else:
            qa, sa = q.unsqueeze(0), scale.reshape(1)
        # dequantise each shard with its owner's scale (a "sum" over one slice per segment)
        out = torch.cat([dequant_sum(qa[w:w + 1], sa[w:w + 1], "fp8_tensor", 128, 1.0, torch.float32) for w in range(W)])
        return out.to(p.dtype), new_hist
    rec = _rt(p, scale)
    return (rc.comm.all_gather(rec).reshape(-1) if W > 1 else rec), new_hist


register(OpSpec(name="fp8_allgather_params", problem_ids=(53,), group="quant", configs={"default": {"shard": 4096}},
                make_inputs=lambda rc, cfg: (rc.randn(cfg["shard"]), (rc.rand(16, salt=1) * 4).float()),
                reference=_fp8ag_ref, ours=_fp8ag_ours, atol=2e-2, rtol=2e-2,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["shard"] * (W - 1))))
