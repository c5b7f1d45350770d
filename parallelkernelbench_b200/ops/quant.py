"""Quantised-wire helpers (csrc/kernels/quant.cu): per-tensor fp8, block int8, dequantise-and-sum."""
from __future__ import annotations

import ctypes

import torch

from .. import _native as nv

_DT = {torch.bfloat16: 0, torch.float32: 1}


def fp8_quantize_scaled(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """e4m3 payload of ``x / scale`` with ``scale`` a one-element fp32 device tensor."""
    xc = x.contiguous()
    y = torch.empty(xc.shape, dtype=torch.uint8, device=x.device)
    nv.check(nv.cuda_lib().pkb_fp8_quant_scaled(nv.ptr(xc), nv.ptr(scale.to(torch.float32).reshape(1)), nv.ptr(y),
                                                nv.c_ll(xc.numel()), _DT[xc.dtype], nv.current_stream()), "pkb_fp8_quant_scaled")
    nv.count_launch()
    return y


def int8_quantize_block(x: torch.Tensor, block: int):
    xc = x.contiguous().view(-1)
    n = xc.numel()
    y = torch.empty(n, dtype=torch.int8, device=x.device)
    s = torch.empty((n + block - 1) // block, dtype=torch.float32, device=x.device)
    nv.check(nv.cuda_lib().pkb_int8_quant_block(nv.ptr(xc), nv.ptr(y), nv.ptr(s), nv.c_ll(n), block, _DT[xc.dtype],
                                                nv.current_stream()), "pkb_int8_quant_block")
    nv.count_launch()
    return y, s


def dequant_sum(payload: torch.Tensor, scales: torch.Tensor, mode: str, block: int = 128, out_scale: float = 1.0,
                out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``payload`` is ``[W, n]`` bytes; returns ``out_scale * sum_w dequant(payload[w])`` as ``[n]``.
    mode: ``"fp8_tensor"`` (scales ``[W]``), ``"fp8_block"`` / ``"int8_block"`` (scales ``[W, ceil(n/block)]``)."""
    W, n = payload.shape
    pc = payload.contiguous()
    out = torch.empty(n, dtype=out_dtype, device=payload.device)
    m = {"fp8_tensor": 0, "fp8_block": 1, "int8_block": 2}[mode]
    nv.check(nv.cuda_lib().pkb_dequant_sum(nv.ptr(pc), nv.ptr(scales.contiguous().to(torch.float32)), nv.ptr(out), W,
                                           nv.c_ll(n), nv.c_ll(n), m, block, nv.c_float(out_scale), _DT[out_dtype],
                                           nv.current_stream()), "pkb_dequant_sum")
    nv.count_launch()
    return out


def fsdp_adamw_fp8(payload: torch.Tensor, scales: torch.Tensor, p: torch.Tensor, m: torch.Tensor, v: torch.Tensor,
                   q_out: torch.Tensor, s_out: torch.Tensor, *, lr: float, beta1: float, beta2: float, eps: float,
                   weight_decay: float, grad_scale: float, step: int, p_bf16: torch.Tensor | None = None) -> None:
    """Owner side of the fp8 gradient exchange: ``payload`` [W, n] e4m3 bytes + ``scales`` [W, n/128]
    are dequantised, summed, scaled by ``grad_scale`` (1/W), applied with AdamW to the fp32 shard
    ``p, m, v`` in place, and the new weights are written as e4m3 + 1x128 scales into ``q_out, s_out``."""
    W, n = payload.shape
    nv.check(nv.cuda_lib().pkb_fsdp_adamw_fp8(nv.ptr(payload.contiguous()), nv.ptr(scales.contiguous()), W, nv.c_ll(n),
                                              nv.ptr(p), nv.ptr(m), nv.ptr(v), nv.ptr(q_out), nv.ptr(s_out), nv.ptr(p_bf16),
                                              nv.c_float(lr), nv.c_float(beta1), nv.c_float(beta2), nv.c_float(eps),
                                              nv.c_float(weight_decay), nv.c_float(grad_scale), int(step),
                                              nv.current_stream()), "pkb_fsdp_adamw_fp8")
    nv.count_launch()


def clip_grad_norm_(tensors: list[torch.Tensor], max_norm: float, comm=None, group=None, pre_scale: list[float] | None = None):
    """Clip by global L2 norm in place, nothing returns to the host: one launch sums the squares of all tensors, one small
    all-reduce combines the ranks, one launch scales every tensor by ``min(1, max_norm / norm)`` read from device memory.
    ``pre_scale[i]`` multiplies tensor i before it is measured (and the tensor stays scaled), which is how expert-parallel
    gradients enter the norm. Returns the global norm as a device scalar."""
    if not tensors:
        raise ValueError("no tensors")
    dt = tensors[0].dtype
    if dt not in (torch.bfloat16, torch.float32) or any(t.dtype != dt or not t.is_contiguous() for t in tensors):
        raise TypeError("contiguous tensors of one dtype (bf16 or fp32) expected")
    dev = tensors[0].device
    acc = torch.zeros(1, dtype=torch.float32, device=dev)
    lib = nv.cuda_lib()
    code = 0 if dt == torch.bfloat16 else 1

    def pack(chunk, scales):
        n = len(chunk)
        return ((ctypes.c_void_p * n)(*[t.data_ptr() for t in chunk]), (ctypes.c_longlong * n)(*[t.numel() for t in chunk]),
                (ctypes.c_float * n)(*scales), n)

    ps = list(pre_scale) if pre_scale is not None else [1.0] * len(tensors)
    for i in range(0, len(tensors), 8):
        ptrs, ns, sc, n = pack(tensors[i:i + 8], ps[i:i + 8])
        nv.check(lib.pkb_clip_sumsq(ptrs, ns, sc, None, n, code, nv.ptr(acc), nv.current_stream()), "pkb_clip_sumsq")
        nv.count_launch()
    if comm is not None and comm.size(group) > 1:
        acc = comm.all_reduce(acc, group=group)
    norm = torch.empty((), dtype=torch.float32, device=dev)
    for i in range(0, len(tensors), 8):
        ptrs, ns, sc, n = pack(tensors[i:i + 8], ps[i:i + 8])
        nv.check(lib.pkb_clip_scale(ptrs, ns, sc, n, code, nv.ptr(acc), 1, nv.c_float(float(max_norm)), nv.ptr(norm),
                                    nv.current_stream()), "pkb_clip_scale")
        nv.count_launch()
    return norm
