"""Quantised-wire helpers (csrc/kernels/quant.cu): per-tensor fp8, block int8, dequantise-and-sum."""
from __future__ import annotations

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
