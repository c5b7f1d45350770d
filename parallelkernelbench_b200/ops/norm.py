"""RMSNorm kernels (csrc/kernels/norm.cu).

``sum_rmsnorm`` is the consumer end of a reduce-scatter: it adds the per-source partial buffers in
a fixed order, scales, and normalises, so the reduced tensor is never stored un-normalised
(reference behaviour: reference/45_reducescatter_fused_rmsnorm.py:23-29,
reference/18_tp_rms_norm.py:9-19).
"""
from __future__ import annotations

import torch

from .. import _native as nv


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6, out: torch.Tensor | None = None) -> torch.Tensor:
    if x.dtype != torch.bfloat16 or gamma.dtype != torch.bfloat16:
        raise TypeError("rmsnorm expects bf16 input and gain")
    cols = x.shape[-1]
    x2 = x.contiguous().view(-1, cols)
    if out is None:
        out = torch.empty_like(x2)
    nv.check(nv.cuda_lib().pkb_rmsnorm_bf16(nv.ptr(x2), nv.ptr(gamma), nv.ptr(out), x2.shape[0], cols,
                                            nv.c_float(eps), nv.current_stream()), "pkb_rmsnorm_bf16")
    nv.count_launch()
    return out.view(x.shape)


def sum_rmsnorm(parts: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6, scale: float = 1.0,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """``parts`` is ``[nsrc, rows, cols]`` (bf16 or fp32, contiguous); returns bf16 ``[rows, cols]``."""
    if parts.dim() != 3 or not parts.is_contiguous():
        raise ValueError("parts must be a contiguous [nsrc, rows, cols] tensor")
    nsrc, rows, cols = parts.shape
    if out is None:
        out = torch.empty((rows, cols), dtype=torch.bfloat16, device=parts.device)
    nv.check(nv.cuda_lib().pkb_sum_rmsnorm(nv.ptr(parts), nv.c_ll(rows * cols), nsrc,
                                           1 if parts.dtype == torch.float32 else 0, nv.ptr(gamma), nv.ptr(out),
                                           rows, cols, nv.c_float(scale), nv.c_float(eps), nv.current_stream()),
             "pkb_sum_rmsnorm")
    nv.count_launch()
    return out
