"""PyTorch restatement of the block-scaled fp8 GEMM (oracle of ``ops.gemm_fp8``; runs on CPU).

Quantisation follows the reference's blocked form, ``scale = amax / 448`` with 1 for an all-zero block
(reference: reference/19_blocked_fp8_quantize.py:7-23, reference/20_blocked_fp8_dequantize.py:6-16):
activations carry one scale per row and 128 consecutive K elements, weights one scale per 128 x 128 block.
The product is ``sum_kb sa[m, kb] * sb[n // 128, kb] * (A8[m, kb-block] . B8[n, kb-block])`` in fp32, which
equals the GEMM of the dequantised operands up to fp32 summation order.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

E4M3_MAX = 448.0


def quantize_rows_1x128(x: torch.Tensor):
    """``x[..., K]`` -> (e4m3 bytes as uint8 ``[..., K]``, fp32 scales ``[..., K // 128]``)."""
    if x.shape[-1] % 128 != 0:
        raise ValueError("last dimension must be a multiple of 128")
    xb = x.float().reshape(*x.shape[:-1], x.shape[-1] // 128, 128)
    s = xb.abs().amax(-1) / E4M3_MAX
    s = torch.where(s == 0, torch.ones_like(s), s)
    q = (xb * (1.0 / s).unsqueeze(-1)).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).reshape(x.shape), s


def quantize_weight_128x128(w: torch.Tensor):
    """``w[..., N, K]`` -> (e4m3 bytes as uint8, fp32 scales ``[..., N // 128, K // 128]``)."""
    *lead, N, K = w.shape
    if N % 128 != 0 or K % 128 != 0:
        raise ValueError("N and K must be multiples of 128")
    wb = w.float().reshape(*lead, N // 128, 128, K // 128, 128)
    s = wb.abs().amax(dim=(-3, -1)) / E4M3_MAX
    s = torch.where(s == 0, torch.ones_like(s), s)
    q = (wb * (1.0 / s)[..., :, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).reshape(w.shape), s


def dequantize_rows_1x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    return q.view(torch.float8_e4m3fn).float() * s.float().repeat_interleave(128, dim=-1)[..., :q.shape[-1]]


def dequantize_weight_128x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    full = s.float().repeat_interleave(128, dim=-2).repeat_interleave(128, dim=-1)
    return q.view(torch.float8_e4m3fn).float() * full


def gemm_fp8_blockscaled_ref(a8: torch.Tensor, sa: torch.Tensor, w8: torch.Tensor, sb: torch.Tensor,
                             offsets: torch.Tensor | None = None, epilogue: str = "none", alpha: float = 1.0):
    """Dense (``w8 [N, K]``) or grouped (``w8 [G, N, K]`` with int ``offsets [G + 1]``) product in fp32.

    ``epilogue``: ``"none"`` -> bf16 ``[M, N]``; ``"swiglu"`` over interleaved (gate, up) columns -> bf16
    ``[M, N // 2]``; ``"swiglu_quant"`` -> (e4m3 bytes ``[M, N // 2]``, fp32 scales ``[M, N // 256]``) of the
    bf16-rounded SwiGLU output. Rows outside every group are zero."""
    a = dequantize_rows_1x128(a8, sa[..., :a8.shape[-1] // 128])
    w = dequantize_weight_128x128(w8, sb)
    if offsets is None:
        acc = a @ w.t()
    else:
        acc = torch.zeros((a.shape[0], w.shape[1]), dtype=torch.float32, device=a.device)
        off = offsets.tolist()
        for e in range(w.shape[0]):
            lo, hi = off[e], min(off[e + 1], a.shape[0])
            if hi > lo:
                acc[lo:hi] = a[lo:hi] @ w[e].t()
    acc = acc * alpha
    if epilogue == "none":
        return acc.to(torch.bfloat16)
    h = (F.silu(acc[:, 0::2]) * acc[:, 1::2]).to(torch.bfloat16)
    if epilogue == "swiglu":
        return h
    if epilogue == "swiglu_quant":
        return quantize_rows_1x128(h)
    raise ValueError(f"unknown epilogue {epilogue!r}")
