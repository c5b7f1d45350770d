"""Block-scaled fp8 GEMM on tcgen05 (kernel: csrc/include/pkb/gemm_fp8.cuh, launcher csrc/kernels/gemm_fp8.cu).

Operands stay in the form the reference's blocked quantiser produces (reference:
reference/19_blocked_fp8_quantize.py:7-23): e4m3 bytes plus fp32 scales, one per row and 128 K elements for
activations, one per 128 x 128 block for weights. The expert FFN of the MoE layer (reference:
reference/31_fused_moe_fwd.py:104-140) can then run on the received fp8 tokens directly: gate/up GEMM with a
SwiGLU + re-quantise epilogue, down GEMM from the re-quantised activations.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as nv

_EPI = {"none": 0, "swiglu": 1, "swiglu_quant": 2, "row_scatter": 3}


def gemm_fp8_blockscaled(a8: torch.Tensor, sa: torch.Tensor, w8: torch.Tensor, sb: torch.Tensor, *,
                         offsets: torch.Tensor | None = None, epilogue: str = "none", alpha: float = 1.0,
                         out: torch.Tensor | None = None, out_scales: torch.Tensor | None = None, num_ctas: int = 0,
                         row_meta: torch.Tensor | None = None, dest_ptrs: list[int] | None = None, dest_pitch: int = 0):
    """``a8 [M, K]`` uint8 (e4m3 bytes) with ``sa [M, >= K/128]`` fp32; ``w8 [N, K]`` (dense) or ``[G, N, K]``
    (grouped, with int32 device ``offsets [G + 1]``) with ``sb [(G,) N/128, K/128]`` fp32.

    Returns bf16 ``[M, N]`` (``"none"``), bf16 ``[M, N/2]`` (``"swiglu"``, interleaved gate/up rows in ``w8``) or
    the pair (uint8 ``[M, N/2]``, fp32 ``[M, N/256]``) for ``"swiglu_quant"``.

    ``"row_scatter"`` stores bf16 row ``m`` as row ``row_meta[m, 1]`` of the buffer at address ``dest_ptrs[row_meta[m, 0]]``
    (``dest_pitch`` elements per row; the buffers may be peers' symmetric memory) and returns None; ``row_meta`` is an int32
    device tensor ``[>= M, 2]``."""
    if a8.dtype != torch.uint8 or w8.dtype != torch.uint8:
        raise TypeError("operands are e4m3 bytes viewed as uint8")
    if sa.dtype != torch.float32 or sb.dtype != torch.float32:
        raise TypeError("scales are fp32")
    grouped = w8.dim() == 3
    if grouped != (offsets is not None):
        raise ValueError("grouped weights [G, N, K] go with offsets [G + 1], dense weights [N, K] without")
    G = w8.shape[0] if grouped else 0
    N, K = w8.shape[-2], w8.shape[-1]
    M = a8.shape[0]
    if a8.dim() != 2 or a8.shape[1] != K or a8.stride(1) != 1 or not w8.is_contiguous() or not sb.is_contiguous():
        raise ValueError("shape mismatch or non-contiguous operand")
    if K % 128 or N % 128 or a8.stride(0) % 16:
        raise ValueError("K and N must be multiples of 128, the row pitch of a8 a multiple of 16")
    if sa.dim() != 2 or sa.shape[0] < M or sa.shape[1] < K // 128 or sa.stride(1) != 1:
        raise ValueError("sa must be [M, >= K/128] with unit inner stride")
    if tuple(sb.shape) != ((G, N // 128, K // 128) if grouped else (N // 128, K // 128)):
        raise ValueError("sb must hold one scale per 128 x 128 block of w8")
    if grouped and (offsets.dtype != torch.int32 or offsets.numel() != G + 1):
        raise ValueError("offsets must be int32 [G + 1]")
    epi = _EPI[epilogue]
    if epi == 3:
        if row_meta is None or row_meta.dtype != torch.int32 or row_meta.shape[-1] != 2 or row_meta.shape[0] < M or not row_meta.is_contiguous():
            raise ValueError("row_meta must be a contiguous int32 [>= M, 2] device tensor")
        if not dest_ptrs or len(dest_ptrs) > 8 or dest_pitch < N or dest_pitch % 8:
            raise ValueError("row_scatter needs 1..8 destination addresses and a row pitch >= N that is a multiple of 8")
        ptrs = (ctypes.c_ulonglong * len(dest_ptrs))(*dest_ptrs)
        nv.check(nv.cuda_lib().pkb_gemm_fp8_blockscaled(
            nv.ptr(a8), nv.c_ll(a8.stride(0)), nv.ptr(sa), nv.c_ll(sa.stride(0)), nv.ptr(w8), nv.c_ll(K), nv.ptr(sb),
            nv.c_ll(K // 128), nv.ptr(None), nv.c_ll(dest_pitch), nv.ptr(None), nv.c_ll(0), nv.ptr(offsets), G, M, N, K,
            nv.c_float(alpha), epi, num_ctas, nv.ptr(row_meta), ptrs, len(dest_ptrs), nv.current_stream()),
            "pkb_gemm_fp8_blockscaled")
        nv.count_launch()
        return None
    n_out = N if epi == 0 else N // 2
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.uint8 if epi == 2 else torch.bfloat16, device=a8.device)
    if out.shape[1] != n_out or out.stride(1) != 1 or out.dtype != (torch.uint8 if epi == 2 else torch.bfloat16):
        raise ValueError("out has the wrong shape or dtype")
    if epi == 2:
        if N % 256:
            raise ValueError("the re-quantising epilogue needs N % 256 == 0")
        if out_scales is None:
            out_scales = torch.empty((M, N // 256), dtype=torch.float32, device=a8.device)
        if out_scales.dtype != torch.float32 or out_scales.shape[0] < M or out_scales.shape[1] < N // 256 or out_scales.stride(1) != 1:
            raise ValueError("out_scales must be fp32 [M, >= N/256]")
    nv.check(nv.cuda_lib().pkb_gemm_fp8_blockscaled(
        nv.ptr(a8), nv.c_ll(a8.stride(0)), nv.ptr(sa), nv.c_ll(sa.stride(0)), nv.ptr(w8), nv.c_ll(K), nv.ptr(sb),
        nv.c_ll(K // 128), nv.ptr(out), nv.c_ll(out.stride(0)), nv.ptr(out_scales),
        nv.c_ll(out_scales.stride(0) if out_scales is not None else 0), nv.ptr(offsets), G, M, N, K, nv.c_float(alpha), epi,
        num_ctas, nv.ptr(None), None, 0, nv.current_stream()), "pkb_gemm_fp8_blockscaled")
    nv.count_launch()
    return (out, out_scales) if epi == 2 else out
