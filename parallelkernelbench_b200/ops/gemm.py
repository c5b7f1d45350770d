"""Dense bf16 GEMM on tcgen05/TMEM (kernel: csrc/include/pkb/gemm_umma.cuh).

Replaces the cuBLAS calls behind ``torch.matmul`` / ``F.linear`` in the reference's tensor-parallel
problems (reference: reference/11_allgather_gemm_AT.py:16, reference/13_gemm_allreduce.py:17,
reference/15_combined_sharded_gemms.py:22-24, reference/16_gemm_reducescatter.py:19).

Operand convention: ``a`` is ``[M, K]`` row-major and ``w`` is ``[N, K]`` row-major (one output
feature per row - the ``torch.nn.Linear`` weight layout), so both operands are K-major and feed
the tensor core through 128-byte-swizzled TMA tiles without a transpose.
"""
from __future__ import annotations

import torch

from .. import _native as nv

EPILOGUES = {"none": 0, "silu": 1, "bias": 2, "bias_silu": 3}


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, *, out: torch.Tensor | None = None,
              bias: torch.Tensor | None = None, epilogue: str = "none", alpha: float = 1.0,
              out_dtype: torch.dtype = torch.bfloat16, block_n: int = 0, num_ctas: int = 0,
              mode: str = "auto") -> torch.Tensor:
    """``out[M, N] = epilogue(alpha * a[M, K] @ w[N, K].T + bias)`` with fp32 accumulation."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise TypeError("gemm_bf16 expects bf16 operands")
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1]:
        raise ValueError(f"shape mismatch: a {tuple(a.shape)} w {tuple(w.shape)} (w must be [N, K])")
    if a.stride(1) != 1 or w.stride(1) != 1:
        raise ValueError("operands must be contiguous along K")
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if out.dtype not in (torch.bfloat16, torch.float32) or out.stride(1) != 1:
        raise ValueError("out must be bf16 or fp32 and contiguous along N")
    if bias is not None:
        epilogue = {"none": "bias", "silu": "bias_silu"}.get(epilogue, epilogue)
        if bias.dtype != torch.bfloat16 or bias.numel() != N:
            raise ValueError("bias must be bf16 [N]")
    lib = nv.cuda_lib()
    if mode == "auto":
        mode = "pair" if (block_n == 0 and M >= 512 and N >= 256) else "single"
    if mode == "pair":
        nv.check(lib.pkb_gemm_bf16_pair(nv.ptr(a), nv.c_ll(a.stride(0)), nv.ptr(w), nv.c_ll(w.stride(0)),
                                        nv.ptr(out), nv.c_ll(out.stride(0)), M, N, K, nv.ptr(bias),
                                        nv.c_float(alpha), EPILOGUES[epilogue],
                                        1 if out.dtype == torch.float32 else 0, num_ctas, nv.current_stream()),
                 "pkb_gemm_bf16_pair")
        nv.count_launch()
        return out
    nv.check(lib.pkb_gemm_bf16(nv.ptr(a), nv.c_ll(a.stride(0)), nv.ptr(w), nv.c_ll(w.stride(0)), nv.ptr(out),
                               nv.c_ll(out.stride(0)), M, N, K, nv.ptr(bias), nv.c_float(alpha),
                               EPILOGUES[epilogue], 1 if out.dtype == torch.float32 else 0, block_n, num_ctas,
                               nv.current_stream()), "pkb_gemm_bf16")
    nv.count_launch()
    return out


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                activation: str = "none") -> torch.Tensor:
    """``F.linear`` on our kernel for inputs of any leading shape."""
    lead = x.shape[:-1]
    y = gemm_bf16(x.reshape(-1, x.shape[-1]), weight, bias=bias, epilogue=activation)
    return y.reshape(*lead, weight.shape[0])


def gemm_bf16_kn(a: torch.Tensor, b: torch.Tensor, *, out: torch.Tensor | None = None, epilogue: str = "none",
                 alpha: float = 1.0, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``a[M, K] @ b[K, N]`` with ``b`` row-major (N contiguous): the tensor core reads B as an
    MN-major operand, so a ``[K, N]`` weight needs no transposed copy."""
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or a.shape[1] != b.shape[0]:
        raise ValueError("gemm_bf16_kn expects bf16 a[M, K] and b[K, N]")
    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("operands must be contiguous along their last dimension")
    M, K = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    nv.check(nv.cuda_lib().pkb_gemm_bf16_bkn(nv.ptr(a), nv.c_ll(a.stride(0)), nv.ptr(b), nv.c_ll(b.stride(0)), nv.ptr(out),
                                             nv.c_ll(out.stride(0)), M, N, K, nv.c_float(alpha), EPILOGUES[epilogue],
                                             1 if out.dtype == torch.float32 else 0, nv.current_stream()),
             "pkb_gemm_bf16_bkn")
    nv.count_launch()
    return out


def gemm_bf16_tn(a_km: torch.Tensor, b_kn: torch.Tensor, *, out: torch.Tensor | None = None, alpha: float = 1.0,
                 out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``a_km.T @ b_kn`` for row-major ``a_km[K, M]`` and ``b_kn[K, N]`` (both MN-major operands): the
    weight-gradient form ``dW = dY.T @ X`` without materialising a transpose."""
    if a_km.dtype != torch.bfloat16 or b_kn.dtype != torch.bfloat16 or a_km.shape[0] != b_kn.shape[0]:
        raise ValueError("gemm_bf16_tn expects bf16 a[K, M] and b[K, N]")
    if a_km.stride(1) != 1 or b_kn.stride(1) != 1:
        raise ValueError("operands must be contiguous along their last dimension")
    K, M = a_km.shape
    N = b_kn.shape[1]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a_km.device)
    nv.check(nv.cuda_lib().pkb_gemm_bf16_tn(nv.ptr(a_km), nv.c_ll(a_km.stride(0)), nv.ptr(b_kn), nv.c_ll(b_kn.stride(0)),
                                            nv.ptr(out), nv.c_ll(out.stride(0)), M, N, K, nv.c_float(alpha),
                                            1 if out.dtype == torch.float32 else 0, nv.current_stream()), "pkb_gemm_bf16_tn")
    nv.count_launch()
    return out
