"""Fused tensor-parallel GEMM + collective ops (kernels: csrc/kernels/fused_tp.cu).

``AllGatherGemm``    all-gather(x) @ w.T (+SiLU) in one launch: communication CTAs push the shard to
                     the peers while the tcgen05 GEMM consumes row chunks as their flags arrive.
``GemmReduceScatterRMSNorm``  (a @ w.T) reduce-scattered over rows, then RMSNorm, in one launch: the
                     GEMM epilogue stores partial tiles into the owner's receive slots over NVLink.
``GemmAllReduce``    (a @ w.T) summed over the ranks (row-parallel linear) in one launch: the same scatter epilogue,
                     then each rank adds the partial slots of its rows and stores the sums on every rank
                     (``multimem.st`` through the switch, or one P2P store per member), closed by a barrier.
``GemmAllGather``    (a @ w.T) gathered along the output features (column-parallel linear) in one launch: the TMA-store
                     epilogue writes every output tile into the gathered result of every rank.
``GemvAllGather``    decode-time LM head for 1, 2 or 4 tokens: memory-bound GEMV over this rank's vocabulary block, bias and the
                     all-gather of the logits in one launch (16-byte ``multimem.st`` / P2P stores, one closing barrier).

All keep their symmetric buffers between calls (steady-state calls allocate nothing), like the
module-level buffer caches of the reference's example solutions
(reference: kernelgen/solution_new_add_cuda.py:70-84) but owned by an object instead of globals.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as nv
from ..parallel.symm_heap import SymmGroup


class AllGatherGemm:
    def __init__(self, group: SymmGroup, rows: int, k: int, chunk_rows: int = 256, comm_ctas: int = 0):
        if rows % 256 != 0:
            raise ValueError("rows per rank must be a multiple of 256 (one CTA-pair tile)")
        while rows % chunk_rows != 0:
            chunk_rows //= 2
        self.group, self.rows, self.k, self.chunk_rows, self.comm_ctas = group, rows, k, chunk_rows, comm_ctas
        W = group.size
        heap = group.heap
        self.gather = heap.empty((W * rows, k), torch.bfloat16)
        self.flags = heap.empty((W * (rows // chunk_rows),), torch.int32)
        self.flags.local.zero_()
        self.epoch = 0

    @property
    def x_slot(self) -> torch.Tensor:
        """This rank's rows of the gather buffer: fill it directly to skip the local copy."""
        r = self.group.rank_in_group
        return self.gather.local[r * self.rows:(r + 1) * self.rows]

    def __call__(self, x_local: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
                 epilogue: str = "none") -> torch.Tensor:
        W = self.group.size
        if x_local.shape != (self.rows, self.k) or x_local.dtype != torch.bfloat16 or not x_local.is_contiguous():
            raise ValueError("x_local must be a contiguous bf16 [rows, k] tensor")
        if w.dtype != torch.bfloat16 or w.shape[1] != self.k or w.stride(1) != 1:
            raise ValueError("w must be bf16 [N, k], contiguous along k")
        n = w.shape[0]
        if out is None:
            out = torch.empty((W * self.rows, n), dtype=torch.bfloat16, device=x_local.device)
        self.epoch += 1
        nv.check(nv.cuda_lib().pkb_tp_ag_gemm(
            self.group.ref, nv.ptr(x_local), self.rows, self.k, ctypes.c_ulonglong(self.gather.offset),
            ctypes.c_ulonglong(self.flags.offset), self.chunk_rows, ctypes.c_uint(self.epoch), nv.ptr(w),
            nv.c_ll(w.stride(0)), nv.ptr(out), nv.c_ll(out.stride(0)), n, {"none": 0, "silu": 1}[epilogue],
            self.comm_ctas, nv.current_stream()), "pkb_tp_ag_gemm")
        nv.count_launch()
        return out


class GemmReduceScatterRMSNorm:
    def __init__(self, group: SymmGroup, rows_per_rank: int, n: int):
        if rows_per_rank % 256 != 0:
            raise ValueError("rows per rank must be a multiple of 256 (one CTA-pair tile)")
        self.group, self.rows, self.n = group, rows_per_rank, n
        heap = group.heap
        self.recv = heap.empty((group.size, rows_per_rank, n), torch.bfloat16)
        self.done = heap.empty((max(rows_per_rank // 128, 4),), torch.int32)
        self.done.local.zero_()
        self.calls = 0

    def __call__(self, a: torch.Tensor, w: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6,
                 scale: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
        W = self.group.size
        if a.shape[0] != W * self.rows or a.dtype != torch.bfloat16 or a.stride(1) != 1:
            raise ValueError("a must be bf16 [W * rows_per_rank, K]")
        if w.shape != (self.n, a.shape[1]) or w.stride(1) != 1:
            raise ValueError("w must be [N, K]")
        if out is None:
            out = torch.empty((self.rows, self.n), dtype=torch.bfloat16, device=a.device)
        self.calls += 1
        nv.check(nv.cuda_lib().pkb_tp_gemm_rs_rmsnorm(
            self.group.ref, nv.ptr(a), nv.c_ll(a.stride(0)), nv.ptr(w), nv.c_ll(w.stride(0)), self.rows, self.n,
            a.shape[1], ctypes.c_ulonglong(self.recv.offset), ctypes.c_ulonglong(self.done.offset),
            ctypes.c_uint(self.calls), nv.ptr(gamma), nv.ptr(out), nv.c_float(eps), nv.c_float(scale),
            nv.current_stream()), "pkb_tp_gemm_rs_rmsnorm")
        nv.count_launch()
        return out


class GemmAllReduce:
    """Row-parallel linear layer with its all-reduce fused in (reference: reference/13_gemm_allreduce.py:17-20).

    ``M = W * rows_per_rank`` rows; the result lives in the symmetric heap and is returned as a view that stays valid
    until the next call of this object."""

    def __init__(self, group: SymmGroup, rows_per_rank: int, n: int, multicast: bool = True):
        if rows_per_rank % 256 != 0:
            raise ValueError("rows per rank must be a multiple of 256 (one CTA-pair tile)")
        if n % 8 != 0:
            raise ValueError("n must be a multiple of 8")
        self.group, self.rows, self.n, self.multicast = group, rows_per_rank, n, multicast
        heap = group.heap
        self.recv = heap.empty((group.size, rows_per_rank, n), torch.bfloat16)
        self.done = heap.empty((max(rows_per_rank // 128, 4),), torch.int32)
        self.out = heap.empty((group.size * rows_per_rank, n), torch.bfloat16)
        self.done.local.zero_()
        self.calls = 0

    def __call__(self, a: torch.Tensor, w: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
        W = self.group.size
        if a.shape[0] != W * self.rows or a.dtype != torch.bfloat16 or a.stride(1) != 1:
            raise ValueError("a must be bf16 [W * rows_per_rank, K_local]")
        if w.shape != (self.n, a.shape[1]) or w.stride(1) != 1 or w.dtype != torch.bfloat16:
            raise ValueError("w must be bf16 [N, K_local]")
        self.calls += 1
        nv.check(nv.cuda_lib().pkb_tp_gemm_allreduce(
            self.group.ref, nv.ptr(a), nv.c_ll(a.stride(0)), nv.ptr(w), nv.c_ll(w.stride(0)), self.rows, self.n, a.shape[1],
            ctypes.c_ulonglong(self.recv.offset), ctypes.c_ulonglong(self.done.offset), ctypes.c_uint(self.calls),
            ctypes.c_ulonglong(self.out.offset), nv.c_float(scale), 1 if self.multicast else 0, nv.current_stream()),
            "pkb_tp_gemm_allreduce")
        nv.count_launch()
        return self.out.local


class GemmAllGather:
    """Column-parallel linear layer with its all-gather along N fused in (reference: reference/14_gemm_allgather.py:17-22).

    The gathered result ``[M, W * n_local]`` lives in the symmetric heap and is returned as a view that stays valid until
    the next call of this object."""

    def __init__(self, group: SymmGroup, m: int, n_local: int):
        if n_local % 64 != 0:
            raise ValueError("n_local must be a multiple of 64 (one TMA-store box)")
        self.group, self.m, self.n_local = group, m, n_local
        self.out = group.heap.empty((m, group.size * n_local), torch.bfloat16)

    def __call__(self, a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, activation: str = "none") -> torch.Tensor:
        if a.shape[0] != self.m or a.dtype != torch.bfloat16 or a.stride(1) != 1:
            raise ValueError("a must be bf16 [M, K]")
        if w.shape != (self.n_local, a.shape[1]) or w.stride(1) != 1 or w.dtype != torch.bfloat16:
            raise ValueError("w must be bf16 [n_local, K]")
        if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != self.n_local):
            raise ValueError("bias must be bf16 [n_local]")
        epi = {"none": 0, "silu": 1}[activation] | (2 if bias is not None else 0)
        nv.check(nv.cuda_lib().pkb_tp_gemm_allgather(
            self.group.ref, nv.ptr(a), nv.c_ll(a.stride(0)), nv.ptr(w), nv.c_ll(w.stride(0)), self.m, self.n_local, a.shape[1],
            nv.ptr(bias), epi, ctypes.c_ulonglong(self.out.offset), nv.current_stream()), "pkb_tp_gemm_allgather")
        nv.count_launch()
        return self.out.local


class GemvAllGather:
    """Vocabulary-parallel LM head at decode time (reference: reference/46_gemv_decode.py:13-18).

    Results alternate between two symmetric buffers, so a returned view stays valid until the call after the next one."""

    def __init__(self, group: SymmGroup, tokens: int, n_local: int, multicast: bool = True):
        if tokens not in (1, 2, 4):
            raise ValueError("1, 2 or 4 tokens per call (use the GEMM for larger batches)")
        if n_local % 8 != 0:
            raise ValueError("n_local must be a multiple of 8")
        self.group, self.m, self.n_local, self.multicast = group, tokens, n_local, multicast
        self.out = [group.heap.empty((tokens, group.size * n_local), torch.bfloat16) for _ in range(2)]
        self.calls = 0

    def __call__(self, h: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        if h.shape[0] != self.m or h.dtype != torch.bfloat16 or not h.is_contiguous():
            raise ValueError("h must be contiguous bf16 [tokens, K]")
        K = h.shape[1]
        if w.shape != (self.n_local, K) or w.stride(1) != 1 or w.dtype != torch.bfloat16 or K % 8 or w.stride(0) % 8:
            raise ValueError("w must be bf16 [n_local, K] with K and its row pitch multiples of 8")
        if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != self.n_local or not bias.is_contiguous()):
            raise ValueError("bias must be contiguous bf16 [n_local]")
        buf = self.out[self.calls & 1]
        self.calls += 1
        nv.check(nv.cuda_lib().pkb_tp_gemv_allgather(self.group.ref, nv.ptr(h), nv.ptr(w), nv.c_ll(w.stride(0)), nv.ptr(bias), self.m,
                                                     self.n_local, K, ctypes.c_ulonglong(buf.offset), 1 if self.multicast else 0,
                                                     nv.current_stream()), "pkb_tp_gemv_allgather")
        nv.count_launch()
        return buf.local
