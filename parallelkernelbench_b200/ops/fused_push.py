"""Elementwise producers fused with the all-gather of their result (kernels: csrc/kernels/fused_push.cu).

``Fp8QuantAllGather``  1x128 e4m3 quantisation whose payload and scales leave the quantising thread for the gathered buffers
                       of every rank (reference: reference/19_blocked_fp8_quantize.py:7-47 quantises, then all-gathers twice).
``RopeAllGather``      rotate-half RoPE of q and k gathered along the sequence in the same launch
                       (reference: reference/17_rope_allgather.py:10-35 rotates, then all-gathers q and k).
Both are one launch with an entry and a closing in-kernel barrier; stores go through the switch (``multimem.st``) when the
group is the whole job, else as one peer store per member. The gathered tensors are views of symmetric buffers owned by
the object and stay valid until its next call.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as nv
from ..parallel.symm_heap import SymmGroup


class Fp8QuantAllGather:
    def __init__(self, group: SymmGroup, shape: tuple, multicast: bool = True):
        if shape[-1] % 128:
            raise ValueError("the last dimension must be a multiple of 128")
        self.group, self.shape, self.multicast = group, tuple(shape), multicast
        n = 1
        for s in shape:
            n *= s
        self.n = n
        heap = group.heap
        self.payload = heap.empty((group.size, *shape), torch.uint8)
        self.scales = heap.empty((group.size, *shape[:-1], shape[-1] // 128), torch.float32)

    def __call__(self, x: torch.Tensor):
        """``x``: bf16, the constructor's shape. Returns ``(payload [W, *shape] uint8, scales [W, ..., last/128] fp32)``."""
        if tuple(x.shape) != self.shape or x.dtype != torch.bfloat16:
            raise ValueError("input must be bf16 with the shape given at construction")
        xc = x.contiguous()
        nv.check(nv.cuda_lib().pkb_fp8_quant_allgather(self.group.ref, nv.ptr(xc), nv.c_ll(self.n), ctypes.c_ulonglong(self.payload.offset),
                                                       ctypes.c_ulonglong(self.scales.offset), 1 if self.multicast else 0,
                                                       nv.current_stream()), "pkb_fp8_quant_allgather")
        nv.count_launch()
        return self.payload.local, self.scales.local


class RopeAllGather:
    def __init__(self, group: SymmGroup, batch: int, t: int, heads_q: int, heads_k: int, dim: int, multicast: bool = True):
        if dim % 16:
            raise ValueError("the head dimension must be a multiple of 16")
        self.group, self.multicast = group, multicast
        self.batch, self.t, self.hq, self.hk, self.dim = batch, t, heads_q, heads_k, dim
        heap = group.heap
        self.q_out = heap.empty((batch, group.size * t, heads_q, dim), torch.bfloat16)
        self.k_out = heap.empty((batch, group.size * t, heads_k, dim), torch.bfloat16)

    def __call__(self, q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
        """``q [b, t, hq, d]``, ``k [b, t, hk, d]``, ``cos`` / ``sin`` ``[b, t, d]`` (bf16). Returns the rotated q and k of all ranks
        concatenated along the sequence: ``[b, W * t, h, d]``."""
        if q.shape != (self.batch, self.t, self.hq, self.dim) or k.shape != (self.batch, self.t, self.hk, self.dim):
            raise ValueError("q / k do not have the shapes given at construction")
        qc, kc = q.contiguous(), k.contiguous()
        cs, sn = cos.to(torch.bfloat16).contiguous(), sin.to(torch.bfloat16).contiguous()
        nv.check(nv.cuda_lib().pkb_rope_allgather(self.group.ref, nv.ptr(qc), nv.ptr(kc), nv.ptr(cs), nv.ptr(sn), self.batch, self.t,
                                                  self.hq, self.hk, self.dim, ctypes.c_ulonglong(self.q_out.offset),
                                                  ctypes.c_ulonglong(self.k_out.offset), 1 if self.multicast else 0,
                                                  nv.current_stream()), "pkb_rope_allgather")
        nv.count_launch()
        return self.q_out.local, self.k_out.local
