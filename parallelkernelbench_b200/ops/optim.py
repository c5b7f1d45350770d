"""Sharded optimiser step with its collectives inside the kernel (kernel: csrc/kernels/optim.cu).

``ZeroAdamStep`` is the data-parallel optimiser step as ONE launch: every rank writes its full bf16 gradient into the
object's symmetric gradient buffer (``grad_buffer``), then ``step`` sums this rank's slice over all ranks (in the switch
through ``multimem.ld_reduce`` when the group is the whole job, else with peer loads), applies Adam(W) to the shard state
in registers and stores the updated bf16 parameters into the gathered parameter buffer of every rank (``multimem.st`` or
peer stores). It replaces reduce-scatter (or all-reduce), optimiser kernel and all-gather of the reference's DDP / ZeRO
workloads (reference: reference/41_zero1_optimizer_shard.py:50-68, reference/42_zero2_optimizer_shard_grad.py:50-67,
reference/43_fused_adam_grad_unshard_allgather.py:28-43).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as nv
from ..parallel.symm_heap import SymmGroup


class ZeroAdamStep:
    def __init__(self, group: SymmGroup, part: int, multicast: bool = True):
        """``part``: elements of one rank's shard (a multiple of 8). Symmetric buffers: the gradient ``[W * part]`` and the
        gathered parameters ``[W * part]``, both bf16, kept between calls."""
        if part <= 0 or part % 8:
            raise ValueError("the shard length must be a positive multiple of 8")
        self.group, self.part, self.multicast = group, part, multicast
        heap = group.heap
        self.grad = heap.empty((group.size * part,), torch.bfloat16)
        self.params = heap.empty((group.size * part,), torch.bfloat16)

    @property
    def grad_buffer(self) -> torch.Tensor:
        """This rank's full gradient goes here (``[W * part]`` bf16; for ``reduce=False`` only the first ``part`` elements)."""
        return self.grad.local

    def step(self, p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, lr: float, beta1: float, beta2: float, eps: float,
             step: int, weight_decay: float = 0.0, grad_scale: float = 1.0, reduce: bool = True, gather: bool = True):
        """``p, m, v``: this rank's shard state ``[part]``, all bf16 or all fp32, updated in place. Returns the gathered bf16
        parameters ``[W * part]`` (a view of the symmetric buffer, valid until the next call) or ``None`` without ``gather``."""
        if not (p.dtype == m.dtype == v.dtype and p.dtype in (torch.bfloat16, torch.float32)):
            raise TypeError("shard state must be all bf16 or all fp32")
        for t in (p, m, v):
            if t.numel() != self.part or not t.is_contiguous():
                raise ValueError("shard state must be contiguous with `part` elements")
        nv.check(nv.cuda_lib().pkb_zero_adam_allgather(
            self.group.ref, ctypes.c_ulonglong(self.grad.offset), 1 if reduce else 0, nv.ptr(p), nv.ptr(m), nv.ptr(v),
            1 if p.dtype == torch.float32 else 0, ctypes.c_ulonglong(self.params.offset), 1 if gather else 0, nv.c_ll(self.part),
            nv.c_float(lr), nv.c_float(beta1), nv.c_float(beta2), nv.c_float(eps), nv.c_float(weight_decay), nv.c_float(grad_scale),
            int(step), 1 if self.multicast else 0, nv.current_stream()), "pkb_zero_adam_allgather")
        nv.count_launch()
        return self.params.local if gather else None
