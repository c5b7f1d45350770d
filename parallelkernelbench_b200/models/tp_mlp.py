"""Tensor-parallel MLP block with sequence-sharded activations (the flagship block).

    all-gather(X) -> X @ W1_r -> SiLU -> @ W2_r -> reduce-scatter over rows -> RMSNorm

Two launches per forward: ``AllGatherGemm`` (gather fused into GEMM1 with the SiLU epilogue) and
``GemmReduceScatterRMSNorm`` (GEMM2 with the reduce-scatter in its epilogue and the RMSNorm in its
consumer phase). Weights are held K-major (``w1`` is ``[ffn_local, hidden]``, ``w2`` is
``[hidden, ffn_local]``), the layout both tcgen05 operands want.

This is the scaled-up, weight-sharded form of the reference's combined sharded GEMM workload
followed by its reduce-scatter + RMSNorm workload (reference: reference/15_combined_sharded_gemms.py:7-32,
reference/45_reducescatter_fused_rmsnorm.py:9-30).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops.tp import AllGatherGemm, GemmReduceScatterRMSNorm


@dataclass
class TPMLPConfig:
    rows_per_rank: int = 2048
    hidden: int = 8192
    ffn: int = 28672          # total intermediate size, sharded over the TP group
    eps: float = 1e-6
    weight_std: float = 0.02

    def ffn_local(self, world: int) -> int:
        if self.ffn % world != 0:
            raise ValueError("ffn must be divisible by the TP size")
        return self.ffn // world


class TPMLPBlock:
    def __init__(self, group, cfg: TPMLPConfig, w1: torch.Tensor, w2: torch.Tensor, gamma: torch.Tensor,
                 comm_ctas: int = 0):
        W = group.size
        f = cfg.ffn_local(W)
        assert w1.shape == (f, cfg.hidden) and w2.shape == (cfg.hidden, f), (w1.shape, w2.shape)
        self.group, self.cfg = group, cfg
        self.w1, self.w2, self.gamma = w1.contiguous(), w2.contiguous(), gamma.contiguous()
        self.ag_gemm = AllGatherGemm(group, cfg.rows_per_rank, cfg.hidden, comm_ctas=comm_ctas)
        self.gemm_rs = GemmReduceScatterRMSNorm(group, cfg.rows_per_rank, cfg.hidden)
        self.h = torch.empty((W * cfg.rows_per_rank, f), dtype=torch.bfloat16, device=w1.device)
        self.out = torch.empty((cfg.rows_per_rank, cfg.hidden), dtype=torch.bfloat16, device=w1.device)

    @property
    def x_slot(self) -> torch.Tensor:
        """Write the step's activations here (a view into the symmetric gather buffer) to avoid a copy."""
        return self.ag_gemm.x_slot

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        self.ag_gemm(x_local, self.w1, out=self.h, epilogue="silu")
        return self.gemm_rs(self.h, self.w2, self.gamma, eps=self.cfg.eps, out=self.out)

    __call__ = forward

    @staticmethod
    def random_weights(cfg: TPMLPConfig, world: int, rank: int, device, seed: int = 0):
        """Random-init shard of the weights: N(0, weight_std), seeded per rank."""
        g = torch.Generator(device=device).manual_seed(1000 + seed * 131 + rank)
        f = cfg.ffn_local(world)
        w1 = (torch.randn(f, cfg.hidden, device=device, generator=g) * cfg.weight_std).to(torch.bfloat16)
        w2 = (torch.randn(cfg.hidden, f, device=device, generator=g) * cfg.weight_std).to(torch.bfloat16)
        gamma = torch.ones(cfg.hidden, device=device, dtype=torch.bfloat16)
        return w1, w2, gamma
