"""PyTorch + NCCL + cuBLAS reference of the tensor-parallel MLP block (oracle and timed baseline)."""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F


class TPMLPReference:
    def __init__(self, world: int, rows_per_rank: int, hidden: int, w1: torch.Tensor, w2: torch.Tensor,
                 gamma: torch.Tensor, eps: float, group=None):
        self.world, self.rows, self.hidden, self.eps, self.group = world, rows_per_rank, hidden, eps, group
        self.w1, self.w2, self.gamma = w1, w2, gamma
        dev = w1.device
        self.x_full = torch.empty((world * rows_per_rank, hidden), dtype=w1.dtype, device=dev)
        self.y_local = torch.empty((rows_per_rank, hidden), dtype=w1.dtype, device=dev)

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_gather_into_tensor(self.x_full, x_local, group=self.group)
            x_full = self.x_full
        else:
            x_full = x_local
        h = F.silu(F.linear(x_full, self.w1))
        partial = F.linear(h, self.w2)
        if self.world > 1:
            dist.reduce_scatter_tensor(self.y_local, partial, group=self.group)
            y = self.y_local
        else:
            y = partial
        yf = y.float()
        return (yf * torch.rsqrt(yf.pow(2).mean(-1, keepdim=True) + self.eps) * self.gamma.float()).to(x_local.dtype)

    __call__ = forward
