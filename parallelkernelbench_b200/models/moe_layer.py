"""Expert-parallel MoE layer: router -> fp8 dispatch -> grouped SwiGLU expert FFN -> combine.

Five of our kernels per forward besides the router: histogram, plan, dispatch (P2P push of fp8 rows
with 1x128 scales), two grouped tcgen05 GEMMs (gate/up with the SwiGLU epilogue, then down, writing
into the symmetric buffer the combine reads), combine (P2P pull, gate-weighted, deterministic order).
The router GEMM runs on the dense tcgen05 kernel; softmax and top-k over a few hundred experts are
PyTorch ops. Reference behaviour: reference/31_fused_moe_fwd.py:254-315 (with shared expert weights;
here every expert has its own).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops.gemm import gemm_bf16
from ..ops.moe import MoEExchange, grouped_gemm, interleave_gate_up


@dataclass
class MoEConfig:
    hidden: int = 7168
    inter: int = 2048
    num_experts: int = 256
    top_k: int = 8
    tokens_per_rank: int = 8192
    capacity_factor: float = 2.0
    fp8_dispatch: bool = True
    weight_std: float = 0.02


class EPMoELayer:
    def __init__(self, group, comm, cfg: MoEConfig, w_router: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                 w_down: torch.Tensor, router_bias: torch.Tensor | None = None):
        """``w_router`` [E, H]; ``w_gate``/``w_up`` [E_local, I, H]; ``w_down`` [E_local, H, I] (all bf16)."""
        self.group, self.comm, self.cfg = group, comm, cfg
        self.w_router, self.router_bias = w_router.contiguous(), router_bias
        self.w_gate_up = interleave_gate_up(w_gate, w_up)
        self.w_down = w_down.contiguous()
        self.ex = MoEExchange(group, cfg.num_experts, cfg.hidden, cfg.tokens_per_rank, cfg.top_k, cfg.capacity_factor,
                              cfg.fp8_dispatch)
        self.h = torch.empty((self.ex.capacity, cfg.inter), dtype=torch.bfloat16, device=w_router.device)

    def route(self, x: torch.Tensor):
        logits = gemm_bf16(x, self.w_router, out_dtype=torch.float32, mode="single", block_n=128)
        if self.router_bias is not None:
            logits = logits + self.router_bias.float()
        gates, idx = torch.topk(torch.softmax(logits, dim=-1), self.cfg.top_k, dim=-1)
        return gates.contiguous(), idx.to(torch.int32).contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        T = x.shape[0]
        gates, idx = self.route(x)
        flat_idx = idx.view(-1)
        self.ex.plan(flat_idx, self.comm)
        xin = self.ex.dispatch(x, flat_idx)
        grouped_gemm(xin, self.w_gate_up, self.ex.offsets, epilogue="swiglu", out=self.h)
        grouped_gemm(self.h, self.w_down, self.ex.offsets, out=self.ex.y.local)
        return self.ex.combine(flat_idx, gates.view(-1), T)

    __call__ = forward

    @staticmethod
    def random_weights(cfg: MoEConfig, world: int, rank: int, device, seed: int = 0):
        el = cfg.num_experts // world
        g = torch.Generator(device=device).manual_seed(31337 + seed)          # router is replicated
        w_router = (torch.randn(cfg.num_experts, cfg.hidden, device=device, generator=g) * cfg.weight_std).to(torch.bfloat16)
        g = torch.Generator(device=device).manual_seed(5000 + seed * 17 + rank)
        mk = lambda *s: (torch.randn(*s, device=device, generator=g) * cfg.weight_std).to(torch.bfloat16)  # noqa: E731
        return w_router, mk(el, cfg.inter, cfg.hidden), mk(el, cfg.inter, cfg.hidden), mk(el, cfg.hidden, cfg.inter)
