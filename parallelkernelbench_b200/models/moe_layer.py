"""Expert-parallel MoE layer: router -> fp8 dispatch -> grouped SwiGLU expert FFN -> combine.

Five of our kernels per forward besides the router: histogram, plan, dispatch (P2P push of fp8 rows
with 1x128 scales), two grouped tcgen05 GEMMs (gate/up with the SwiGLU epilogue, then down, writing
into the symmetric buffer the combine reads), combine (P2P pull, gate-weighted, deterministic order).
The router GEMM runs on the dense tcgen05 kernel; softmax and top-k over a few hundred experts are
PyTorch ops. ``push_combine`` moves the way home into the down GEMM: the dispatch delivers (sender, assignment index) with every row, the
GEMM's epilogue stores each output row straight into the sender's buffer over NVLink, and the combine kernel only reads local
memory after its barrier.
Reference behaviour: reference/31_fused_moe_fwd.py:254-315 (with shared expert weights;
here every expert has its own).

``fp8_experts`` keeps the received tokens in e4m3: the expert weights are quantised once to e4m3 with
128 x 128 block scales, the gate/up GEMM runs block-scaled on the fp8 tokens with a SwiGLU + 1x128
re-quantise epilogue and the down GEMM consumes that directly - no dequantise pass and no bf16 copy of
the received tokens or of the hidden activations.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops.gemm import gemm_bf16
from ..ops.gemm_fp8 import gemm_fp8_blockscaled
from ..ops.moe import MoEExchange, grouped_gemm, grouped_gemm_scatter, interleave_gate_up, route_topk


@dataclass
class MoEConfig:
    hidden: int = 7168
    inter: int = 2048
    num_experts: int = 256
    top_k: int = 8
    tokens_per_rank: int = 8192
    capacity_factor: float = 2.0
    fp8_dispatch: bool = True
    fp8_experts: bool = False
    push_combine: bool = False      # the down GEMM's epilogue stores each output row in its token owner's memory
    fused_router: bool = True       # softmax + top-k + histogram in one kernel (up to 256 experts) instead of PyTorch ops + histogram kernel
    weight_std: float = 0.02


class EPMoELayer:
    def __init__(self, group, comm, cfg: MoEConfig, w_router: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                 w_down: torch.Tensor, router_bias: torch.Tensor | None = None):
        """``w_router`` [E, H]; ``w_gate``/``w_up`` [E_local, I, H]; ``w_down`` [E_local, H, I] (all bf16)."""
        self.group, self.comm, self.cfg = group, comm, cfg
        self.w_router, self.router_bias = w_router.contiguous(), router_bias
        self.router_bias_f32 = None if router_bias is None else router_bias.float().contiguous()
        if cfg.fused_router and cfg.num_experts > 256:
            cfg.fused_router = False             # the one-warp-per-token router kernel holds at most 256 experts in registers
        self.w_gate_up = interleave_gate_up(w_gate, w_up)
        self.w_down = w_down.contiguous()
        self.ex = MoEExchange(group, cfg.num_experts, cfg.hidden, cfg.tokens_per_rank, cfg.top_k, cfg.capacity_factor,
                              cfg.fp8_dispatch, push_combine=cfg.push_combine)
        dev = w_router.device
        if cfg.fp8_experts:
            from ..refs.gemm_fp8 import quantize_weight_128x128

            if not cfg.fp8_dispatch or cfg.hidden % 128 or cfg.inter % 128:
                raise ValueError("fp8 experts need the fp8 dispatch and hidden, inter multiples of 128")
            self.w8_gate_up, self.s_gate_up = quantize_weight_128x128(self.w_gate_up)
            self.w8_down, self.s_down = quantize_weight_128x128(self.w_down)
            self.w_gate_up = self.w_down = None
            self.h8 = torch.empty((self.ex.capacity, cfg.inter), dtype=torch.uint8, device=dev)
            self.h_scales = torch.empty((self.ex.capacity, cfg.inter // 128), dtype=torch.float32, device=dev)
        else:
            self.h = torch.empty((self.ex.capacity, cfg.inter), dtype=torch.bfloat16, device=dev)

    def route(self, x: torch.Tensor):
        logits = gemm_bf16(x, self.w_router, out_dtype=torch.float32, mode="single", block_n=128)
        if self.cfg.fused_router:
            gates, idx, _ = route_topk(logits, self.router_bias_f32, self.cfg.top_k, counts=self.ex.counts)
            return gates, idx
        if self.router_bias is not None:
            logits = logits + self.router_bias.float()
        gates, idx = torch.topk(torch.softmax(logits, dim=-1), self.cfg.top_k, dim=-1)
        return gates.contiguous(), idx.to(torch.int32).contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        T = x.shape[0]
        gates, idx = self.route(x)
        flat_idx = idx.view(-1)
        self.ex.plan(flat_idx, self.comm, counts_ready=self.cfg.fused_router)
        if self.cfg.fp8_experts:
            x8, xs = self.ex.dispatch(x, flat_idx, dequantize=False)
            gemm_fp8_blockscaled(x8, xs, self.w8_gate_up, self.s_gate_up, offsets=self.ex.offsets, epilogue="swiglu_quant",
                                 out=self.h8, out_scales=self.h_scales)
            if self.cfg.push_combine:
                gemm_fp8_blockscaled(self.h8, self.h_scales, self.w8_down, self.s_down, offsets=self.ex.offsets,
                                     epilogue="row_scatter", row_meta=self.ex.recv_meta.local, dest_ptrs=self.ex.home_ptrs(),
                                     dest_pitch=self.cfg.hidden)
            else:
                gemm_fp8_blockscaled(self.h8, self.h_scales, self.w8_down, self.s_down, offsets=self.ex.offsets,
                                     out=self.ex.y.local)
        else:
            xin = self.ex.dispatch(x, flat_idx)
            grouped_gemm(xin, self.w_gate_up, self.ex.offsets, epilogue="swiglu", out=self.h)
            if self.cfg.push_combine:
                grouped_gemm_scatter(self.h, self.w_down, self.ex.offsets, self.ex.recv_meta.local, self.ex.home_ptrs(),
                                     self.cfg.hidden)
            else:
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
