"""Llama-style decoder with an FSDP training step (fp8 parameter all-gather, fp8 gradient exchange
fused with sharded AdamW, vocab-parallel cross-entropy).

Two implementations share this file's structure:

* ``impl="ours"``   GEMMs on the tcgen05 kernels (forward ``x W^T``, input gradient through the
  MN-major-B kernel, weight gradient through the transposed-A kernel - no transposed copies),
  flash-attention forward, RMSNorm, RoPE and cross-entropy on our kernels, parameters gathered as
  e4m3 bytes + 1x128 scales over the symmetric heap, gradients sent as fp8 slices and reduced inside
  the fused dequant-sum + AdamW + requantise kernel.
* ``impl="torch"``  the PyTorch + NCCL + cuBLAS baseline of the same step (bf16 all-gather,
  reduce-scatter, library attention, torch AdamW arithmetic).

Attention forward and backward of ``impl="ours"`` are the tcgen05 flash-attention kernels.
Reference ancestors: reference/47_fsdp_step_e2e.py, reference/52_fp8_reduce_scatter_grads.py,
reference/53_fp8_allgather_params.py, reference/73_vocab_parallel_cross_entropy_loss.py,
reference/17_rope_allgather.py, reference/18_tp_rms_norm.py.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F


@dataclass
class LlamaConfig:
    layers: int = 32
    hidden: int = 4096
    ffn: int = 14336
    heads: int = 32
    kv_heads: int = 8
    vocab: int = 128256
    seq: int = 4096
    rope_theta: float = 5e5
    eps: float = 1e-5
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    adam_eps: float = 1e-8
    weight_decay: float = 0.1
    weight_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    def layer_shapes(self) -> list[tuple[str, tuple[int, int]]]:
        d = self.head_dim
        return [("wqkv", ((self.heads + 2 * self.kv_heads) * d, self.hidden)), ("wo", (self.hidden, self.heads * d)),
                ("wgu", (2 * self.ffn, self.hidden)), ("wdown", (self.hidden, self.ffn)),
                ("norm1", (1, self.hidden)), ("norm2", (1, self.hidden))]

    def layer_numel(self) -> int:
        return sum(a * b for _, (a, b) in self.layer_shapes())


# =================================================================================================
# autograd functions over our kernels
# =================================================================================================
class _Linear(torch.autograd.Function):
    """y = x @ w.T ; dx = dy @ w (w read as an MN-major operand) ; dw = dy.T @ x (transposed-A kernel)."""

    @staticmethod
    def forward(ctx, x, w):
        from ..ops import gemm_bf16

        ctx.save_for_backward(x, w)
        return gemm_bf16(x, w)

    @staticmethod
    def backward(ctx, dy):
        from ..ops import gemm_bf16_kn, gemm_bf16_tn

        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        return gemm_bf16_kn(dy, w), gemm_bf16_tn(dy, x)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, eps):
        from ..ops import rmsnorm

        ctx.save_for_backward(x, gamma)
        ctx.eps = eps
        return rmsnorm(x, gamma.reshape(-1), eps)

    @staticmethod
    def backward(ctx, dy):
        from ..ops import rmsnorm_bwd

        x, gamma = ctx.saved_tensors
        dx, dg = rmsnorm_bwd(x, gamma, dy.contiguous(), ctx.eps)
        return dx, dg.to(gamma.dtype).reshape(gamma.shape), None


class _SwiGLU(torch.autograd.Function):
    """``silu(gate) * up`` over the packed [tokens, 2 * ffn] projection, forward and backward in one pass each."""

    @staticmethod
    def forward(ctx, gu):
        from ..ops import swiglu_fwd

        ctx.save_for_backward(gu)
        return swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, da):
        from ..ops import swiglu_bwd

        (gu,) = ctx.saved_tensors
        return swiglu_bwd(gu, da.contiguous())


class _Rope(torch.autograd.Function):
    """Rotate-half RoPE; the backward is the inverse rotation (same kernel with the sine negated)."""

    @staticmethod
    def forward(ctx, x, cos, sin):
        from ..ops import rope

        ctx.save_for_backward(cos, sin)
        return rope(x, cos, sin)

    @staticmethod
    def backward(ctx, dy):
        from ..ops import rope

        cos, sin = ctx.saved_tensors
        return rope(dy.contiguous(), cos, -sin), None, None


class _SplitQKV(torch.autograd.Function):
    """[S, (Hq + 2 Hkv) d] -> q [1, S, Hq, d], k, v [1, S, Hkv, d] (contiguous). The backward is one concatenation; autograd's
    own slice backward would zero-fill three projection-sized tensors and add them up."""

    @staticmethod
    def forward(ctx, qkv, hq, hkv, d):
        S = qkv.shape[0]
        ctx.dims = (hq, hkv, d)
        q = qkv[:, :hq * d].reshape(1, S, hq, d).contiguous()
        k = qkv[:, hq * d:(hq + hkv) * d].reshape(1, S, hkv, d).contiguous()
        v = qkv[:, (hq + hkv) * d:].reshape(1, S, hkv, d).contiguous()
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        hq, hkv, d = ctx.dims
        S = dq.shape[1]
        return torch.cat([dq.reshape(S, hq * d), dk.reshape(S, hkv * d), dv.reshape(S, hkv * d)], dim=1), None, None, None


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):
        from ..ops.attention import flash_attn_fwd

        out, lse = flash_attn_fwd(q, k, v, causal=True, scale=scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops.attention import flash_attn_bwd

        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = flash_attn_bwd(q, k, v, out, lse, dout.contiguous(), causal=True, scale=ctx.scale)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None


def rope_tables(cfg: LlamaConfig, device, dtype=torch.bfloat16):
    d = cfg.head_dim
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))
    ang = torch.arange(cfg.seq, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([ang.cos(), ang.cos()], -1).to(dtype), torch.cat([ang.sin(), ang.sin()], -1).to(dtype)


# =================================================================================================
# one decoder layer, either on our kernels or on PyTorch library ops
# =================================================================================================
def _rot_half(x, cos, sin):
    h = x.shape[-1] // 2
    return x * cos.unsqueeze(-2) + torch.cat([-x[..., h:], x[..., :h]], -1) * sin.unsqueeze(-2)


def _rms_torch(x, g, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * g.float().reshape(-1)).to(x.dtype)


def layer_forward(cfg: LlamaConfig, p: dict, x: torch.Tensor, cos, sin, impl: str) -> torch.Tensor:
    """``x`` is ``[S, hidden]`` (one sequence). ``p`` maps parameter names to bf16 tensors."""
    S, d, Hq, Hkv = x.shape[0], cfg.head_dim, cfg.heads, cfg.kv_heads
    ours = impl == "ours"
    lin = _Linear.apply if ours else (lambda a, w: F.linear(a, w))
    norm = (lambda a, g: _RMSNorm.apply(a, g, cfg.eps)) if ours else (lambda a, g: _rms_torch(a, g, cfg.eps))
    h = norm(x, p["norm1"])
    qkv = lin(h, p["wqkv"])
    if ours:
        q, k, v = _SplitQKV.apply(qkv, Hq, Hkv, d)
    else:
        q = qkv[:, :Hq * d].reshape(1, S, Hq, d)
        k = qkv[:, Hq * d:(Hq + Hkv) * d].reshape(1, S, Hkv, d)
        v = qkv[:, (Hq + Hkv) * d:].reshape(1, S, Hkv, d).contiguous()
    scale = 1.0 / math.sqrt(d)
    if ours:
        q, k = _Rope.apply(q, cos, sin), _Rope.apply(k, cos, sin)
        att = _FlashAttention.apply(q, k, v, scale)
    else:
        q, k = _rot_half(q, cos, sin), _rot_half(k, cos, sin)
        att = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                             scale=scale, enable_gqa=True).transpose(1, 2)
    x = x + lin(att.reshape(S, Hq * d), p["wo"])
    h2 = norm(x, p["norm2"])
    gu = lin(h2, p["wgu"])
    a = _SwiGLU.apply(gu) if ours else F.silu(gu[:, :cfg.ffn]) * gu[:, cfg.ffn:]
    return x + lin(a.contiguous(), p["wdown"])


class _SplitFlat(torch.autograd.Function):
    """The tensors of one layer as views of its flat parameter buffer. The backward writes the flat gradient with ONE
    concatenation; autograd's own slice backward would zero-fill a flat-sized buffer and add into it once per tensor
    (fourteen passes over 436 MB per Llama-8B layer, 15 % of a step's kernel time)."""

    @staticmethod
    def forward(ctx, flat, shapes):
        ctx.shapes, ctx.total = shapes, flat.numel()
        out, o = [], 0
        for a, b in shapes:
            out.append(flat[o:o + a * b].view(a, b))
            o += a * b
        return tuple(out)

    @staticmethod
    def backward(ctx, *grads):
        parts, used = [], 0
        ref = next(g for g in grads if g is not None)
        for (a, b), g in zip(ctx.shapes, grads):
            parts.append(g.reshape(-1) if g is not None else ref.new_zeros(a * b))
            used += a * b
        if used < ctx.total:
            parts.append(ref.new_zeros(ctx.total - used))        # padding of the flat buffer to the shard grid
        return torch.cat(parts), None


def split_layer_params(cfg: LlamaConfig, flat: torch.Tensor) -> dict:
    names = [name for name, _ in cfg.layer_shapes()]
    shapes = tuple(shape for _, shape in cfg.layer_shapes())
    if flat.requires_grad:
        return dict(zip(names, _SplitFlat.apply(flat, shapes)))
    out, o = {}, 0
    for name, (a, b) in cfg.layer_shapes():
        out[name] = flat[o:o + a * b].view(a, b)
        o += a * b
    return out


class _VocabParallelLoss(torch.autograd.Function):
    """Mean cross-entropy of ``hidden_all @ head_shard.T`` with the vocabulary sharded over the ranks.

    forward : local logits GEMM, one pass of row statistics, ONE packed exchange, loss per token
    backward: d logits = (softmax - onehot) / tokens from the saved log-sum-exp; d hidden through the
              MN-major-B GEMM (the caller reduce-scatters it to the token owners); d head = dlogits^T hidden
    """

    @staticmethod
    def forward(ctx, hidden_all, head_shard, targets_all, comm, vocab_start, impl):
        ours = impl == "ours"
        if ours:
            from ..ops import ce_local_stats, gemm_bf16

            logits = gemm_bf16(hidden_all, head_shard)
            stats = ce_local_stats(logits, targets_all, vocab_start)
            allst = comm.all_gather(stats) if comm is not None and comm.size() > 1 else stats.unsqueeze(0)
        else:
            logits = F.linear(hidden_all, head_shard)
            lf = logits.float()
            mx = lf.max(-1).values
            se = torch.exp(lf - mx[:, None]).sum(-1)
            t = targets_all - vocab_start
            inr = (t >= 0) & (t < lf.shape[1])
            tg = torch.where(inr, lf.gather(1, t.clamp(0, lf.shape[1] - 1)[:, None])[:, 0], torch.zeros_like(mx))
            stats = torch.stack([mx, se, tg], -1)
            if dist.is_initialized() and dist.get_world_size() > 1:
                allst = torch.empty((dist.get_world_size(), *stats.shape), device=stats.device)
                dist.all_gather_into_tensor(allst.view(-1, 3), stats.contiguous())
            else:
                allst = stats.unsqueeze(0)
        gmax = allst[..., 0].max(0).values
        lse = torch.log((allst[..., 1] * torch.exp(allst[..., 0] - gmax)).sum(0)) + gmax
        loss = (lse - allst[..., 2].sum(0)).mean()
        ctx.save_for_backward(hidden_all, head_shard, logits, lse, targets_all)
        ctx.vocab_start, ctx.ours = vocab_start, ours
        return loss

    @staticmethod
    def backward(ctx, dloss):
        hidden_all, head_shard, logits, lse, targets = ctx.saved_tensors
        n = logits.shape[0]
        if ctx.ours and logits.dtype == torch.bfloat16 and logits.shape[1] % 8 == 0:
            from ..ops import ce_backward, gemm_bf16_kn, gemm_bf16_tn

            dlog = ce_backward(logits, lse, targets, ctx.vocab_start, 1.0 / n, upstream=dloss)
            return gemm_bf16_kn(dlog, head_shard), gemm_bf16_tn(dlog, hidden_all), None, None, None, None
        dlog = torch.exp(logits.float() - lse[:, None])
        t = targets - ctx.vocab_start
        inr = (t >= 0) & (t < logits.shape[1])
        rows = torch.nonzero(inr, as_tuple=True)[0]
        dlog[rows, t[rows]] -= 1.0
        dlog = (dlog * (dloss / n)).to(logits.dtype)
        if ctx.ours:
            from ..ops import gemm_bf16_kn, gemm_bf16_tn

            return gemm_bf16_kn(dlog, head_shard), gemm_bf16_tn(dlog, hidden_all), None, None, None, None
        return dlog @ head_shard, dlog.t() @ hidden_all, None, None, None, None


# =================================================================================================
# FSDP engine
# =================================================================================================
class _GatherRows(torch.autograd.Function):
    """all-gather of ``[S, H]`` rows over the ranks; the backward reduce-scatters the gradient."""

    @staticmethod
    def forward(ctx, x, eng):
        ctx.eng = eng
        return eng.all_gather_rows(x)

    @staticmethod
    def backward(ctx, dy):
        return ctx.eng.reduce_scatter_rows(dy.contiguous()), None


class _Unit:
    """One flat parameter group: fp32 master shard + Adam moments, and the shard in wire format."""

    def __init__(self, eng, shapes: list[tuple[str, tuple[int, int]]], seed: int):
        cfg, W, r, dev = eng.cfg, eng.W, eng.rank, eng.device
        self.eng, self.shapes = eng, shapes
        self.numel = sum(a * b for _, (a, b) in shapes)
        self.padded = (self.numel + 128 * W - 1) // (128 * W) * (128 * W)
        self.shard = self.padded // W
        g = torch.Generator(device=dev).manual_seed(seed)
        full = torch.zeros(self.padded, device=dev, dtype=torch.float32)
        o = 0
        for name, (a, b) in shapes:
            if name.startswith("norm"):
                full[o:o + a * b] = 1.0
            else:
                full[o:o + a * b] = torch.randn(a * b, device=dev, generator=g) * cfg.weight_std
            o += a * b
        self.master = full[r * self.shard:(r + 1) * self.shard].clone()
        del full
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        if eng.impl == "ours":
            from ..ops import fp8_quantize_1x128

            q, s = fp8_quantize_1x128(self.master.view(-1, 128))
            self.q8, self.s8 = q.view(-1).contiguous(), s.view(-1).contiguous()
        else:
            self.bf16 = self.master.to(torch.bfloat16)

    def state(self) -> dict:
        """This rank's shard: fp32 master and Adam moments plus the wire-format copy (e4m3 bytes and 1x128 scales, or bf16)."""
        d = {"master": self.master, "m": self.m, "v": self.v}
        d.update({"q8": self.q8, "s8": self.s8} if self.eng.impl == "ours" else {"bf16": self.bf16})
        return d

    def load_state(self, d: dict) -> None:
        for k, t in self.state().items():
            if k not in d or d[k].shape != t.shape or d[k].dtype != t.dtype:
                raise ValueError(f"checkpoint shard lacks {k!r} or has another shape / dtype (other world size or config?)")
            t.copy_(d[k])

    def gather(self) -> torch.Tensor:
        eng = self.eng
        if eng.impl == "ours":
            from ..ops import fp8_dequantize_1x128

            if eng.W > 1:
                q = eng.comm.all_gather(self.q8).view(-1)
                s = eng.comm.all_gather(self.s8).view(-1)
            else:
                q, s = self.q8, self.s8
            return fp8_dequantize_1x128(q.view(-1, 128), s.view(-1, 1), torch.bfloat16).view(-1)
        if eng.W > 1:
            full = torch.empty(self.padded, device=eng.device, dtype=torch.bfloat16)
            dist.all_gather_into_tensor(full, self.bf16)
            return full
        return self.bf16.clone()

    def reduce_and_step(self, grad: torch.Tensor, step: int) -> None:
        eng, cfg = self.eng, self.eng.cfg
        if eng.impl == "ours":
            from ..ops import fp8_quantize_1x128
            from ..ops.quant import fsdp_adamw_fp8

            q, s = fp8_quantize_1x128(grad.view(-1, 128))
            q, s = q.view(eng.W, self.shard), s.view(eng.W, self.shard // 128)
            if eng.W > 1:
                q, s = eng.comm.all_to_all(q), eng.comm.all_to_all(s)      # fp8 slices travel, 1 byte/element
            fsdp_adamw_fp8(q, s, self.master, self.m, self.v, self.q8, self.s8, lr=cfg.lr, beta1=cfg.beta1, beta2=cfg.beta2,
                           eps=cfg.adam_eps, weight_decay=cfg.weight_decay, grad_scale=1.0, step=step)
            return
        if eng.W > 1:
            gs = torch.empty(self.shard, device=eng.device, dtype=grad.dtype)
            dist.reduce_scatter_tensor(gs, grad.contiguous())
        else:
            gs = grad
        g = gs.float()
        self.master.mul_(1.0 - cfg.lr * cfg.weight_decay)
        self.m.mul_(cfg.beta1).add_(g, alpha=1.0 - cfg.beta1)
        self.v.mul_(cfg.beta2).addcmul_(g, g, value=1.0 - cfg.beta2)
        denom = (self.v / (1.0 - cfg.beta2 ** step)).sqrt_().add_(cfg.adam_eps)
        self.master.addcdiv_(self.m, denom, value=-cfg.lr / (1.0 - cfg.beta1 ** step))
        self.bf16.copy_(self.master)


class FSDPLlama:
    """Sharded Llama decoder: ``step(tokens, targets)`` runs forward, backward and the optimiser."""

    def __init__(self, ctx, cfg: LlamaConfig, impl: str = "ours"):
        self.ctx, self.cfg, self.impl = ctx, cfg, impl
        self.W, self.rank, self.device = ctx.world, ctx.rank, ctx.device
        self.comm = None
        if impl == "ours":
            from ..parallel.comm import Comm

            self.comm = Comm(ctx)
        if cfg.vocab % self.W != 0:
            raise ValueError("vocab must be divisible by the number of ranks")
        self.embed = _Unit(self, [("embed", (cfg.vocab, cfg.hidden))], seed=11)
        self.units = [_Unit(self, cfg.layer_shapes(), seed=100 + l) for l in range(cfg.layers)]
        vl = cfg.vocab // self.W
        g = torch.Generator(device=self.device).manual_seed(7000 + self.rank)
        self.head_master = torch.randn(vl, cfg.hidden, device=self.device, generator=g) * cfg.weight_std
        self.head_m, self.head_v = torch.zeros_like(self.head_master), torch.zeros_like(self.head_master)
        self.head = self.head_master.to(torch.bfloat16).requires_grad_()
        self.final_gain = torch.ones(1, cfg.hidden, device=self.device, dtype=torch.bfloat16)
        self.cos, self.sin = rope_tables(cfg, self.device)
        self.steps = 0

    # -- sharded checkpoint --------------------------------------------------------------------------
    def save_sharded(self, directory: str) -> str:
        """Write this rank's shard of the whole training state (every unit's fp32 master, Adam moments and wire-format
        copy, the vocabulary-parallel head with its moments, the step count) to ``directory/rank_<r>_of_<W>.pt``.
        Every rank calls it; nothing is gathered. Returns the file written."""
        import os

        os.makedirs(directory, exist_ok=True)
        cpu = lambda d: {k: v.detach().cpu() for k, v in d.items()}  # noqa: E731
        blob = {"format": 1, "world": self.W, "rank": self.rank, "impl": self.impl, "steps": self.steps,
                "config": {k: getattr(self.cfg, k) for k in ("vocab", "hidden", "layers", "heads", "kv_heads", "ffn")
                           if hasattr(self.cfg, k)},
                "embed": cpu(self.embed.state()), "units": [cpu(u.state()) for u in self.units],
                "head": cpu({"master": self.head_master, "m": self.head_m, "v": self.head_v, "bf16": self.head.data})}
        path = os.path.join(directory, f"rank_{self.rank}_of_{self.W}.pt")
        tmp = path + ".tmp"
        torch.save(blob, tmp)
        os.replace(tmp, path)          # a reader never sees a half-written file
        return path

    def load_sharded(self, directory: str) -> int:
        """Restore what :meth:`save_sharded` wrote (same world size, implementation and config). Returns the step count."""
        import os

        path = os.path.join(directory, f"rank_{self.rank}_of_{self.W}.pt")
        blob = torch.load(path, map_location=self.device)
        if blob.get("format") != 1 or blob["world"] != self.W or blob["rank"] != self.rank or blob["impl"] != self.impl:
            raise ValueError(f"{path}: written by rank {blob.get('rank')} of {blob.get('world')} with implementation "
                             f"{blob.get('impl')!r}; this is rank {self.rank} of {self.W} with {self.impl!r}")
        for k, v in blob["config"].items():
            if getattr(self.cfg, k) != v:
                raise ValueError(f"{path}: config mismatch on {k}: checkpoint {v}, model {getattr(self.cfg, k)}")
        if len(blob["units"]) != len(self.units):
            raise ValueError(f"{path}: {len(blob['units'])} layers in the checkpoint, {len(self.units)} in the model")
        with torch.no_grad():
            self.embed.load_state(blob["embed"])
            for u, d in zip(self.units, blob["units"]):
                u.load_state(d)
            h = blob["head"]
            self.head_master.copy_(h["master"])
            self.head_m.copy_(h["m"])
            self.head_v.copy_(h["v"])
            self.head.data.copy_(h["bf16"])
        self.steps = int(blob["steps"])
        return self.steps

    # -- collectives over rows ---------------------------------------------------------------------
    def all_gather_rows(self, x):
        if self.W == 1:
            return x
        if self.impl == "ours":
            return self.comm.all_gather(x.contiguous()).view(-1, x.shape[1])
        out = torch.empty((self.W * x.shape[0], x.shape[1]), device=x.device, dtype=x.dtype)
        dist.all_gather_into_tensor(out, x.contiguous())
        return out

    def reduce_scatter_rows(self, dy):
        if self.W == 1:
            return dy
        if self.impl == "ours":
            return self.comm.reduce_scatter(dy)
        out = torch.empty((dy.shape[0] // self.W, dy.shape[1]), device=dy.device, dtype=dy.dtype)
        dist.reduce_scatter_tensor(out, dy)
        return out

    def _gather_targets(self, t):
        if self.W == 1:
            return t
        if self.impl == "ours":
            return self.comm.all_gather(t.contiguous()).view(-1)
        out = torch.empty(self.W * t.numel(), device=t.device, dtype=t.dtype)
        dist.all_gather_into_tensor(out, t.contiguous())
        return out

    # -- one training step -------------------------------------------------------------------------
    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        self.steps += 1
        step = self.steps

        def hooked(unit):
            flat = unit.gather().requires_grad_()

            def on_grad(t, unit=unit):
                unit.reduce_and_step(t.grad, step)      # exchange + optimiser as soon as this unit's gradient exists
                t.grad = None
            flat.register_post_accumulate_grad_hook(on_grad)
            return flat

        emb = hooked(self.embed)
        x = F.embedding(tokens, emb[:cfg.vocab * cfg.hidden].view(cfg.vocab, cfg.hidden))
        for unit in self.units:
            flat = hooked(unit)
            x = layer_forward(cfg, split_layer_params(cfg, flat), x, self.cos, self.sin, self.impl)
        xn = _RMSNorm.apply(x, self.final_gain, cfg.eps) if self.impl == "ours" else _rms_torch(x, self.final_gain, cfg.eps)
        hidden_all = _GatherRows.apply(xn, self)
        loss = _VocabParallelLoss.apply(hidden_all, self.head, self._gather_targets(targets), self.comm,
                                        self.rank * (cfg.vocab // self.W), self.impl)
        loss.backward()
        # vocabulary-parallel head: every rank saw all tokens, so its gradient is already complete
        g = self.head.grad
        if self.impl == "ours":
            from ..ops import adam_step

            with torch.no_grad():
                adam_step(self.head_master, self.head_m, self.head_v, g.contiguous(), lr=cfg.lr, beta1=cfg.beta1, beta2=cfg.beta2,
                          eps=cfg.adam_eps, step=step, weight_decay=cfg.weight_decay, decoupled=True, p_bf16=self.head.data)
        else:
            with torch.no_grad():
                gf = g.float()
                self.head_master.mul_(1.0 - cfg.lr * cfg.weight_decay)
                self.head_m.mul_(cfg.beta1).add_(gf, alpha=1.0 - cfg.beta1)
                self.head_v.mul_(cfg.beta2).addcmul_(gf, gf, value=1.0 - cfg.beta2)
                denom = (self.head_v / (1.0 - cfg.beta2 ** step)).sqrt_().add_(cfg.adam_eps)
                self.head_master.addcdiv_(self.head_m, denom, value=-cfg.lr / (1.0 - cfg.beta1 ** step))
                self.head.data.copy_(self.head_master)
        self.head.grad = None
        return loss.detach()
