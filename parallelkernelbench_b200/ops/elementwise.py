"""Memory-bound kernels (csrc/kernels/elementwise.cu): RoPE, fp8 1x128 quantise / dequantise, fused
Adam(W), vocab-parallel cross-entropy, LayerNorm-backward column reductions, tensor-parallel RMSNorm.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as nv

_DT = {torch.bfloat16: 0, torch.float32: 1}


def _dt(t: torch.Tensor) -> int:
    if t.dtype not in _DT:
        raise TypeError(f"unsupported dtype {t.dtype} (bf16 or fp32)")
    return _DT[t.dtype]


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE. ``x`` is ``[..., heads, dim]``, ``cos``/``sin`` are ``[..., dim]`` over the same
    leading (token) dimensions (reference semantics: reference/17_rope_allgather.py:10-29)."""
    dim, heads = x.shape[-1], x.shape[-2]
    xc = x.contiguous()
    tokens = xc.numel() // (heads * dim)
    cs, sn = cos.to(x.dtype).contiguous(), sin.to(x.dtype).contiguous()
    if cs.numel() != tokens * dim:
        raise ValueError("cos/sin must have one row of `dim` values per token")
    out = torch.empty_like(xc)
    nv.check(nv.cuda_lib().pkb_rope(nv.ptr(xc), nv.ptr(cs), nv.ptr(sn), nv.ptr(out), nv.c_ll(tokens), heads, dim, _dt(xc),
                                    nv.current_stream()), "pkb_rope")
    nv.count_launch()
    return out


def fp8_quantize_1x128(x: torch.Tensor, pow2_scales: bool = False):
    """e4m3 payload (uint8 view) + one fp32 scale per 128 consecutive elements of the last dimension.
    ``scale = amax / 448`` (1 when the block is all zero) as in reference/19_blocked_fp8_quantize.py:14-20;
    ``pow2_scales`` rounds the scale up to a power of two (UE8M0-compatible, exactly invertible)."""
    if x.shape[-1] % 128 != 0:
        raise ValueError("last dimension must be a multiple of 128")
    xc = x.contiguous()
    y = torch.empty(xc.shape, dtype=torch.uint8, device=x.device)
    s = torch.empty((*xc.shape[:-1], xc.shape[-1] // 128), dtype=torch.float32, device=x.device)
    nv.check(nv.cuda_lib().pkb_fp8_quant_1x128(nv.ptr(xc), nv.ptr(y), nv.ptr(s), nv.c_ll(xc.numel()), _dt(xc),
                                               1 if pow2_scales else 0, nv.current_stream()), "pkb_fp8_quant_1x128")
    nv.count_launch()
    return y, s


def fp8_dequantize_1x128(y: torch.Tensor, s: torch.Tensor, dtype: torch.dtype = torch.bfloat16,
                         valid_rows: torch.Tensor | None = None) -> torch.Tensor:
    """``y`` e4m3 bytes with one fp32 scale per 128 values. ``valid_rows`` (an int32 device scalar, for 2-D ``y``): only that
    many leading rows hold data - the rest of the result is left unwritten (a receive buffer sized for the worst case is
    dequantised as far as it was filled, without the count coming to the host)."""
    yc = y.contiguous().view(torch.uint8)
    out = torch.empty(yc.shape, dtype=dtype, device=y.device)
    if valid_rows is not None:
        if yc.dim() != 2 or valid_rows.dtype != torch.int32:
            raise ValueError("valid_rows needs a 2-D input and an int32 device scalar")
        nv.check(nv.cuda_lib().pkb_fp8_dequant_1x128_rows(nv.ptr(yc), nv.ptr(s.contiguous()), nv.ptr(out), nv.c_ll(yc.shape[0]),
                                                          nv.c_ll(yc.shape[1]), _DT[dtype], nv.ptr(valid_rows), nv.current_stream()),
                 "pkb_fp8_dequant_1x128_rows")
    else:
        nv.check(nv.cuda_lib().pkb_fp8_dequant_1x128(nv.ptr(yc), nv.ptr(s.contiguous()), nv.ptr(out), nv.c_ll(yc.numel()),
                                                     _DT[dtype], nv.current_stream()), "pkb_fp8_dequant_1x128")
    nv.count_launch()
    return out


def adam_step(p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, g: torch.Tensor, *, lr: float, beta1: float, beta2: float,
              eps: float, step: int, weight_decay: float = 0.0, decoupled: bool = True, grad_scale: float = 1.0,
              p_bf16: torch.Tensor | None = None) -> None:
    """In-place Adam / AdamW on fp32 ``p, m, v``; ``g`` is fp32 or bf16. ``p_bf16`` receives a bf16 copy."""
    for t in (p, m, v):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise TypeError("p, m, v must be contiguous fp32")
    nv.check(nv.cuda_lib().pkb_adam(nv.ptr(p), nv.ptr(m), nv.ptr(v), nv.ptr(g.contiguous()), nv.ptr(p_bf16),
                                    nv.c_ll(p.numel()), _dt(g), nv.c_float(lr), nv.c_float(beta1), nv.c_float(beta2),
                                    nv.c_float(eps), nv.c_float(weight_decay), nv.c_float(grad_scale), int(step),
                                    1 if decoupled else 0, nv.current_stream()), "pkb_adam")
    nv.count_launch()


def ce_local_stats(logits: torch.Tensor, target: torch.Tensor, vocab_start: int) -> torch.Tensor:
    """``[rows, 3]`` fp32: local max, sum exp(x - local max), target logit (0 if not on this rank)."""
    lc = logits.contiguous().view(-1, logits.shape[-1])
    rows, vl = lc.shape
    stats = torch.empty((rows, 3), dtype=torch.float32, device=logits.device)
    nv.check(nv.cuda_lib().pkb_ce_stats(nv.ptr(lc), nv.ptr(target.contiguous().view(-1).to(torch.int64)), nv.ptr(stats), rows,
                                        vl, nv.c_ll(vocab_start), _dt(lc), nv.current_stream()), "pkb_ce_stats")
    nv.count_launch()
    return stats


def ce_finalize(stats_all: torch.Tensor) -> torch.Tensor:
    """``stats_all`` is ``[W, rows, 3]``; returns the per-row loss ``[rows]`` (fp32)."""
    W, rows, _ = stats_all.shape
    loss = torch.empty(rows, dtype=torch.float32, device=stats_all.device)
    nv.check(nv.cuda_lib().pkb_ce_finalize(nv.ptr(stats_all.contiguous()), nv.ptr(loss), rows, W, nv.current_stream()),
             "pkb_ce_finalize")
    nv.count_launch()
    return loss


def vocab_parallel_cross_entropy(logits_local: torch.Tensor, target: torch.Tensor, comm, group=None) -> torch.Tensor:
    """Megatron-style vocab-parallel CE: one local pass, ONE packed exchange of three values per row
    (the reference issues three all-reduces: reference/73_vocab_parallel_cross_entropy_loss.py:22-40)."""
    g = comm.group(group)
    vl = logits_local.shape[-1]
    stats = ce_local_stats(logits_local, target, g.rank_in_group * vl)
    allst = comm.all_gather(stats, g)
    return ce_finalize(allst).view(target.shape)


def ln_bwd_colreduce(xhat: torch.Tensor, dy: torch.Tensor):
    """``dgamma = sum_rows dY * Xhat``, ``dbeta = sum_rows dY`` (fp32)."""
    xc, dc = xhat.contiguous(), dy.contiguous()
    rows, cols = xc.view(-1, xc.shape[-1]).shape
    dg = torch.empty(cols, dtype=torch.float32, device=xhat.device)
    db = torch.empty(cols, dtype=torch.float32, device=xhat.device)
    nv.check(nv.cuda_lib().pkb_ln_bwd_colreduce(nv.ptr(xc), nv.ptr(dc), nv.ptr(dg), nv.ptr(db), rows, cols, _dt(xc),
                                                nv.current_stream()), "pkb_ln_bwd_colreduce")
    nv.count_launch()
    return dg, db


def tp_rmsnorm(x_local: torch.Tensor, gamma_local: torch.Tensor, eps: float, group) -> torch.Tensor:
    """RMSNorm over a hidden dimension sharded across ``group`` (a SymmGroup): the cross-rank sum of
    squares is exchanged inside the kernel through the symmetric heap."""
    if x_local.dtype != torch.bfloat16:
        raise TypeError("tp_rmsnorm expects bf16")
    xc = x_local.contiguous().view(-1, x_local.shape[-1])
    rows, cl = xc.shape
    sums = group.heap.named(("tp_rms_sums", group.channel), (max(rows, 4),), torch.float32)
    y = torch.empty_like(xc)
    nv.check(nv.cuda_lib().pkb_tp_rmsnorm(group.ref, nv.ptr(xc), nv.ptr(gamma_local.contiguous()), nv.ptr(y), rows, cl,
                                          nv.c_ll(cl * group.size), nv.c_float(eps), ctypes.c_ulonglong(sums.offset),
                                          nv.current_stream()), "pkb_tp_rmsnorm")
    nv.count_launch()
    return y.view(x_local.shape)


def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    """``gu`` [rows, 2F] bf16 (gate columns, then up columns) -> ``silu(gate) * up`` [rows, F], one pass."""
    rows, F2 = gu.shape
    guc = gu.contiguous()
    out = torch.empty((rows, F2 // 2), dtype=gu.dtype, device=gu.device)
    nv.check(nv.cuda_lib().pkb_swiglu_fwd(nv.ptr(guc), nv.ptr(out), nv.c_ll(rows), F2 // 2, nv.current_stream()), "pkb_swiglu_fwd")
    nv.count_launch()
    return out


def swiglu_bwd(gu: torch.Tensor, da: torch.Tensor) -> torch.Tensor:
    """Gradient of :func:`swiglu_fwd` with respect to ``gu`` ([rows, 2F]), one pass."""
    rows, F2 = gu.shape
    guc, dac = gu.contiguous(), da.contiguous()
    dgu = torch.empty_like(guc)
    nv.check(nv.cuda_lib().pkb_swiglu_bwd(nv.ptr(guc), nv.ptr(dac), nv.ptr(dgu), nv.c_ll(rows), F2 // 2, nv.current_stream()),
             "pkb_swiglu_bwd")
    nv.count_launch()
    return dgu


def rmsnorm_bwd(x: torch.Tensor, gamma: torch.Tensor, dy: torch.Tensor, eps: float):
    """Backward of ``y = x * rsqrt(mean(x^2) + eps) * gamma`` for bf16 ``x, dy`` [rows, H]: returns (dx bf16, dgamma fp32)."""
    rows, H = x.shape
    xc, dyc, gc = x.contiguous(), dy.contiguous(), gamma.reshape(-1).contiguous()
    dx = torch.empty_like(xc)
    dg = torch.zeros(H, dtype=torch.float32, device=x.device)
    nv.check(nv.cuda_lib().pkb_rmsnorm_bwd(nv.ptr(xc), nv.ptr(gc), nv.ptr(dyc), nv.ptr(dx), nv.ptr(dg), rows, H, nv.c_float(eps),
                                           nv.current_stream()), "pkb_rmsnorm_bwd")
    nv.count_launch()
    return dx, dg


def ce_backward(logits: torch.Tensor, lse: torch.Tensor, target: torch.Tensor, vocab_start: int, scale: float,
                upstream: torch.Tensor | None = None) -> torch.Tensor:
    """``(softmax - onehot) * scale`` over a vocabulary shard, from the global log-sum-exp of every row (bf16, one pass).
    ``upstream`` is an optional fp32 device scalar multiplied in (the incoming gradient of the loss; no host read)."""
    rows, V = logits.shape
    lc = logits.contiguous()
    out = torch.empty_like(lc)
    nv.check(nv.cuda_lib().pkb_ce_bwd(nv.ptr(lc), nv.ptr(lse.float().contiguous()), nv.ptr(target.contiguous().view(-1).to(torch.int64)),
                                      nv.ptr(out), nv.c_ll(rows), V, nv.c_ll(vocab_start), nv.c_float(scale),
                                      nv.ptr(upstream.float().contiguous()) if upstream is not None else None, nv.current_stream()),
             "pkb_ce_bwd")
    nv.count_launch()
    return out
