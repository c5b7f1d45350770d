"""Python entry points of the small project-derived compute kernels (csrc/kernels/wild.cu)."""
from __future__ import annotations

import ctypes

import torch

from .. import _native as nv


def disco_contract(x: torch.Tensor, row_ptr: torch.Tensor, col: torch.Tensor, val: torch.Tensor, rows: int, nlon_out: int) -> torch.Tensor:
    """``x`` [BC, nlat_in, nlon_in] fp32; CSR (``row_ptr`` int32 [rows+1], ``col`` int32 = lat * nlon_in + lon, ``val`` fp32).
    Returns ``y`` [BC, rows, nlon_out] with ``y[b,r,p] = sum_e val[e] * x[b, lat_e, (lon_e + p*(nlon_in/nlon_out)) % nlon_in]``."""
    bc, nlat_in, nlon_in = x.shape
    xc = x.contiguous()
    y = torch.empty((bc, rows, nlon_out), dtype=torch.float32, device=x.device)
    nv.check(nv.cuda_lib().pkb_disco_contract(nv.ptr(xc), nv.ptr(row_ptr), nv.ptr(col), nv.ptr(val), nv.ptr(y), nv.c_ll(bc), rows,
                                              nlat_in, nlon_in, nlon_out, nv.current_stream()), "pkb_disco_contract")
    nv.count_launch()
    return y


def delta_rule_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """Gated delta-rule recurrence. ``q, k`` [BH, T, K]; ``v`` [BH, T, V]; ``decay`` [BH, T, K] or [BH, T, 1]; ``beta`` [BH, T]
    (all fp32, already normalised / activated). Returns ``out`` [BH, T, V] fp32."""
    BH, T, K = q.shape
    V = v.shape[-1]
    f = lambda t: t.float().contiguous()  # noqa: E731
    q, k, v, decay, beta = f(q), f(k), f(v), f(decay), f(beta)
    out = torch.empty((BH, T, V), dtype=torch.float32, device=q.device)
    nv.check(nv.cuda_lib().pkb_delta_rule_scan(nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(decay), nv.ptr(beta), nv.ptr(out), nv.c_ll(BH), T, K,
                                               V, decay.shape[-1], nv.current_stream()), "pkb_delta_rule_scan")
    nv.count_launch()
    return out


def halo_conv1d_zigzag(x: torch.Tensor, weight: torch.Tensor, group) -> torch.Tensor:
    """Depthwise causal conv1d of ``x`` [B, C, 2L] (this rank's two zigzag chunks) with ``weight`` [C, 1, KS]; the halos
    come from the neighbours' memory inside the same launch."""
    B, C, L2 = x.shape
    KS = weight.shape[-1]
    xc, wc = x.contiguous(), weight.reshape(C, KS).contiguous()
    if xc.dtype not in (torch.bfloat16, torch.float32) or wc.dtype != xc.dtype:
        raise TypeError("bf16 or fp32 tensors of one dtype expected")
    tails = group.heap.named(("halo1d_tails", group.channel, B, C, KS, str(x.dtype)), (2, B * C, KS - 1), x.dtype)
    y = torch.empty_like(xc)
    nv.check(nv.cuda_lib().pkb_halo_conv1d_zigzag(group.ref, nv.ptr(xc), nv.ptr(wc), nv.ptr(y), ctypes.c_ulonglong(tails.offset), B, C,
                                                  L2 // 2, KS, 0 if xc.dtype == torch.bfloat16 else 1, nv.current_stream()),
             "pkb_halo_conv1d_zigzag")
    nv.count_launch()
    return y
