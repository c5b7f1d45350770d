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


def kalman_block_step(H: torch.Tensor, err: torch.Tensor, w: torch.Tensor, P: torch.Tensor, lam: float, all_reduce=None):
    """One step of the block Kalman-filter optimiser in fp64 (reference: reference/63_deepmd_kalman_filter_optimizer.py:20-32).

    ``H``, ``w`` [nb, n, 1]; ``P`` [nb, n, n]; ``err`` a one-element tensor on the device; ``lam`` a host float. ``all_reduce``
    sums the one-element denominator over the ranks (``None`` on one rank). Returns ``(w_new [nb, n, 1], P_new [nb, n, n])``.
    Three launches read P twice and write it once; the denominator and the error never leave the device."""
    nb, n = P.shape[0], P.shape[1]
    for t in (H, w, P, err):
        if t.dtype != torch.float64 or not t.is_cuda:
            raise TypeError("fp64 CUDA tensors expected")
    if P.shape != (nb, n, n) or H.numel() != nb * n or w.numel() != nb * n or err.numel() != 1:
        raise ValueError("shapes: H, w [nb, n, 1]; P [nb, n, n]; err one element")
    Pc, Hc, wc, ec = P.contiguous(), H.contiguous(), w.contiguous(), err.reshape(1).contiguous()
    K = torch.empty((nb, n, 1), dtype=torch.float64, device=P.device)
    s = torch.empty(1, dtype=torch.float64, device=P.device)
    lib = nv.cuda_lib()
    nv.check(lib.pkb_kalman_gain(nv.ptr(Pc), nv.ptr(Hc), nv.ptr(K), nv.ptr(s), nv.c_ll(nb), n, ctypes.c_double(lam), nv.current_stream()),
             "pkb_kalman_gain")
    nv.count_launch(2)
    if all_reduce is not None:
        s = all_reduce(s).contiguous()
    P_new, w_new = torch.empty_like(Pc), torch.empty_like(wc)
    nv.check(lib.pkb_kalman_update(nv.ptr(Pc), nv.ptr(K), nv.ptr(wc), nv.ptr(ec), nv.ptr(s), nv.ptr(P_new), nv.ptr(w_new), nv.c_ll(nb), n,
                                   ctypes.c_double(lam), nv.current_stream()), "pkb_kalman_update")
    nv.count_launch()
    return w_new, P_new


def _sk_splits(B: int, want: int = 32) -> tuple[int, int]:
    """Row splits of the column pass: (number of splits, rows per split), no split empty."""
    rows = max(1, -(-B // want))
    return -(-B // rows), rows


def sinkhorn_rowdot(t: torch.Tensor, r: torch.Tensor, temp: float) -> torch.Tensor:
    """``v[b] = sum_p exp(t[b, p] / temp) * r[p]`` for ``t`` [B, P] fp32, without materialising the exponentials."""
    B, P = t.shape
    v = torch.empty(B, dtype=torch.float32, device=t.device)
    nv.check(nv.cuda_lib().pkb_sinkhorn_rowdot(nv.ptr(t), nv.ptr(r), nv.ptr(v), B, P, ctypes.c_double(temp), nv.current_stream()),
             "pkb_sinkhorn_rowdot")
    nv.count_launch()
    return v


def sinkhorn_coldot(t: torch.Tensor, c: torch.Tensor, temp: float) -> torch.Tensor:
    """``u[p] = sum_b exp(t[b, p] / temp) * c[b]``: partial sums per row split from the kernel, added here in a fixed order."""
    B, P = t.shape
    splits, _ = _sk_splits(B)
    partial = torch.empty((splits, P), dtype=torch.float32, device=t.device)
    nv.check(nv.cuda_lib().pkb_sinkhorn_coldot(nv.ptr(t), nv.ptr(c), nv.ptr(partial), B, P, splits, ctypes.c_double(temp), nv.current_stream()),
             "pkb_sinkhorn_coldot")
    nv.count_launch()
    return partial.sum(0) if splits > 1 else partial[0]


def sinkhorn_knopp(t: torch.Tensor, temp: float, iters: int, all_reduce=None) -> torch.Tensor:
    """Sinkhorn-Knopp normalisation of ``exp(t / temp)`` with the batch sharded over the ranks
    (reference: reference/80_dinov2_distributed_sinkhorn_knopp.py:16-35). ``t`` [B, P]; ``all_reduce`` sums a small fp32
    vector over the ranks (``None`` on one rank). The matrix is never rewritten: a scale per prototype and a scale per sample
    carry the iterations, each pass recomputes the exponentials from ``t``, and the result [B, P] is written once."""
    if not t.is_cuda:
        raise TypeError("CUDA tensor expected")
    t = t.float().contiguous()
    B, P = t.shape
    ar = all_reduce if all_reduce is not None else (lambda x: x)
    dev = t.device
    r = torch.ones(P, dtype=torch.float32, device=dev)
    head = ar(torch.stack([torch.tensor(float(B), device=dev), sinkhorn_rowdot(t, r, temp).sum()]))   # batch size and mass in one exchange
    total_batch, mass = head[0], head[1]
    c = torch.full((B,), 1.0, dtype=torch.float32, device=dev) / mass
    for _ in range(iters):
        R = ar((r * sinkhorn_coldot(t, c, temp)).contiguous())
        r = r / R / P
        c = c / (c * sinkhorn_rowdot(t, r, temp)) / total_batch
    cs = (c * total_batch).contiguous()
    out = torch.empty_like(t)
    nv.check(nv.cuda_lib().pkb_sinkhorn_scale(nv.ptr(t), nv.ptr(r), nv.ptr(cs), nv.ptr(out), B, P, ctypes.c_double(temp), nv.current_stream()),
             "pkb_sinkhorn_scale")
    nv.count_launch()
    return out
