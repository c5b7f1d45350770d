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


KNN_MAX_CANDIDATES = 4096


def knn_topk_local(sim: torch.Tensor, labels: torch.Tensor, k: int, classes: int | None = None):
    """The ``k`` most similar training rows per query (reference: reference/79_dinov2_distributed_knn.py:7-14).
    ``sim`` [R, N] fp32, ``labels`` int64 with N entries. With ``classes`` the similarities [R, k] and the class votes
    [R, classes] come back (the single-rank result); without, (similarity, label) pairs [R, k, 2] for the exchange."""
    R, N = sim.shape
    if sim.dtype != torch.float32 or labels.dtype != torch.int64 or labels.numel() != N or N > KNN_MAX_CANDIDATES:
        raise ValueError("fp32 similarities [R, N <= 4096] and N int64 labels expected")
    sc, lc = sim.contiguous(), labels.reshape(-1).contiguous()
    pairs = sims = votes = None
    if classes is None:
        pairs = torch.empty((R, k, 2), dtype=torch.float32, device=sim.device)
    else:
        sims = torch.empty((R, k), dtype=torch.float32, device=sim.device)
        votes = torch.empty((R, classes), dtype=torch.float32, device=sim.device)
    nv.check(nv.cuda_lib().pkb_knn_topk(nv.ptr(sc), nv.ptr(lc), nv.c_ll(R), nv.c_ll(N), nv.c_ll(0), 1, N, 1, k, classes or 0,
                                        nv.ptr(pairs) if pairs is not None else None, nv.ptr(sims) if sims is not None else None,
                                        nv.ptr(votes) if votes is not None else None, nv.current_stream()), "pkb_knn_topk")
    nv.count_launch()
    return pairs if classes is None else (sims, votes)


def knn_merge_votes(lists: torch.Tensor, k: int, classes: int):
    """Merge the candidate lists of all ranks (reference: reference/79_dinov2_distributed_knn.py:43-65): ``lists``
    [W, Q, k', 2] fp32 pairs as the exchange delivered them. Returns the ``k`` best similarities [Q, k] and the votes [Q, classes]."""
    W, Q, kk, two = lists.shape
    if lists.dtype != torch.float32 or two != 2 or W * kk > KNN_MAX_CANDIDATES:
        raise ValueError("fp32 pairs [W, Q, k, 2] with W * k <= 4096 expected")
    lc = lists.contiguous()
    sims = torch.empty((Q, k), dtype=torch.float32, device=lists.device)
    votes = torch.empty((Q, classes), dtype=torch.float32, device=lists.device)
    nv.check(nv.cuda_lib().pkb_knn_topk(nv.ptr(lc), None, nv.c_ll(Q), nv.c_ll(kk * 2), nv.c_ll(Q * kk * 2), W, kk, 2, k, classes, None,
                                        nv.ptr(sims), nv.ptr(votes), nv.current_stream()), "pkb_knn_topk")
    nv.count_launch()
    return sims, votes


def mask_iou_suppress(logits: torch.Tensor, last: torch.Tensor, threshold: float, reverse: bool = False) -> torch.Tensor:
    """Which of the ``n`` masks are suppressed by an overlapping mask that was occluded less recently
    (reference: reference/81_sam3_allgather_iou_suppression.py:30-48). ``logits`` [n, H, W] fp32 (a mask is ``logits > 0``),
    ``last`` int64 [n]. Returns a bool vector [n]. The masks are packed to one bit per pixel; the pairwise pass counts bits."""
    n = logits.shape[0]
    hw = logits[0].numel()
    if logits.dtype != torch.float32 or last.dtype != torch.int64 or last.numel() != n or hw % 32 != 0:
        raise ValueError("fp32 logits [n, H, W] with H * W a multiple of 32 and n int64 occlusion indices expected")
    lc, lastc = logits.contiguous(), last.contiguous()
    bits = torch.empty((n, hw // 32), dtype=torch.int32, device=logits.device)
    area = torch.empty(n, dtype=torch.int32, device=logits.device)
    sup = torch.zeros(n, dtype=torch.int32, device=logits.device)
    nv.check(nv.cuda_lib().pkb_mask_iou_suppress(nv.ptr(lc), nv.ptr(lastc), nv.ptr(bits), nv.ptr(area), nv.ptr(sup), n, hw,
                                                 ctypes.c_double(threshold), int(bool(reverse)), nv.current_stream()), "pkb_mask_iou_suppress")
    nv.count_launch(2 if n > 1 else 1)
    return sup.bool()


def siglip_loss_from_products(prod: torch.Tensor, scale: float, bias: float, diag_offset: int) -> torch.Tensor:
    """Sigmoid contrastive loss of this rank's images against all text blocks (reference: reference/58_openclip_contrastive_loss.py):
    ``prod`` [B, N] fp32 are the raw image-text products, the matching text of image ``i`` is column ``diag_offset + i``.
    Returns ``-sum logsigmoid(label * (scale * prod + bias)) / B`` as a 0-dim tensor; one pass over ``prod``."""
    B, N = prod.shape
    if prod.dtype != torch.float32 or not prod.is_cuda:
        raise TypeError("fp32 CUDA products expected")
    pc = prod.contiguous()
    blocks = min(B, 592)
    partial = torch.empty(blocks, dtype=torch.float32, device=prod.device)
    nv.check(nv.cuda_lib().pkb_siglip_loss_partials(nv.ptr(pc), nv.ptr(partial), B, N, diag_offset, ctypes.c_double(scale), ctypes.c_double(bias),
                                                    blocks, nv.current_stream()), "pkb_siglip_loss_partials")
    nv.count_launch()
    return partial.sum()
