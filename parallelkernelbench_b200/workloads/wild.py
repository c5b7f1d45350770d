"""Workloads taken from open-source projects (contrastive loss, distributed FFTs, Gaussian splatting, graph
sampling, recurrent attention, halo convolutions, sorting, ...).

Every op has the PyTorch + process-group restatement of what the project does (``reference``) and our form (``ours``):
the exchange runs on this package's symmetric-heap collectives (one launch each, peer loads land data in its final
layout) and the dense math on the tcgen05 GEMM where it is GEMM-shaped. FFTs stay on the FFT library in both forms.
Each section names the reference file it restates.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..harness.roofline import Cost
from ..utils.ragged import Ragged, compact_padded, permute_segments_padded
from .registry import OpSpec, RunCtx, register
from .ulysses import _a2a_ref


def _is_gloo() -> bool:
    return dist.is_initialized() and dist.get_backend() == "gloo"


def _ag_ref(t: torch.Tensor, W: int, group=None) -> torch.Tensor:
    """[W, *t.shape] over the process group."""
    if W == 1:
        return t.unsqueeze(0)
    parts = [torch.empty_like(t) for _ in range(W)]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.stack(parts)


def _mm_nt(rc: RunCtx, a: torch.Tensor, b: torch.Tensor, out_f32: bool = False) -> torch.Tensor:
    """``a[M,K] @ b[N,K]^T`` - tcgen05 GEMM for bf16 on a GPU, PyTorch otherwise."""
    if rc.dist.is_cuda and a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0:
        from ..ops import gemm_bf16

        return gemm_bf16(a.contiguous(), b.contiguous(), out_dtype=torch.float32 if out_f32 else torch.bfloat16)
    y = a.float() @ b.float().t()
    return y if out_f32 else y.to(a.dtype)


# =================================================================================================
# 58: sigmoid contrastive loss with text features visiting every rank (reference/58_openclip_contrastive_loss.py)
# =================================================================================================
def _siglip_inputs(rc: RunCtx, cfg):
    img = F.normalize(rc.randn(cfg["b_local"], cfg["d"], dtype=torch.float32), dim=-1).to(rc.dtype)
    txt = F.normalize(rc.randn(cfg["b_local"], cfg["d"], dtype=torch.float32, salt=1), dim=-1).to(rc.dtype)
    return (img, txt, 10.0, -10.0)


def _siglip_block(img, txt, scale, bias, negative_only):
    logits = scale * (img.float() @ txt.float().t()) + bias
    if negative_only:
        return -F.logsigmoid(-logits).sum() / img.shape[0]
    labels = -torch.ones_like(logits)
    labels.diagonal().fill_(1)
    return -F.logsigmoid(labels * logits).sum() / img.shape[0]


def _siglip_ref(rc, img, txt, scale, bias):
    """Neighbour ring: W - 1 hops, each a send/recv pair followed by a GEMM on the visiting block."""
    W, r = rc.world, rc.rank
    loss = _siglip_block(img, txt, scale, bias, False)
    cur = txt
    for _ in range(W - 1):
        nxt = torch.empty_like(cur)
        ops = [dist.P2POp(dist.isend, cur.contiguous(), (r + 1) % W), dist.P2POp(dist.irecv, nxt, (r - 1) % W)]
        for q in dist.batch_isend_irecv(ops):
            q.wait()
        loss = loss + _siglip_block(img, nxt, scale, bias, True)
        cur = nxt
    return loss


def _siglip_ours(rc, img, txt, scale, bias):
    """Every rank reads all text blocks at once (one gather launch), ONE GEMM against all of them, one reduction."""
    W, r = rc.world, rc.rank
    B = img.shape[0]
    allt = rc.comm.all_gather(txt.contiguous()).reshape(W * B, -1) if W > 1 else txt
    if rc.dist.is_cuda:
        from ..ops.wild import siglip_loss_from_products

        return siglip_loss_from_products(_mm_nt(rc, img, allt, out_f32=True), scale, bias, r * B)   # the whole epilogue in one pass
    logits = _mm_nt(rc, img, allt, out_f32=True) * scale + bias
    sign = -torch.ones_like(logits)
    idx = torch.arange(B, device=img.device)
    sign[idx, r * B + idx] = 1.0
    return -F.logsigmoid(sign * logits).sum() / B


register(OpSpec(name="siglip_loss", problem_ids=(58,), group="wild",
                configs={"default": {"b_local": 128, "d": 1024}, "small": {"b_local": 8, "d": 16}, "large": {"b_local": 4096, "d": 1024}},
                make_inputs=_siglip_inputs, reference=_siglip_ref, ours=_siglip_ours, atol=5e-2, rtol=2e-2,
                cost=lambda cfg, W: Cost(flops=2.0 * cfg["b_local"] ** 2 * W * cfg["d"], nvlink_bytes=(W - 1) * cfg["b_local"] * cfg["d"] * 2)))


# =================================================================================================
# 59 / 60: 2-D real FFT and its inverse with one dimension sharded
# (reference/59_physicsnemo_distributed_rfft.py, reference/60_physicsnemo_distributed_irfft.py)
# =================================================================================================
def _a2a_c(rc, x: torch.Tensor, sd: int, gd: int, ours: bool) -> torch.Tensor:
    """Permuting all-to-all of a complex tensor (moved as pairs of floats)."""
    if rc.world == 1:
        return x.contiguous()
    xr = torch.view_as_real(x.contiguous())
    sd, gd = sd % x.ndim, gd % x.ndim
    y = rc.comm.all_to_all_permute(xr, sd, gd) if ours else _a2a_ref(xr, sd, gd, rc.world)
    return torch.view_as_complex(y.contiguous())


def _rfft_inputs(rc: RunCtx, cfg):
    W = rc.world
    H, Wd = cfg["h"], cfg["w"]
    full = torch.randn(cfg["b"], H, Wd, device=rc.device, generator=rc.gen(shared=True))
    wl = Wd // W
    return (full[:, :, rc.rank * wl:(rc.rank + 1) * wl].contiguous(), (H, Wd))


def _rfft(rc, x, s, ours):
    x1 = torch.fft.fft(x, n=s[0], dim=1, norm="ortho")              # along the unsharded dimension
    x1 = _a2a_c(rc, x1, 1, 2, ours)                                  # now dim 1 is sharded and dim 2 is whole
    x2 = torch.fft.fft(x1, n=s[1], dim=2, norm="ortho")
    return torch.view_as_real(x2[:, :, :x2.shape[2] // 2 + 1].contiguous())


register(OpSpec(name="distributed_rfft2", problem_ids=(59,), group="wild",
                configs={"default": {"b": 16, "h": 1024, "w": 1024}, "small": {"b": 2, "h": 16, "w": 16}},
                make_inputs=_rfft_inputs, reference=lambda rc, x, s: _rfft(rc, x, s, False), ours=lambda rc, x, s: _rfft(rc, x, s, True),
                atol=1e-3, rtol=1e-3,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["b"] * cfg["h"] * cfg["w"] / max(W, 1) * 8 * (W - 1) / max(W, 1))))


def _irfft_inputs(rc: RunCtx, cfg):
    W = rc.world
    B, C, H, Wd = cfg["b"], cfg["c"], cfg["h"], cfg["w"]
    real = torch.randn(B, C, H, Wd, device=rc.device, generator=rc.gen(shared=True))
    spec = torch.fft.rfft2(real, s=(H, Wd), dim=(-2, -1), norm="ortho")
    hl = H // W
    return (spec[:, :, rc.rank * hl:(rc.rank + 1) * hl].contiguous(), (H, Wd))


def _irfft_ref(rc, x, s):
    """Hermitian completion through an all-gather of the whole padded spectrum, as the project does it."""
    W, r = rc.world, rc.rank
    H, Wd = s
    orig = x.shape[-1]
    pad = F.pad(x, (0, Wd - orig))
    pad[..., orig:] = torch.flip(torch.conj(pad[..., 1:Wd - orig + 1]), dims=[-1])
    if W > 1:
        full = torch.view_as_complex(_ag_ref(torch.view_as_real(pad.contiguous()), W).contiguous())   # [W, B, C, hl, Wd]
        full = full.permute(1, 2, 0, 3, 4).reshape(pad.shape[0], pad.shape[1], H, Wd).contiguous()
    else:
        full = pad
    full[:, :, 1:, orig:] = torch.flip(full[:, :, 1:, orig:], dims=[2])
    hl = H // W
    mine = full[:, :, r * hl:(r + 1) * hl].contiguous()
    x1 = torch.fft.ifft(mine, n=Wd, dim=-1, norm="ortho")
    x1 = _a2a_c(rc, x1, 3, 2, False)
    return torch.fft.ifft(x1, n=H, dim=2, norm="ortho").real.contiguous()


def _irfft_ours(rc, x, s):
    """The Hermitian half of row h is the conjugate of row (H - h) % H: fetch just those rows from their owners with
    the remote row-gather kernel (1/W of the traffic of gathering everything), then the same two FFT passes."""
    W, r = rc.world, rc.rank
    H, Wd = s
    B, C, hl, orig = x.shape
    rows = torch.view_as_real(x.permute(2, 0, 1, 3).contiguous())                      # [hl, B, C, orig, 2]
    want = (H - torch.arange(r * hl, (r + 1) * hl, device=x.device)) % H
    mirror = torch.view_as_complex(rc.comm.row_gather(rows, want).contiguous()).permute(1, 2, 0, 3)   # [B, C, hl, orig]
    pad = torch.empty((B, C, hl, Wd), dtype=x.dtype, device=x.device)
    pad[..., :orig] = x
    pad[..., orig:] = torch.flip(torch.conj(mirror[..., 1:Wd - orig + 1]), dims=[-1])
    x1 = torch.fft.ifft(pad, n=Wd, dim=-1, norm="ortho")
    x1 = _a2a_c(rc, x1, 3, 2, True)
    return torch.fft.ifft(x1, n=H, dim=2, norm="ortho").real.contiguous()


register(OpSpec(name="distributed_irfft2", problem_ids=(60,), group="wild",
                configs={"default": {"b": 2, "c": 10, "h": 720, "w": 1440}, "small": {"b": 1, "c": 2, "h": 16, "w": 32}},
                make_inputs=_irfft_inputs, reference=_irfft_ref, ours=_irfft_ours, atol=1e-3, rtol=1e-3,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["b"] * cfg["c"] * cfg["h"] * cfg["w"] / max(W, 1) * 8 * (W - 1) / max(W, 1))))


# =================================================================================================
# 61: Gaussian-splat projection, survivors redistributed to the rank that owns each camera
# (reference/61_gsplat_3d_gaussian_splatting.py)
# =================================================================================================
def _gs_inputs(rc: RunCtx, cfg):
    n, D = cfg["n_local"], 3
    means = torch.stack([(rc.rand(n) - 0.5) * 1.5, (rc.rand(n, salt=1) - 0.5) * 1.5, rc.rand(n, salt=2) * 2.0 + 2.0], -1).to(rc.dtype)
    quats = rc.randn(n, 4, salt=3)
    scales = (rc.rand(n, 3, salt=4) * 0.02).to(rc.dtype)
    opac = (rc.rand(n, salt=5) * 0.8 + 0.1).to(rc.dtype)
    colors = rc.rand(n, D, salt=6).to(rc.dtype)
    w, h = cfg["width"], cfg["height"]
    view = torch.eye(4, device=rc.device).reshape(1, 4, 4).repeat(cfg["cams"], 1, 1)
    view[:, 0, 3] = 0.05 * rc.rank                                   # every rank looks from a slightly different place
    K = torch.eye(3, device=rc.device).reshape(1, 3, 3).repeat(cfg["cams"], 1, 1)
    K[:, 0, 0] = K[:, 1, 1] = 0.8 * min(w, h)
    K[:, 0, 2], K[:, 1, 2] = w * 0.5, h * 0.5
    return (means, quats, scales, opac, colors, view.to(rc.dtype), K.to(rc.dtype), w, h)


def _gs_pad(rc, cap, cam, gid, radii, m2, depth, con, op, col, count):
    """Fixed-capacity outputs so that both implementations return tensors of the same shape."""
    def pad(t):
        out = torch.zeros((cap, *t.shape[1:]), dtype=t.dtype, device=t.device)
        out[:t.shape[0]] = t
        return out
    return {"count": count, "camera_ids": pad(cam), "gaussian_ids": pad(gid), "radii": pad(radii), "means2d": pad(m2),
            "depths": pad(depth), "conics": pad(con), "opacities": pad(op), "colors": pad(col)}


def _gs_ref(rc, means, quats, scales, opac, colors, view, K, w, h):
    from ..refs.gsplat import project

    W, N, C = rc.world, means.shape[0], view.shape[0]
    Va = _ag_ref(view.float(), W).reshape(W * C, 4, 4)
    Ka = _ag_ref(K.float(), W).reshape(W * C, 3, 3)
    radii, m2, depth, con = project(means, quats, scales, Va, Ka, w, h)
    valid = (radii > 0).all(-1)                                      # [W*C, N]
    cam, gid = torch.where(valid)
    rows = [radii[valid].float(), m2[valid], depth[valid][:, None], con[valid], opac.float()[gid][:, None], colors.float()[gid],
            (cam % C).float()[:, None], (gid + rc.rank * N).float()[:, None]]
    data = torch.cat(rows, -1)
    counts = torch.bincount(cam // C, minlength=W)
    if W > 1:
        recv_counts = torch.empty_like(counts)
        if _is_gloo():
            allc = _ag_ref(counts, W)
            recv_counts = allc[:, rc.rank].contiguous()
            alld = [torch.empty((int(allc[s].sum()), data.shape[1]), device=data.device) for s in range(W)]
            padded = torch.zeros((int(allc.sum(1).max()), data.shape[1]), device=data.device)
            padded[:data.shape[0]] = data
            got = _ag_ref(padded, W)
            parts = []
            for s in range(W):
                off = int(allc[s, :rc.rank].sum())
                parts.append(got[s, off:off + int(allc[s, rc.rank])])
            data = torch.cat(parts)
            del alld
        else:
            dist.all_to_all_single(recv_counts, counts)
            out = torch.empty((int(recv_counts.sum()), data.shape[1]), device=data.device)
            dist.all_to_all_single(out, data, output_split_sizes=recv_counts.tolist(), input_split_sizes=counts.tolist())
            data = out
    D = colors.shape[1]
    cnt = torch.tensor(data.shape[0], dtype=torch.int32, device=data.device)
    return _gs_pad(rc, W * N * C, data[:, 9 + D].int(), data[:, 10 + D].int(), data[:, 0:2].int(), data[:, 2:4], data[:, 4], data[:, 5:8],
                   data[:, 8], data[:, 9:9 + D], cnt)


def _gs_ours(rc, means, quats, scales, opac, colors, view, K, w, h):
    W, N, C = rc.world, means.shape[0], view.shape[0]
    if not rc.dist.is_cuda:
        return _gs_ref(rc, means, quats, scales, opac, colors, view, K, w, h)
    from ..ops.gsplat import HEADER_WORDS, gsplat_project_exchange

    g = rc.comm.group()
    cams = torch.cat([view.float().reshape(C, 16), K.float().reshape(C, 9)], 1)
    allc = rc.comm.all_gather(cams).reshape(W * C, 25) if W > 1 else cams
    rec, count = gsplat_project_exchange(g, means, quats, scales, opac, colors, allc[:, :16], allc[:, 16:], C, w, h)
    D = colors.shape[1]
    keep = (torch.arange(rec.shape[0], device=rec.device) < count)[:, None]
    rec = torch.where(keep, rec, torch.zeros_like(rec))
    fl = rec.view(torch.float32)
    return {"count": count.clone(), "camera_ids": rec[:, 0], "gaussian_ids": rec[:, 1], "radii": rec[:, 2:4], "means2d": fl[:, 4:6],
            "depths": fl[:, 6], "conics": fl[:, 7:10], "opacities": fl[:, 10], "colors": fl[:, HEADER_WORDS:HEADER_WORDS + D]}


register(OpSpec(name="gsplat_projection", problem_ids=(61,), group="wild",
                configs={"default": {"n_local": 1024, "cams": 1, "width": 512, "height": 512},
                         "small": {"n_local": 300, "cams": 2, "width": 64, "height": 64},
                         "large": {"n_local": 100000, "cams": 2, "width": 1920, "height": 1080}},
                make_inputs=_gs_inputs, reference=_gs_ref, ours=_gs_ours, atol=1e-5, rtol=1e-5,
                doc="projection + culling + ordered compaction + peer stores in three launches; pure arithmetic, no graphics API"))


# =================================================================================================
# 62: discrete-continuous convolution on the sphere over a polar x azimuth mesh
# (reference/62_torchharmonics_spherical_convolution.py)
# =================================================================================================
def _disco_mesh(rc: RunCtx):
    from ..parallel.mesh import Mesh2D

    if "disco_mesh" not in rc.cache:
        az = 2 if rc.world % 2 == 0 else 1
        rc.cache["disco_mesh"] = Mesh2D.build(rc.world, az, rc.rank, inner_name="azimuth", outer_name="polar")
    return rc.cache["disco_mesh"]


def _disco_inputs(rc: RunCtx, cfg):
    m = _disco_mesh(rc)
    az, pol = m.inner, m.outer
    B, C, Ksz = cfg["batch"], cfg["chans"], 3
    nlat = -(-cfg["nlat"] // pol) * pol
    nlon = -(-2 * nlat // az) * az
    nlat_l, nlon_l = nlat // pol, nlon // az
    x = rc.randn(B, C, nlat_l, nlon_l, dtype=torch.float32)
    weight = rc.randn(C, C, Ksz, dtype=torch.float32, shared=True, salt=1)
    bias = rc.randn(C, dtype=torch.float32, shared=True, salt=2)
    # sparse filter: a few entries per (kernel, output latitude) row, columns inside this rank's latitude band
    E = min(4, nlat_l * nlon)
    k_idx = torch.arange(Ksz, device=rc.device).view(-1, 1, 1).expand(Ksz, nlat, E)
    o_idx = torch.arange(nlat, device=rc.device).view(1, -1, 1).expand(Ksz, nlat, E)
    e_idx = torch.arange(E, device=rc.device).view(1, 1, -1).expand(Ksz, nlat, E)
    lat_l = (o_idx - m.outer_rank * nlat_l) % nlat_l
    lon = (o_idx + e_idx * (k_idx + 1)) % nlon
    cols = (lat_l * nlon + lon).reshape(-1).int()
    vals = (torch.randn(Ksz * nlat * E, device=rc.device, generator=rc.gen(salt=3)) * 0.05)
    row_ptr = (torch.arange(Ksz * nlat + 1, device=rc.device) * E).int()
    return (x, row_ptr, cols, vals, weight, bias, nlat, nlon)


def _disco_contract_torch(x, row_ptr, cols, vals, rows, nlon_out):
    BC, nlat_in, nlon_in = x.shape
    E = cols.numel() // rows
    lat = (cols.long() // nlon_in).view(rows, E)
    lon = (cols.long() % nlon_in).view(rows, E)
    p = torch.arange(nlon_out, device=x.device) * (nlon_in // nlon_out)
    y = torch.zeros((BC, rows, nlon_out), dtype=x.dtype, device=x.device)
    for e in range(E):
        idx = (lon[:, e, None] + p[None, :]) % nlon_in                   # [rows, P]
        y += vals.view(rows, E)[:, e].view(1, rows, 1) * x[:, lat[:, e]].gather(2, idx.unsqueeze(0).expand(BC, -1, -1))
    return y


def _disco(rc, x, row_ptr, cols, vals, weight, bias, nlat, nlon, ours):
    m = _disco_mesh(rc)
    az, pol = m.inner, m.outer
    B, C, nlat_l, nlon_l = x.shape
    Ksz = weight.shape[2]
    def a2a(t, sd, gd):
        if az == 1:
            return t
        if ours:
            return rc.comm.all_to_all_permute(t, sd, gd, group=m.inner_ranks)
        ins = [c.contiguous() for c in t.chunk(az, dim=sd)]
        outs = [torch.empty_like(ins[0]) for _ in range(az)]
        if _is_gloo():
            for i, src in enumerate(m.inner_ranks):
                buf = torch.stack(ins) if src == rc.rank else torch.empty((az, *ins[0].shape), dtype=t.dtype, device=t.device)
                dist.broadcast(buf, src, group=m.inner_group)
                outs[i].copy_(buf[m.inner_rank])
        else:
            dist.all_to_all(outs, ins, group=m.inner_group)
        return torch.cat(outs, dim=gd).contiguous()
    xt = a2a(x, 1, 3)                                                      # [B, C/az, nlat_l, nlon]
    Cl = xt.shape[1]
    rows = Ksz * nlat
    if ours and rc.dist.is_cuda:
        from ..ops.wild import disco_contract

        y = disco_contract(xt.reshape(B * Cl, nlat_l, nlon), row_ptr, cols, vals, rows, nlon)
    else:
        y = _disco_contract_torch(xt.reshape(B * Cl, nlat_l, nlon), row_ptr, cols, vals, rows, nlon)
    y = y.view(B, Cl, Ksz, nlat, nlon)
    if pol > 1:                                                             # sum the latitude-band contributions, keep my band
        if ours:
            yl = rc.comm.reduce_scatter(y.permute(3, 0, 1, 2, 4).contiguous(), group=m.outer_ranks).permute(1, 2, 3, 0, 4).contiguous()
        else:
            yf = y.contiguous()
            dist.all_reduce(yf, group=m.outer_group)
            yl = yf[:, :, :, m.outer_rank * nlat_l:(m.outer_rank + 1) * nlat_l].contiguous()
    else:
        yl = y
    yl = a2a(yl, 4, 1)                                                      # [B, C, K, nlat_l, nlon/az]
    out = torch.einsum("bckxy,ock->boxy", yl, weight)
    return out + bias.view(1, -1, 1, 1)


register(OpSpec(name="disco_s2_convolution", problem_ids=(62,), group="wild",
                configs={"default": {"batch": 32, "chans": 8, "nlat": 128}, "small": {"batch": 2, "chans": 4, "nlat": 8}},
                make_inputs=_disco_inputs, reference=lambda rc, *a: _disco(rc, *a, ours=False), ours=lambda rc, *a: _disco(rc, *a, ours=True),
                atol=1e-3, rtol=1e-3))


# =================================================================================================
# 63: block Kalman-filter optimiser step in fp64 (reference/63_deepmd_kalman_filter_optimizer.py)
# =================================================================================================
def _kalman_inputs(rc: RunCtx, cfg):
    nb, n = cfg["blocks"], cfg["block"]
    H = rc.randn(nb, n, 1, dtype=torch.float64) * 0.01
    w = rc.randn(nb, n, 1, dtype=torch.float64, salt=1)
    P = torch.eye(n, dtype=torch.float64, device=rc.device).repeat(nb, 1, 1) + 0.01 * rc.randn(nb, n, n, dtype=torch.float64, salt=2)
    P = 0.5 * (P + P.transpose(1, 2))
    err = rc.randn(1, dtype=torch.float64, salt=3).reshape(())
    return (H, err, w, P, 0.98, 0.9987)


def _kalman(rc, H, err, w, P, lam, nue, ours):
    """All blocks batched (the project loops over them); the scalar and the weights cross ranks."""
    W = rc.world
    if ours and rc.dist.is_cuda and P.dtype == torch.float64:
        from ..ops.wild import kalman_block_step

        w_new, P_new = kalman_block_step(H, err, w, P, lam, all_reduce=rc.comm.all_reduce if W > 1 else None)
        allw = rc.comm.all_gather(w_new) if W > 1 else w_new.unsqueeze(0)
        lam_next = torch.tensor(nue * lam + 1 - nue, dtype=torch.float64, device=H.device)
        return {"weights": allw.reshape(-1, w.shape[1], 1), "P": P_new, "lambda": lam_next}
    K = torch.bmm(P, H)                                                   # [nb, n, 1]
    tmp = (lam + torch.bmm(H.transpose(1, 2), K)).sum().reshape(1)
    if W > 1:
        tmp = rc.comm.all_reduce(tmp) if ours else _allreduce_ref(tmp)
    A = 1.0 / tmp
    w_new = w + A * err * K
    P_new = (1.0 / lam) * (P - A * torch.bmm(K, K.transpose(1, 2)))
    if W > 1:
        allw = rc.comm.all_gather(w_new.contiguous()) if ours else _ag_ref(w_new.contiguous(), W)
    else:
        allw = w_new.unsqueeze(0)
    lam_next = torch.tensor(nue * lam + 1 - nue, dtype=torch.float64, device=H.device)
    return {"weights": allw.reshape(-1, w.shape[1], 1), "P": P_new, "lambda": lam_next}


def _allreduce_ref(t):
    t = t.clone()
    dist.all_reduce(t)
    return t


register(OpSpec(name="kalman_filter_step", problem_ids=(63,), group="wild",
                configs={"default": {"blocks": 8, "block": 1024}, "small": {"blocks": 2, "block": 16}},
                make_inputs=_kalman_inputs, reference=lambda rc, *a: _kalman(rc, *a, ours=False), ours=lambda rc, *a: _kalman(rc, *a, ours=True),
                atol=1e-9, rtol=1e-9,
                cost=lambda cfg, W: Cost(hbm_bytes=3.0 * cfg["blocks"] * cfg["block"] ** 2 * 8)))   # P read twice, written once


# =================================================================================================
# graph workloads (64-69)
# =================================================================================================
def _a2av_ref(x: torch.Tensor, send_counts: torch.Tensor):
    """Variable all-to-all over the world group with the host round trip the projects pay. Returns (rows, recv_counts)."""
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts)
    rs, ss = recv_counts.tolist(), send_counts.tolist()
    out = x.new_empty((sum(rs), *x.shape[1:]))
    dist.all_to_all_single(out, x.contiguous(), output_split_sizes=rs, input_split_sizes=ss)
    return out, recv_counts


def _heap_copy(rc: RunCtx, name: str, t: torch.Tensor):
    """A tensor that does not change during the job (graph structure, embedding table), placed in the symmetric heap
    once so that peers can read it in place."""
    key = (name, t.data_ptr(), tuple(t.shape))
    if key not in rc.cache:
        buf = rc.comm.heap.named((name, tuple(t.shape), str(t.dtype)), t.shape, t.dtype)
        buf.local.copy_(t)
        rc.comm.barrier()
        rc.cache[key] = buf.local
    return rc.cache[key]


def _remote_rows(rc: RunCtx, name: str, table: torch.Tensor, owner: torch.Tensor, local_idx: torch.Tensor) -> torch.Tensor:
    """``table_of_rank(owner[i])[local_idx[i]]`` for every i: direct peer loads on a GPU, a gather of the tables on CPU."""
    n = table.shape[0]
    if rc.world == 1:
        return table[local_idx]
    if rc.dist.is_cuda:
        from ..ops.collectives import row_gather

        return row_gather(_heap_copy(rc, name, table), owner * n + local_idx, rc.comm.group(), resident=True)
    return rc.comm.row_gather(table, owner * n + local_idx)


# ---- 64: two-hop neighbour sampling (reference/64_gnn_neighbor_sampling.py) -----------------------
def _gnn_inputs(rc: RunCtx, cfg):
    W = rc.world
    n = -(-cfg["nodes"] // W) * W
    deg = cfg["degree"]
    colptr = torch.arange(n + 1, device=rc.device, dtype=torch.int64) * deg
    row = ((torch.arange(n, device=rc.device).unsqueeze(1) + torch.arange(1, deg + 1, device=rc.device).unsqueeze(0)) % n).reshape(-1)
    node_to_rank = torch.arange(n, device=rc.device) % W
    seeds = (torch.arange(cfg["seeds"], device=rc.device) + rc.rank * cfg["seeds"]) % n
    return (seeds, list(cfg["fanouts"]), colptr, row.contiguous(), node_to_rank)


def _first_seen_unique(node: torch.Tensor, out_node: torch.Tensor):
    """Unique values of cat(node, out_node) in order of first appearance; also the new ones only."""
    comb = torch.cat([node, out_node])
    uniq, inv = torch.unique(comb, return_inverse=True)
    first = torch.full((uniq.numel(),), comb.numel(), dtype=torch.int64, device=comb.device)
    first.scatter_reduce_(0, inv, torch.arange(comb.numel(), device=comb.device), reduce="amin")
    order = first.sort().values
    allnodes = comb[order]
    return allnodes[node.numel():], allnodes


def _gnn_finish(node, node_dupl, dst_dupl, edges):
    if node_dupl.numel() == 0:
        return {"node": node, "row": node.new_empty(0), "col": node.new_empty(0), "edge": edges}
    assoc = torch.full((int(node.max()) + 1,), -1, dtype=torch.int64, device=node.device)
    assoc[node] = torch.arange(node.numel(), device=node.device)
    return {"node": node, "row": assoc[node_dupl], "col": assoc[dst_dupl], "edge": edges}


def _gnn_ref(rc, seeds, fanouts, colptr, row, node_to_rank):
    """Requests routed to the owners, owners sample, replies routed back (five exchanges per hop with host syncs)."""
    W = rc.world
    src, node = seeds.clone(), seeds.clone()
    nd, dd, ed = [seeds.new_empty(0)], [seeds.new_empty(0)], [seeds.new_empty(0)]
    for k in fanouts:
        owner = node_to_rank[src]
        order = torch.argsort(owner, stable=True)
        req = src[order]
        if W > 1:
            got, recv_counts = _a2av_ref(req, torch.bincount(owner, minlength=W))
        else:
            got, recv_counts = req, torch.tensor([req.numel()], device=req.device)
        start = colptr[got]
        take = torch.clamp(colptr[got + 1] - start, max=k)
        j = torch.arange(k, device=src.device)[None, :]
        valid = j < take[:, None]
        eid = (start[:, None] + j)[valid]
        nbr = row[eid]
        if W > 1:
            bounds = torch.cumsum(recv_counts, 0)
            seg = torch.searchsorted(bounds, torch.arange(got.numel(), device=src.device), right=True)
            per_dst = torch.zeros(W, dtype=torch.int64, device=src.device).index_add_(0, seg, take)
            nbr_b, _ = _a2av_ref(nbr, per_dst)
            eid_b, _ = _a2av_ref(eid, per_dst)
            take_b, _ = _a2av_ref(take, recv_counts)
        else:
            nbr_b, eid_b, take_b = nbr, eid, take
        # replies arrive grouped by owner in request order: put them back into the order of `src`
        take_src = torch.empty_like(take_b)
        take_src[order] = take_b
        starts_sorted = torch.cumsum(take_b, 0) - take_b
        starts_src = torch.empty_like(starts_sorted)
        starts_src[order] = starts_sorted
        jj = torch.arange(k, device=src.device)[None, :]
        vsrc = jj < take_src[:, None]
        pos = (starts_src[:, None] + jj)[vsrc]
        out_node, out_edge = nbr_b[pos], eid_b[pos]
        out_dst = src[:, None].expand(-1, k)[vsrc]
        if out_node.numel() == 0:
            break
        src, node = _first_seen_unique(node, out_node)
        nd.append(out_node); dd.append(out_dst); ed.append(out_edge)
    return _gnn_finish(node, torch.cat(nd), torch.cat(dd), torch.cat(ed))


def _gnn_ours(rc, seeds, fanouts, colptr, row, node_to_rank):
    """The requester reads the owner's adjacency in place: per hop two remote row gathers (degree bounds, neighbours),
    no request/reply exchange and no host round trip for split sizes."""
    src, node = seeds.clone(), seeds.clone()
    nd, dd, ed = [seeds.new_empty(0)], [seeds.new_empty(0)], [seeds.new_empty(0)]
    for k in fanouts:
        owner = node_to_rank[src]
        bounds = _remote_rows(rc, "gnn_colptr", colptr, torch.cat([owner, owner]), torch.cat([src, src + 1]))
        start, end = bounds[:src.numel()], bounds[src.numel():]
        take = torch.clamp(end - start, max=k)
        j = torch.arange(k, device=src.device)[None, :]
        valid = j < take[:, None]
        eid = (start[:, None] + j)[valid]
        out_node = _remote_rows(rc, "gnn_row", row, owner[:, None].expand(-1, k)[valid], eid)
        out_dst = src[:, None].expand(-1, k)[valid]
        if out_node.numel() == 0:
            break
        src, node = _first_seen_unique(node, out_node)
        nd.append(out_node); dd.append(out_dst); ed.append(eid)
    return _gnn_finish(node, torch.cat(nd), torch.cat(dd), torch.cat(ed))


register(OpSpec(name="gnn_neighbor_sampling", problem_ids=(64,), group="wild",
                configs={"default": {"nodes": 10000, "degree": 16, "seeds": 512, "fanouts": (10, 5)},
                         "small": {"nodes": 64, "degree": 4, "seeds": 8, "fanouts": (3, 2)}},
                make_inputs=_gnn_inputs, reference=_gnn_ref, ours=_gnn_ours, atol=0, rtol=0))


# ---- 65 / 66: feature exchange forward and backward -------------------------------------------------
def _fx_inputs(rc: RunCtx, cfg):
    W = rc.world
    R, Hd = cfg["rows_per_peer"], cfg["hidden"]
    seed_size = max(1, R * W * 3 // 4)
    return (rc.randn(seed_size, Hd), rc.randint(0, seed_size, (R * W,), salt=1), R)


def _rot_dst(j, r, W):
    return (j + r) % W          # chunk j of rank r goes to rank (j + r) % W and arrives as chunk (r_src - r_dst) % W


def _fx_ref(rc, feats, ids, R):
    W, r = rc.world, rc.rank
    gathered = feats[ids]
    if W == 1:
        return gathered
    chunks = list(gathered.split(R))
    send = torch.stack([chunks[(d - r) % W] for d in range(W)])           # indexed by destination
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send)
    return torch.cat([recv[(j + r) % W] for j in range(W)])               # chunk j came from rank (j + r) % W


def _fx_ours(rc, feats, ids, R):
    """Only the row ids travel ahead (a few KB); the rows are then read from the owners' feature tables straight into
    their final place, so the gathered copy is never materialised at the source."""
    W, r = rc.world, rc.rank
    if W == 1:
        return feats[ids]
    all_ids = rc.comm.all_gather(ids.contiguous())                        # [W, W*R]
    j = torch.arange(W, device=feats.device)
    s = (j + r) % W                                                        # source of my chunk j
    js = (r - s) % W                                                       # which of its chunks that is
    want = all_ids[s[:, None], (js * R)[:, None] + torch.arange(R, device=feats.device)[None, :]]     # [W, R]
    return rc.comm.row_gather(feats, (s[:, None] * feats.shape[0] + want).reshape(-1))


register(OpSpec(name="gnn_feature_exchange", problem_ids=(65,), group="wild",
                configs={"default": {"rows_per_peer": 128, "hidden": 128}, "small": {"rows_per_peer": 4, "hidden": 8},
                         "large": {"rows_per_peer": 16384, "hidden": 256}},
                make_inputs=_fx_inputs, reference=_fx_ref, ours=_fx_ours, atol=0, rtol=0,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["rows_per_peer"] * (W - 1) * cfg["hidden"] * 2)))


def _fxb_inputs(rc: RunCtx, cfg):
    W = rc.world
    R, Hd = cfg["rows_per_peer"], cfg["hidden"]
    seed_size = max(1, R * W // 2)
    return (rc.randn(R * W, Hd, dtype=torch.float32), rc.randint(0, seed_size, (R * W,), salt=1), seed_size, R)


def _fxb(rc, grad, ids, seed_size, R, ours):
    W, r = rc.world, rc.rank
    if W > 1:
        chunks = list(grad.split(R))
        send = torch.stack([chunks[(d - r) % W] for d in range(W)])
        if ours:
            recv = rc.comm.all_to_all(send)
        else:
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send)
        got = torch.cat([recv[(j + r) % W] for j in range(W)])
    else:
        got = grad
    return torch.zeros((seed_size, grad.shape[1]), dtype=grad.dtype, device=grad.device).index_add_(0, ids, got)


register(OpSpec(name="gnn_feature_exchange_backward", problem_ids=(66,), group="wild",
                configs={"default": {"rows_per_peer": 128, "hidden": 128}, "small": {"rows_per_peer": 4, "hidden": 8}},
                make_inputs=_fxb_inputs, reference=lambda rc, *a: _fxb(rc, *a, ours=False), ours=lambda rc, *a: _fxb(rc, *a, ours=True),
                atol=1e-4, rtol=1e-4))


# ---- 67: route sparse (index, value) rows to the owner index % W ------------------------------------
def _se_inputs(rc: RunCtx, cfg):
    n = -(-cfg["nodes"] // rc.world) * rc.world
    return (rc.randint(0, n, (cfg["nnz"],)), rc.randn(cfg["nnz"], cfg["hidden"], salt=1))


def _se_ref(rc, idx, value):
    W = rc.world
    if W == 1:
        return {"idx": idx, "value": value}
    owner = idx % W
    perm = torch.argsort(owner, stable=True)
    counts = torch.bincount(owner, minlength=W)
    ri, _ = _a2av_ref(idx[perm], counts)
    rv, _ = _a2av_ref(value[perm], counts)
    return {"idx": ri, "value": rv}


def _se_ours(rc, idx, value):
    """Counts stay on the device; index and value rows travel in ONE variable exchange (the index rides in the row)."""
    W = rc.world
    if W == 1:
        return {"idx": idx, "value": value}
    owner = idx % W
    perm = torch.argsort(owner, stable=True)
    counts = torch.bincount(owner, minlength=W)
    vb = value[perm].contiguous().view(torch.uint8).view(idx.numel(), -1)
    packed = torch.cat([idx[perm].view(-1, 1).view(torch.uint8).view(idx.numel(), 8), vb], 1).contiguous()
    cap = idx.numel() * W
    out, _recv, total = rc.comm.all_to_all_v(packed, counts, cap)
    # the number of received rows stays on the device: both results are capacity buffers with a device-side length
    return {"idx": Ragged(out[:, :8].contiguous().view(torch.int64).view(-1), total),
            "value": Ragged(out[:, 8:].contiguous().view(value.dtype).view(cap, -1), total)}


register(OpSpec(name="gnn_sparse_embedding_route", problem_ids=(67,), group="wild",
                configs={"default": {"nodes": 100000, "nnz": 1024, "hidden": 128}, "small": {"nodes": 64, "nnz": 16, "hidden": 8}},
                make_inputs=_se_inputs, reference=_se_ref, ours=_se_ours, atol=0, rtol=0))


# ---- 68: fetch rows of a sharded table, then project -------------------------------------------------
def _sf_inputs(rc: RunCtx, cfg):
    W, S, E = rc.world, cfg["shard_rows"], cfg["dim"]
    base = torch.arange(cfg["queries"], device=rc.device)
    ids = ((base + rc.rank) % W) * S + (base * 7 + rc.rank) % S
    return (rc.randn(S, E), ids, rc.randn(E, E, std=1.0 / math.sqrt(E), shared=True, salt=1))


def _sf_ref(rc, shard, ids, proj):
    W, r, S = rc.world, rc.rank, shard.shape[0]
    if W == 1:
        return shard[ids] @ proj
    owner = (ids // S).clamp(max=W - 1)
    order = torch.argsort(owner, stable=True)
    counts = torch.bincount(owner, minlength=W)
    got, recv_counts = _a2av_ref(ids[order], counts)
    rows = shard[got - r * S]
    back, _ = _a2av_ref(rows, recv_counts)
    return back[torch.argsort(order, stable=True)] @ proj


def _sf_ours(rc, shard, ids, proj):
    """Rows come straight from the owners' shards (the table sits in the symmetric heap for the whole job) and feed the
    projection GEMM; no request/reply exchange."""
    W, S = rc.world, shard.shape[0]
    owner = (ids // S).clamp(max=W - 1)
    emb = _remote_rows(rc, "sf_table", shard, owner, ids - owner * S)
    if rc.dist.is_cuda and emb.dtype == torch.bfloat16:
        key = ("sf_proj_t", proj.data_ptr())
        if key not in rc.cache:
            rc.cache[key] = proj.t().contiguous()
        return _mm_nt(rc, emb, rc.cache[key])
    return emb @ proj


register(OpSpec(name="gnn_sparse_feature_fetch_projection", problem_ids=(68,), group="wild",
                configs={"default": {"shard_rows": 1 << 20, "dim": 256, "queries": 20000}, "small": {"shard_rows": 64, "dim": 16, "queries": 32},
                         "full": {"shard_rows": 13875000, "dim": 256, "queries": 20000}},
                make_inputs=_sf_inputs, reference=_sf_ref, ours=_sf_ours, atol=5e-2, rtol=2e-2,
                cost=lambda cfg, W: Cost(flops=2.0 * cfg["queries"] * cfg["dim"] ** 2, nvlink_bytes=cfg["queries"] * cfg["dim"] * 2 * (W - 1) / max(W, 1))))


# ---- 69: rank of the positive among gathered negatives -----------------------------------------------
def _ns_inputs(rc: RunCtx, cfg):
    n = cfg["pos"] + rc.rank % 3
    return (rc.randn(n), rc.randn(n, cfg["neg"], salt=1), cfg["pos"] + 2)      # last: an upper bound of the rows of any rank


def _ns_ref(rc, pos, neg, cap=None):
    W = rc.world
    if W > 1:
        sizes = torch.zeros(W, dtype=torch.int64, device=pos.device)
        sizes[rc.rank] = pos.shape[0]
        dist.all_reduce(sizes)
        rs = sizes.tolist()
        parts_p = [torch.empty(n, dtype=pos.dtype, device=pos.device) for n in rs]
        parts_n = [torch.empty((n, neg.shape[1]), dtype=neg.dtype, device=pos.device) for n in rs]
        for s in range(W):                                                 # sizes differ: one broadcast per member
            if s == rc.rank:
                parts_p[s].copy_(pos); parts_n[s].copy_(neg)
            dist.broadcast(parts_p[s], s); dist.broadcast(parts_n[s], s)
        pos, neg = torch.cat(parts_p), torch.cat(parts_n)
    scores = torch.sigmoid(torch.cat([pos.view(-1, 1), neg], 1).float())
    _, order = torch.sort(scores, dim=1, descending=True, stable=True)
    return torch.nonzero(order == 0)[:, 1] + 1


def _ns_ours(rc, pos, neg, cap):
    """Rank = 1 + number of negatives that beat the positive: counted where the rows live, only the ranks (8 bytes per
    row instead of the whole score matrix) are gathered, with the row counts carried on the device; the result is a
    capacity buffer with a device-side length."""
    W = rc.world
    local = 1 + (torch.sigmoid(neg.float()) > torch.sigmoid(pos.float()).view(-1, 1)).sum(1)
    if W == 1:
        return local
    padded = torch.zeros(cap + 1, dtype=torch.int64, device=pos.device)
    padded[:local.numel()] = local
    padded[cap] = local.numel()
    allr = rc.comm.all_gather(padded)                                      # [W, cap + 1]
    rows, total = compact_padded(allr[:, :cap], allr[:, cap])
    return Ragged(rows, total)


register(OpSpec(name="gnn_negative_scoring", problem_ids=(69,), group="wild",
                configs={"default": {"pos": 128, "neg": 1000}, "small": {"pos": 5, "neg": 16}},
                make_inputs=_ns_inputs, reference=_ns_ref, ours=_ns_ours, atol=0, rtol=0))


# =================================================================================================
# 70: redistribution of a keyed jagged tensor (reference/70_torchrec_kjt_all2all.py)
# =================================================================================================
def _kjt_inputs(rc: RunCtx, cfg):
    W = rc.world
    key_splits = [1 + (d % 3) for d in range(W)]
    F_, B = sum(key_splits), cfg["batch"]
    lengths = rc.randint(5, 21, (F_ * B,))
    values = rc.randint(0, 1000000, (int(lengths.sum()),), salt=1)
    return (lengths, values, key_splits, B)


def _segment_permute(data: torch.Tensor, seg_len: torch.Tensor, order: torch.Tensor) -> torch.Tensor:
    """Concatenate the segments of ``data`` (lengths ``seg_len``) in the order ``order`` - on the device, no Python loop."""
    starts = torch.cumsum(seg_len, 0) - seg_len
    new_len = seg_len[order]
    total = int(new_len.sum())
    seg_of = torch.repeat_interleave(torch.arange(order.numel(), device=data.device), new_len, output_size=total)
    new_starts = torch.cumsum(new_len, 0) - new_len
    return data[starts[order][seg_of] + (torch.arange(total, device=data.device) - new_starts[seg_of])]


def _kjt(rc, lengths, values, key_splits, B, ours):
    W, r = rc.world, rc.rank
    dev = lengths.device
    ks = torch.tensor(key_splits, device=dev)
    len_counts = ks * B                                                    # lengths sent to each destination
    feat_sum = lengths.view(-1, B).sum(1)                                  # values per feature
    ends = [sum(key_splits[:d + 1]) for d in range(W)]                     # host integers: the key split is a Python list
    val_counts = torch.stack([feat_sum[e - k:e].sum() for e, k in zip(ends, key_splits)])
    if W > 1:
        if ours:
            # capacities are upper bounds that every rank computes alike (lengths are at most 20 per entry)
            ksm, nf = max(key_splits), sum(key_splits)
            rl, _, tl = rc.comm.all_to_all_v(lengths.view(-1, 1).contiguous(), len_counts, ksm * B * W, max_send_rows=nf * B)
            rv, _, tv = rc.comm.all_to_all_v(values.view(-1, 1).contiguous(), val_counts, 20 * ksm * B * W, max_send_rows=20 * nf * B)
            rl, rv = rl.view(-1)[:key_splits[r] * B * W], rv.view(-1)             # rv: capacity buffer, tv values valid
        else:
            rl, _ = _a2av_ref(lengths, len_counts)
            rv, _ = _a2av_ref(values, val_counts)
    else:
        rl, rv = lengths, values
    local = key_splits[r]
    # received order is (source rank, feature); the consumer wants (feature, source rank)
    recat = torch.tensor([f + s * local for f in range(local) for s in range(W)], device=dev)
    l2 = rl.view(W * local, B)
    values_out = permute_segments_padded(rv, l2.sum(1), recat) if (ours and W > 1) else _segment_permute(rv, l2.sum(1), recat)
    return {"lengths": l2[recat].reshape(-1), "values": values_out,
            "stride": torch.tensor(B * W, device=dev)}


register(OpSpec(name="kjt_all_to_all", problem_ids=(70,), group="wild",
                configs={"default": {"batch": 512}, "small": {"batch": 4}},
                make_inputs=_kjt_inputs, reference=lambda rc, *a: _kjt(rc, *a, ours=False), ours=lambda rc, *a: _kjt(rc, *a, ours=True),
                atol=0, rtol=0))


# =================================================================================================
# 71: depthwise causal conv1d with halos from the neighbours, zigzag layout
# (reference/71_hyena_conv1d_boundary_exchange.py)
# =================================================================================================
def _h1_inputs(rc: RunCtx, cfg):
    return (rc.randn(cfg["batch"], cfg["channels"], 2 * cfg["chunk"]), rc.randn(cfg["channels"], 1, cfg["ksize"], salt=1) * 0.3)


def _h1_ref(rc, x, w):
    W, r = rc.world, rc.rank
    B, C, L2 = x.shape
    L, P = L2 // 2, w.shape[-1] - 1
    ch = x.view(B, C, 2, L)
    tail_a, tail_b = ch[:, :, 0, L - P:].contiguous(), ch[:, :, 1, L - P:].contiguous()
    prev_a, next_b = torch.zeros_like(tail_a), tail_a.clone()
    ops = []
    if r > 0:
        ops += [dist.P2POp(dist.irecv, prev_a, r - 1), dist.P2POp(dist.isend, tail_b, r - 1)]
    if r < W - 1:
        ops += [dist.P2POp(dist.isend, tail_a, r + 1), dist.P2POp(dist.irecv, next_b, r + 1)]
    if ops:
        for q in dist.batch_isend_irecv(ops):
            q.wait()
    xs = ch.permute(2, 0, 1, 3).reshape(2 * B, C, L)
    xp = torch.cat([torch.cat([prev_a, next_b], 0), xs], -1)
    y = F.conv1d(xp.float(), w.float(), groups=C).to(x.dtype)
    return y.view(2, B, C, L).permute(1, 2, 0, 3).reshape(B, C, L2)


def _h1_ours(rc, x, w):
    if rc.dist.is_cuda and x.dtype in (torch.bfloat16, torch.float32):
        from ..ops.wild import halo_conv1d_zigzag

        return halo_conv1d_zigzag(x, w, rc.comm.group())
    W, r = rc.world, rc.rank
    B, C, L2 = x.shape
    L, P = L2 // 2, w.shape[-1] - 1
    ch = x.view(B, C, 2, L)
    tails = rc.comm.all_gather(ch[:, :, :, L - P:].contiguous()) if W > 1 else ch[:, :, :, L - P:].unsqueeze(0)
    prev_a = tails[r - 1][:, :, 0] if r > 0 else torch.zeros_like(tails[0][:, :, 0])
    next_b = tails[r + 1][:, :, 1] if r < W - 1 else tails[r][:, :, 0]
    xs = ch.permute(2, 0, 1, 3).reshape(2 * B, C, L)
    xp = torch.cat([torch.cat([prev_a, next_b], 0), xs], -1)
    y = F.conv1d(xp.float(), w.float(), groups=C).to(x.dtype)
    return y.view(2, B, C, L).permute(1, 2, 0, 3).reshape(B, C, L2)


register(OpSpec(name="hyena_conv1d_halo", problem_ids=(71,), group="wild",
                configs={"default": {"batch": 1, "channels": 1024, "chunk": 1024, "ksize": 7}, "small": {"batch": 2, "channels": 8, "chunk": 16, "ksize": 4}},
                make_inputs=_h1_inputs, reference=_h1_ref, ours=_h1_ours, atol=3e-2, rtol=2e-2,
                cost=lambda cfg, W: Cost(hbm_bytes=2 * cfg["batch"] * cfg["channels"] * 2 * cfg["chunk"] * 2)))


# =================================================================================================
# 72: Hyena long convolution, sequence <-> channel exchanges around an FFT convolution
# (reference/72_hyena_forward_cp.py)
# =================================================================================================
def _hy_inputs(rc: RunCtx, cfg):
    C, L, FL = cfg["channels"], cfg["local_seq"], cfg["filter"]
    h = (torch.arange(C * FL, device=rc.device, dtype=torch.float32).reshape(C, FL) / (C * FL)).to(rc.dtype)
    bias = (torch.arange(C, device=rc.device, dtype=torch.float32) / C).to(rc.dtype)
    return (rc.randn(1, C, L), rc.randn(1, C, L, salt=1), rc.randn(1, C, L, salt=2), h, bias)


def _zz_index(n: int, device, inverse: bool) -> torch.Tensor:
    """Chunk order of the zigzag layout: rank r holds chunks (r, n-1-r); ``inverse`` gives natural order from rank order."""
    half = n // 2
    idx = torch.empty(n, dtype=torch.long, device=device)
    idx[0::2] = torch.arange(half, device=device)
    idx[1::2] = torch.arange(n - 1, half - 1, -1, device=device)
    return torch.argsort(idx) if inverse else idx


def _fftconv(u, kern, bias):
    L = u.shape[-1]
    n = 2 * L
    kf = torch.fft.rfft(kern.float(), n=n) / n
    y = torch.fft.irfft(torch.fft.rfft(u.float(), n=n) * kf.unsqueeze(0), n=n, norm="forward")[..., :L]
    return (y + u.float() * bias.float().unsqueeze(-1)).to(u.dtype)


def _hyena(rc, x1, x2, v, h, bias, ours):
    W, r = rc.world, rc.rank
    B, C, L = x1.shape
    Cl = C // W
    def to_full(ts):
        if W == 1:
            return list(ts)
        if ours:                                                           # the three tensors ride in ONE exchange
            full = rc.comm.all_to_all_permute(torch.stack(ts), 2, 3)      # [3, B, C/W, W*L] in rank order
            outs = list(full.unbind(0))
        else:
            outs = [_a2a_ref(t, 1, 2, W) for t in ts]
        idx = _zz_index(2 * W, x1.device, True)
        return [o.reshape(B, Cl, 2 * W, L // 2).index_select(2, idx).reshape(B, Cl, W * L) for o in outs]
    f1, f2, fv = to_full([x1, x2, v])
    z = f1 * _fftconv(f2 * fv, h[r * Cl:(r + 1) * Cl, :], bias[r * Cl:(r + 1) * Cl])
    if W > 1:
        z = z.reshape(B, Cl, 2 * W, L // 2).index_select(2, _zz_index(2 * W, z.device, False)).reshape(B, Cl, W * L)
        z = rc.comm.all_to_all_permute(z.contiguous(), 2, 1) if ours else _a2a_ref(z.contiguous(), 2, 1, W)
    return z.transpose(1, 2).contiguous()


register(OpSpec(name="hyena_forward_cp", problem_ids=(72,), group="wild",
                configs={"default": {"channels": 1024, "local_seq": 2048, "filter": 4096}, "small": {"channels": 8, "local_seq": 16, "filter": 32}},
                make_inputs=_hy_inputs, reference=lambda rc, *a: _hyena(rc, *a, ours=False), ours=lambda rc, *a: _hyena(rc, *a, ours=True),
                atol=5e-2, rtol=3e-2))


# =================================================================================================
# 74 / 75: gated delta-rule attention (reference/74_fla_kimi_delta_attention_cp_tp.py,
# reference/75_fla_gated_deltanet_cp.py)
# =================================================================================================
def _delta_recurrence_torch(q, k, v, decay, beta):
    """q, k [BH,T,K]; v [BH,T,V]; decay [BH,T,K or 1]; beta [BH,T]; the step-by-step form."""
    BH, T, K = q.shape
    S = torch.zeros(BH, K, v.shape[-1], dtype=torch.float32, device=q.device)
    out = torch.empty(BH, T, v.shape[-1], dtype=torch.float32, device=q.device)
    for t in range(T):
        S = decay[:, t].unsqueeze(-1) * S
        u = (v[:, t] - torch.bmm(k[:, t].unsqueeze(1), S).squeeze(1)) * beta[:, t].unsqueeze(-1)
        S = S + k[:, t].unsqueeze(-1) * u.unsqueeze(1)
        out[:, t] = torch.bmm(q[:, t].unsqueeze(1), S).squeeze(1)
    return out


def _delta_run(rc, q, k, v, decay, beta, ours):
    """Inputs [B, T, H, *] -> output [B, T, H, V]."""
    B, T, H, K = q.shape
    bh = lambda t: t.float().permute(0, 2, 1, 3).reshape(B * H, T, t.shape[-1]).contiguous()  # noqa: E731
    args = (bh(q), bh(k), bh(v), bh(decay), beta.float().permute(0, 2, 1).reshape(B * H, T).contiguous())
    if ours and rc.dist.is_cuda and K in (32, 64, 128, 256):
        from ..ops.wild import delta_rule_scan

        o = delta_rule_scan(*args)
    else:
        o = _delta_recurrence_torch(*args)
    return o.view(B, H, T, -1).permute(0, 2, 1, 3).contiguous()


def _kda_inputs(rc: RunCtx, cfg):
    T, H, K, V = cfg["local_seq"], cfg["heads"], cfg["k"], cfg["v"]
    a_log = torch.linspace(-0.1, 0.1, H, device=rc.device).to(rc.dtype)
    dt_bias = torch.linspace(-0.1, 0.1, H * K, device=rc.device).to(rc.dtype)
    return (rc.randn(1, T, H, K), rc.randn(1, T, H, K, salt=1), rc.randn(1, T, H, V, salt=2), rc.randn(1, T, H, K, salt=3),
            rc.randn(1, T, H, salt=4), a_log, dt_bias)


def _kda_prep(q, k, g, beta, a_log, dt_bias):
    H, K = q.shape[2], q.shape[3]
    decay = torch.exp(-5.0 * torch.sigmoid(a_log.float().exp().view(1, 1, H, 1) * (g.float() + dt_bias.float().view(H, K))))
    return F.normalize(q.float(), dim=-1) * K ** -0.5, F.normalize(k.float(), dim=-1), decay, beta.float().sigmoid()


def _kda_ref(rc, q, k, v, g, beta, a_log, dt_bias):
    """Every rank gathers the whole sequence and runs the recurrence for all heads, then keeps its rows."""
    W, r = rc.world, rc.rank
    T = q.shape[1]
    if W > 1:
        gs = lambda t: _ag_ref(t, W).transpose(0, 1).reshape(t.shape[0], W * T, *t.shape[2:])  # noqa: E731
        q, k, v, g, beta = gs(q), gs(k), gs(v), gs(g), gs(beta)
    qn, kn, decay, bs = _kda_prep(q, k, g, beta, a_log, dt_bias)
    out = _delta_run(rc, qn, kn, v, decay, bs, False).to(v.dtype)
    return out[:, r * T:(r + 1) * T].contiguous()


def _kda_ours(rc, q, k, v, g, beta, a_log, dt_bias):
    """The recurrence is sequential in time but independent per head: one exchange gives every rank H/W heads of the
    whole sequence (all five inputs packed), the scan kernel runs once per head instead of W times, one exchange back."""
    W, r = rc.world, rc.rank
    H, K, V = q.shape[2], q.shape[3], v.shape[3]
    qn, kn, decay, bs = _kda_prep(q, k, g, beta, a_log, dt_bias)
    packed = torch.cat([qn, kn, v.float(), decay, bs.unsqueeze(-1)], -1)     # [B, T, H, 3K + V + 1]
    if W > 1:
        packed = rc.comm.all_to_all_permute(packed.contiguous(), 2, 1)      # [B, W*T, H/W, .]
    qn, kn, vv, decay, bs = packed.split([K, K, V, K, 1], -1)
    out = _delta_run(rc, qn, kn, vv, decay, bs.squeeze(-1), True)
    if W > 1:
        out = rc.comm.all_to_all_permute(out.contiguous(), 1, 2)
    return out.to(v.dtype)


register(OpSpec(name="kimi_delta_attention_cp", problem_ids=(74,), group="wild",
                configs={"default": {"local_seq": 64, "heads": 16, "k": 128, "v": 128}, "small": {"local_seq": 8, "heads": 8, "k": 32, "v": 16}},
                make_inputs=_kda_inputs, reference=_kda_ref, ours=_kda_ours, atol=3e-2, rtol=3e-2))


def _gdn_inputs(rc: RunCtx, cfg):
    W = rc.world
    T, K, V = cfg["local_seq"], cfg["k"], cfg["v"]
    H = -(-cfg["heads"] // W) * W
    a_log = torch.linspace(-0.1, 0.1, H, device=rc.device).to(rc.dtype)
    dt_bias = torch.linspace(-0.1, 0.1, H, device=rc.device).to(rc.dtype)
    return (rc.randn(1, T, H, K), rc.randn(1, T, H, K, salt=1), rc.randn(1, T, H, V, salt=2), rc.randn(1, T, H, salt=3),
            torch.sigmoid(rc.randn(1, T, H, salt=4).float()).to(rc.dtype), a_log, dt_bias)


def _gdn(rc, q, k, v, gate, beta, a_log, dt_bias, ours):
    W, r = rc.world, rc.rank
    H, K, V = q.shape[2], q.shape[3], v.shape[3]
    Hl = H // W
    if W > 1:
        if ours:                                                           # five tensors, one exchange
            packed = torch.cat([q.float(), k.float(), v.float(), gate.float().unsqueeze(-1), beta.float().unsqueeze(-1)], -1)
            packed = rc.comm.all_to_all_permute(packed.contiguous(), 2, 1)
            q, k, v, gate, beta = packed.split([K, K, V, 1, 1], -1)
            gate, beta = gate.squeeze(-1), beta.squeeze(-1)
        else:
            q, k, v = (_a2a_ref(t, 2, 1, W) for t in (q, k, v))
            gate, beta = (_a2a_ref(t.unsqueeze(-1), 2, 1, W).squeeze(-1) for t in (gate, beta))
    al, db = a_log[r * Hl:(r + 1) * Hl].float(), dt_bias[r * Hl:(r + 1) * Hl].float()
    qn = F.normalize(q.float(), dim=-1, eps=1e-6) * K ** -0.5
    kn = F.normalize(k.float(), dim=-1, eps=1e-6)
    decay = torch.exp(-al.exp().view(1, 1, Hl) * F.softplus(gate.float() + db.view(1, 1, Hl))).unsqueeze(-1)
    out = _delta_run(rc, qn, kn, v.float(), decay, beta.float(), ours)
    if W > 1:
        out = rc.comm.all_to_all_permute(out.contiguous(), 1, 2) if ours else _a2a_ref(out.contiguous(), 1, 2, W)
    return out.to(v.dtype)


register(OpSpec(name="gated_deltanet_cp", problem_ids=(75,), group="wild",
                configs={"default": {"local_seq": 64, "heads": 6, "k": 256, "v": 512}, "small": {"local_seq": 8, "heads": 4, "k": 32, "v": 16}},
                make_inputs=_gdn_inputs, reference=lambda rc, *a: _gdn(rc, *a, ours=False), ours=lambda rc, *a: _gdn(rc, *a, ours=True),
                atol=3e-2, rtol=3e-2))


# =================================================================================================
# 76: conv3d with the input channels sharded, partial outputs summed over the ranks
# (reference/76_opensora_conv3d_allreduce.py)
# =================================================================================================
def _c3_inputs(rc: RunCtx, cfg):
    cin_l = cfg["cout"] // rc.world
    x = rc.randn(1, cin_l, cfg["t"], cfg["h"], cfg["w"])
    w = rc.randn(cfg["cout"], cin_l, 3, 3, 3, salt=1) * (1.0 / math.sqrt(27 * cfg["cout"]))
    bias = torch.linspace(-0.1, 0.1, cfg["cout"], device=rc.device).to(rc.dtype)
    return (x, w, bias)


def _c3_ref(rc, x, w, bias):
    out = F.conv3d(x, w)
    if rc.world > 1:
        dist.all_reduce(out)
    return out + bias.view(1, -1, 1, 1, 1)


def _c3_ours(rc, x, w, bias):
    """The convolution as ONE tcgen05 GEMM over unfolded patches ([positions, Cin*27] x [Cout, Cin*27]^T, fp32 out), the
    partial sums reduced by the all-reduce kernel (in-switch for large tensors) and the bias added on the way out."""
    Cout, Cin = w.shape[:2]
    _, _, T, H, Wd = x.shape
    To, Ho, Wo = T - 2, H - 2, Wd - 2
    if rc.dist.is_cuda and x.dtype == torch.bfloat16 and (Cin * 27) % 8 == 0:
        patches = x[0].unfold(1, 3, 1).unfold(2, 3, 1).unfold(3, 3, 1)            # [Cin, To, Ho, Wo, 3, 3, 3]
        a = patches.permute(1, 2, 3, 0, 4, 5, 6).reshape(To * Ho * Wo, Cin * 27).contiguous()
        out = _mm_nt(rc, a, w.reshape(Cout, Cin * 27), out_f32=True)               # [positions, Cout]
        if rc.world > 1:
            out = rc.comm.all_reduce(out)
        out = (out + bias.float().view(1, -1)).to(x.dtype)
        return out.t().reshape(1, Cout, To, Ho, Wo).contiguous()
    out = F.conv3d(x, w)
    if rc.world > 1:
        out = rc.comm.all_reduce(out.contiguous())
    return out + bias.view(1, -1, 1, 1, 1)


register(OpSpec(name="conv3d_allreduce", problem_ids=(76,), group="wild",
                configs={"default": {"cout": 512, "t": 19, "h": 66, "w": 66}, "small": {"cout": 8, "t": 4, "h": 6, "w": 6}},
                make_inputs=_c3_inputs, reference=_c3_ref, ours=_c3_ours, atol=5e-2, rtol=3e-2,
                cost=lambda cfg, W: Cost(flops=2.0 * (cfg["t"] - 2) * (cfg["h"] - 2) * (cfg["w"] - 2) * cfg["cout"] * cfg["cout"] / max(W, 1) * 27,
                                         nvlink_bytes=2.0 * (W - 1) / max(W, 1) * (cfg["t"] - 2) * (cfg["h"] - 2) * (cfg["w"] - 2) * cfg["cout"] * 2)))


# =================================================================================================
# 77: context-shuffled attention over ranges (reference/77_magi1_cso_async_attention.py)
# =================================================================================================
def _cso_inputs(rc: RunCtx, cfg):
    W = rc.world
    ranges, spb, D = cfg["ranges"], cfg["spb"], cfg["d"]
    Hq = -(-cfg["hq"] // W) * W
    Hkv = cfg["hkv"] if (cfg["hkv"] % W == 0 or W % cfg["hkv"] == 0) else W
    q = rc.randn(ranges * spb, Hq, D)
    kv = torch.cat([rc.randn(ranges * spb, Hkv, D, salt=1), rc.randn(ranges * spb, Hkv, D, salt=2)], -1)
    clip = cfg.get("clip") or W * spb
    return (q, kv, ranges, min(clip, W * spb))


def _cso(rc, q, kv, ranges, clip, ours):
    W = rc.world
    tokens, Hq, D = q.shape
    spb = tokens // ranges
    if kv.shape[1] < W:
        kv = kv.repeat_interleave(W // kv.shape[1], dim=1)
    q4, kv4 = q.view(ranges, spb, Hq, D), kv.reshape(ranges, spb, kv.shape[1], 2 * D)
    if W > 1:
        if ours:
            q4, kv4 = rc.comm.all_to_all_permute(q4.contiguous(), 2, 1), rc.comm.all_to_all_permute(kv4.contiguous(), 2, 1)
        else:
            q4, kv4 = _a2a_ref(q4, 2, 1, W), _a2a_ref(kv4, 2, 1, W)
    kv4 = kv4[:, :clip]
    k, v = kv4[..., :D].contiguous(), kv4[..., D:].contiguous()
    if ours and rc.dist.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128):
        from ..ops.attention import flash_attn_fwd

        o = flash_attn_fwd(q4.contiguous(), k, v, causal=False, scale=D ** -0.5, return_lse=False)[0]   # every range is one batch entry
    else:
        rep = q4.shape[2] // k.shape[2]
        s = torch.einsum("rqhd,rkhd->rhqk", q4.float(), k.float().repeat_interleave(rep, 2)) * D ** -0.5
        o = torch.einsum("rhqk,rkhd->rqhd", torch.softmax(s, -1), v.float().repeat_interleave(rep, 2)).to(q.dtype)
    if W > 1:
        o = rc.comm.all_to_all_permute(o.contiguous(), 1, 2) if ours else _a2a_ref(o.contiguous(), 1, 2, W)
    return o.reshape(tokens, Hq, D)


register(OpSpec(name="cso_range_attention", problem_ids=(77,), group="wild",
                configs={"default": {"ranges": 4, "spb": 2700, "hq": 48, "hkv": 8, "d": 128}, "small": {"ranges": 2, "spb": 6, "hq": 4, "hkv": 2, "d": 16}},
                make_inputs=_cso_inputs, reference=lambda rc, *a: _cso(rc, *a, ours=False), ours=lambda rc, *a: _cso(rc, *a, ours=True),
                atol=3e-2, rtol=3e-2))


# =================================================================================================
# 78: tile-parallel decode with seam blending (reference/78_magi1_tile_parallel_vae_decode.py)
# =================================================================================================
def _vae_inputs(rc: RunCtx, cfg):
    z = torch.randn(1, cfg["c"], cfg["t"], cfg["h"], cfg["w"], device=rc.device, generator=rc.gen(shared=True)).to(torch.bfloat16 if rc.dist.is_cuda else rc.dtype)
    return (z, cfg["tile_t"], cfg["tile_hw"], cfg["tile_hw"], 0.25, 0.0, cfg["up_s"], cfg["up_t"])


def _decode_tile(tile, up_s, up_t):
    d = F.interpolate(tile.float(), scale_factor=(up_t, up_s, up_s), mode="trilinear", align_corners=False)
    if d.shape[1] < 3:
        d = d.repeat(1, -(-3 // d.shape[1]), 1, 1, 1)
    return d[:, :3].to(tile.dtype)


def _blend(prev, cur, extent, dim):
    extent = min(prev.shape[dim], cur.shape[dim], extent)
    if extent <= 0:
        return cur
    ratio = (torch.arange(extent, device=cur.device, dtype=torch.float32) / extent).view([-1 if i == dim else 1 for i in range(5)])
    head = prev.narrow(dim, prev.shape[dim] - extent, extent).float() * (1.0 - ratio) + cur.narrow(dim, 0, extent).float() * ratio
    cur.narrow(dim, 0, extent).copy_(head.to(cur.dtype))
    return cur


def _vae(rc, z, tl, th, tw, sp_ov, t_ov, up_s, up_t, ours):
    W, r = rc.world, rc.rank
    st, sh, sw = int(tl * (1 - t_ov)), int(th * (1 - sp_ov)), int(tw * (1 - sp_ov))
    rt, rh, rw = tl * up_t, th * up_s, tw * up_s
    bt, bh, bw = int(rt * t_ov), int(rh * sp_ov), int(rw * sp_ov)
    nt, nh, nw = -(-z.shape[2] // st), -(-z.shape[3] // sh), -(-z.shape[4] // sw)
    tiles = [(a, b, c) for a in range(nt) for b in range(nh) for c in range(nw)]
    lat = [z[:, :, a * st:a * st + tl, b * sh:b * sh + th, c * sw:c * sw + tw] for a, b, c in tiles]
    order = sorted(range(len(tiles)), key=lambda i: lat[i].numel(), reverse=True)
    per_rank = [order[s::W] for s in range(W)]
    def shape_dec(i):
        return (1, 3, lat[i].shape[2] * up_t, lat[i].shape[3] * up_s, lat[i].shape[4] * up_s)
    def gather(local, shapes_of):
        """Every rank ends up with every tile. All sizes follow from the tiling, so no shape exchange is needed."""
        if W == 1:
            return {i: t for i, t in zip(per_rank[0], local)}
        flat = torch.cat([t.reshape(-1) for t in local]) if local else z.new_empty(0)
        sizes = [sum(math.prod(shapes_of(i)) for i in per_rank[s]) for s in range(W)]
        cap = max(sizes)
        buf = torch.zeros(cap, dtype=flat.dtype, device=flat.device)
        buf[:flat.numel()] = flat
        allb = rc.comm.all_gather(buf) if ours else _ag_ref(buf, W)
        out = {}
        for s in range(W):
            o = 0
            for i in per_rank[s]:
                n = math.prod(shapes_of(i))
                out[i] = allb[s, o:o + n].view(shapes_of(i))
                o += n
        return out
    dec = gather([_decode_tile(lat[i], up_s, up_t) for i in per_rank[r]], shape_dec)
    idx_of = {t: i for i, t in enumerate(tiles)}
    blended = []
    for i in per_rank[r]:
        a, b, c = tiles[i]
        cur = dec[i].clone()
        if a > 0:
            cur = _blend(dec[idx_of[(a - 1, b, c)]], cur, bt, 2)
        if b > 0:
            cur = _blend(dec[idx_of[(a, b - 1, c)]], cur, bh, 3)
        if c > 0:
            cur = _blend(dec[idx_of[(a, b, c - 1)]], cur, bw, 4)
        blended.append(cur[:, :, :rt - bt, :rh - bh, :rw - bw].contiguous())
    def shape_bl(i):
        s = shape_dec(i)
        return (1, 3, min(s[2], rt - bt), min(s[3], rh - bh), min(s[4], rw - bw))
    allb = gather(blended, shape_bl)
    return torch.cat([torch.cat([torch.cat([allb[idx_of[(a, b, c)]] for c in range(nw)], 4) for b in range(nh)], 3) for a in range(nt)], 2)


register(OpSpec(name="tile_parallel_vae_decode", problem_ids=(78,), group="wild",
                configs={"default": {"c": 16, "t": 6, "h": 90, "w": 90, "tile_t": 3, "tile_hw": 32, "up_s": 8, "up_t": 4},
                         "small": {"c": 4, "t": 4, "h": 10, "w": 10, "tile_t": 2, "tile_hw": 4, "up_s": 2, "up_t": 2}},
                make_inputs=_vae_inputs, reference=lambda rc, *a: _vae(rc, *a, ours=False), ours=lambda rc, *a: _vae(rc, *a, ours=True),
                atol=2e-2, rtol=2e-2))


# =================================================================================================
# 79: distributed k-nearest-neighbour search (reference/79_dinov2_distributed_knn.py)
# =================================================================================================
def _knn_inputs(rc: RunCtx, cfg):
    Q, N, D = cfg["queries"], cfg["train"], cfg["d"]
    test = F.normalize(rc.randn(Q, D, dtype=torch.float32), dim=1).to(rc.dtype)
    train = F.normalize(rc.randn(N, D, dtype=torch.float32, salt=1), dim=1).to(rc.dtype)
    labels = (rc.rank * N + torch.arange(N, device=rc.device)) % cfg["classes"]
    return (test, train.t().contiguous(), labels.view(1, N), min(cfg["k"], N), cfg["classes"])


def _knn_votes(sims, labels, classes):
    votes = torch.zeros((sims.shape[0], classes), dtype=torch.float32, device=sims.device)
    votes.scatter_add_(1, labels, torch.ones_like(sims, dtype=torch.float32))
    return {"sims": sims.float(), "votes": votes / sims.shape[1]}


def _knn_ref(rc, test, train_t, labels, k, classes):
    """One round per owner: broadcast its queries, local similarity + top-k everywhere, gather on the owner, merge."""
    W, r = rc.world, rc.rank
    result = None
    for owner in range(W):
        qs = test.clone()
        if W > 1:
            dist.broadcast(qs, owner)
        sims, idx = (qs.float() @ train_t.float()).topk(k, dim=1)
        lab = labels.expand(qs.shape[0], -1).gather(1, idx)
        if W > 1:
            gs = [torch.empty_like(sims) for _ in range(W)] if r == owner else None
            gl = [torch.empty_like(lab) for _ in range(W)] if r == owner else None
            dist.gather(sims, gs, dst=owner)
            dist.gather(lab, gl, dst=owner)
            if r == owner:
                s_all, l_all = torch.cat(gs, 1), torch.cat(gl, 1)
                top, ti = s_all.topk(k, dim=1)
                result = (top, l_all.gather(1, ti))
        else:
            result = (sims, lab)
    return _knn_votes(result[0], result[1], classes)


def _knn_ours(rc, test, train_t, labels, k, classes):
    """All queries of all ranks at once: one gather, ONE GEMM against the local shard, one top-k, one exchange that
    hands every owner its W candidate lists (similarity and label packed together), one merge."""
    W, r = rc.world, rc.rank
    Q = test.shape[0]
    allq = rc.comm.all_gather(test.contiguous()).reshape(W * Q, -1) if W > 1 else test
    if rc.dist.is_cuda and test.dtype == torch.bfloat16:
        from ..ops import gemm_bf16_kn

        sim = gemm_bf16_kn(allq.contiguous(), train_t.contiguous(), out_dtype=torch.float32)
    else:
        sim = allq.float() @ train_t.float()
    if rc.dist.is_cuda and sim.shape[1] <= 4096 and W * k <= 4096 and classes <= 4096:
        from ..ops.wild import knn_merge_votes, knn_topk_local

        # one block per query sorts its candidates in shared memory; the k best leave as (similarity, label) pairs in the
        # layout of the exchange, and the merge on the owner writes similarities and votes from the same kernel
        if W == 1:
            s1, v1 = knn_topk_local(sim.float(), labels, k, classes)
            return {"sims": s1, "votes": v1}
        got = rc.comm.all_to_all(knn_topk_local(sim.float(), labels, k).view(W, Q, k, 2))
        s1, v1 = knn_merge_votes(got, k, classes)
        return {"sims": s1, "votes": v1}
    sims, idx = sim.topk(k, dim=1)
    lab = labels.expand(sims.shape[0], -1).gather(1, idx)
    if W > 1:
        packed = torch.stack([sims.float(), lab.float()], -1).view(W, Q, k, 2).contiguous()
        got = rc.comm.all_to_all(packed)                                      # [W(source), Q, k, 2] for my queries
        s_all = got[..., 0].permute(1, 0, 2).reshape(Q, W * k)
        l_all = got[..., 1].permute(1, 0, 2).reshape(Q, W * k).long()
        sims, ti = s_all.topk(k, dim=1)
        lab = l_all.gather(1, ti)
    return _knn_votes(sims, lab, classes)


register(OpSpec(name="distributed_knn", problem_ids=(79,), group="wild",
                configs={"default": {"queries": 32, "train": 2048, "d": 384, "k": 200, "classes": 1000},
                         "small": {"queries": 4, "train": 64, "d": 16, "k": 5, "classes": 10}},
                make_inputs=_knn_inputs, reference=_knn_ref, ours=_knn_ours, atol=2e-2, rtol=2e-2,
                # similarity GEMM of all ranks' queries against the local shard; queries gathered, candidate lists exchanged
                cost=lambda cfg, W: Cost(flops=2.0 * W * cfg["queries"] * cfg["train"] * cfg["d"],
                                         nvlink_bytes=(W - 1) * cfg["queries"] * (cfg["d"] * 2 + min(cfg["k"], cfg["train"]) * 8))))


# =================================================================================================
# 80: Sinkhorn-Knopp normalisation with the batch sharded (reference/80_dinov2_distributed_sinkhorn_knopp.py)
# =================================================================================================
def _sk_inputs(rc: RunCtx, cfg):
    return (rc.randn(cfg["batch"], cfg["prototypes"], dtype=torch.float32) * 0.01, 0.07, 3)


def _sk_ref(rc, t, temp, iters):
    W = rc.world
    ar = (lambda x: _allreduce_ref(x)) if W > 1 else (lambda x: x)
    q = torch.exp(t.float() / temp).T.contiguous()
    total_batch = ar(torch.tensor([float(t.shape[0])], device=t.device))
    P = q.shape[0]
    q /= ar(q.sum().reshape(1))
    for _ in range(iters):
        q /= ar(q.sum(dim=1, keepdim=True))
        q /= P
        q /= q.sum(dim=0, keepdim=True)
        q /= total_batch
    q *= total_batch
    return q.T.contiguous()


def _sk_ours(rc, t, temp, iters):
    """The matrix is never rewritten: a row scale per prototype and a column scale per sample carry the iterations, each
    of which is two matrix-vector passes over exp(t/temp) and one small all-reduce; the result is written once."""
    W = rc.world
    ar = (lambda x: rc.comm.all_reduce(x)) if W > 1 else (lambda x: x)
    if rc.dist.is_cuda:
        from ..ops.wild import sinkhorn_knopp

        return sinkhorn_knopp(t, temp, iters, all_reduce=ar if W > 1 else None)   # the exponentials are never stored either
    E = torch.exp(t.float() / temp)                                           # [B, P]
    B, P = E.shape
    head = ar(torch.stack([torch.tensor(float(B), device=t.device), E.sum()]))   # batch size and mass in one exchange
    total_batch, mass = head[0], head[1]
    r = torch.ones(P, device=t.device)
    c = torch.full((B,), 1.0, device=t.device) / mass
    for _ in range(iters):
        R = ar((r * torch.mv(E.t(), c)).contiguous())
        r = r / R / P
        c = c / (c * torch.mv(E, r)) / total_batch
    return E * r.view(1, P) * (c * total_batch).view(B, 1)


register(OpSpec(name="sinkhorn_knopp", problem_ids=(80,), group="wild",
                configs={"default": {"batch": 1024, "prototypes": 16384}, "small": {"batch": 8, "prototypes": 32}},
                make_inputs=_sk_inputs, reference=_sk_ref, ours=_sk_ours, atol=1e-7, rtol=1e-3,
                # one pass for the mass, two per iteration (three iterations), one read and one write for the result
                cost=lambda cfg, W: Cost(hbm_bytes=9.0 * cfg["batch"] * cfg["prototypes"] * 4, nvlink_bytes=3.0 * cfg["prototypes"] * 4 * (W - 1))))


# =================================================================================================
# 81: gather of object masks and IoU suppression (reference/81_sam3_allgather_iou_suppression.py)
# =================================================================================================
def _sam_inputs(rc: RunCtx, cfg):
    W = rc.world
    counts = [1 + ((i + rc.trial) % 3) for i in range(W)]
    n, H, Wd = counts[rc.rank], cfg["h"], cfg["w"]
    yy = torch.arange(H, device=rc.device).view(1, H, 1)
    xx = torch.arange(Wd, device=rc.device).view(1, 1, Wd)
    cc = torch.arange(n, device=rc.device).view(n, 1, 1)
    masks = rc.randn(n, H, Wd) + (((yy + xx + cc + rc.rank) % 5 == 0).to(rc.dtype) * 4.0 - 1.0)
    scores = torch.linspace(-5.0, 5.0, n, device=rc.device).to(rc.dtype)
    last = (torch.arange(sum(counts), device=rc.device) % 5) - 1
    return (masks, scores, counts, last, 0.7)


def _sam(rc, masks, scores, counts, last, thr, ours):
    W = rc.world
    cap = max(counts)
    def gv(t):
        if W == 1:
            return t.float()
        pad = torch.zeros((cap, *t.shape[1:]), dtype=torch.float32, device=t.device)
        pad[:t.shape[0]] = t.float()
        allp = rc.comm.all_gather(pad) if ours else _ag_ref(pad, W)
        return torch.cat([allp[s, :counts[s]] for s in range(W)])
    mg, sg = gv(masks), gv(scores)
    n = mg.shape[0]
    if ours and rc.dist.is_cuda and mg[0].numel() % 32 == 0:
        from ..ops.wild import mask_iou_suppress

        sup = mask_iou_suppress(mg, last, thr)                     # bit-packed masks, one block per pair
        return {"masks": torch.where(sup.view(n, 1, 1), torch.full_like(mg, -10.0), mg), "scores": sg, "suppressed": sup}
    b = (mg > 0).flatten(1).float()
    inter = b @ b.t()
    area = b.sum(1)
    iou = inter / (area[:, None] + area[None, :] - inter).clamp_min(1.0)
    over = torch.triu(iou >= thr, diagonal=1)
    li, lj = last.view(n, 1), last.view(1, n)
    sup = (over & (li > lj) & (lj > -1)).any(1) | (over & (lj > li) & (li > -1)).any(0)
    mg = mg.clone()
    mg[sup] = -10.0
    return {"masks": mg, "scores": sg, "suppressed": sup}


register(OpSpec(name="mask_iou_suppression", problem_ids=(81,), group="wild",
                configs={"default": {"h": 256, "w": 256}, "small": {"h": 8, "w": 8}},
                make_inputs=_sam_inputs, reference=lambda rc, *a: _sam(rc, *a, ours=False), ours=lambda rc, *a: _sam(rc, *a, ours=True),
                atol=1e-5, rtol=1e-5,
                # about two masks per rank: gathered as fp32, read once for packing and once for the output, written once
                cost=lambda cfg, W: Cost(hbm_bytes=3.0 * 2 * W * cfg["h"] * cfg["w"] * 4, nvlink_bytes=2.0 * (W - 1) * cfg["h"] * cfg["w"] * 4)))


# =================================================================================================
# 82 / 83 / 84: vocabulary-parallel log-probabilities with top-k / top-p filtering, and the backward
# (reference/82_vocab_parallel_log_prob_topk.py, reference/83_vocab_parallel_log_prob_topk_chunked.py,
#  reference/84_vocab_parallel_log_prob_topk_chunked_backward.py)
# =================================================================================================
def _topk_topp(logits, top_k, top_p):
    """Returns (filtered logits, keep mask); same selection rule as the sampling code the projects use."""
    V = logits.shape[-1]
    srt, idx = logits.sort(dim=-1, descending=False)
    keep = torch.ones_like(srt, dtype=torch.bool)
    if top_k and top_k > 0:
        kk = min(int(top_k), V)
        keep = srt >= srt[..., V - kk:V - kk + 1]
        srt = srt.masked_fill(~keep, float("-inf"))
    if top_p is not None and top_p < 1.0:
        pm = torch.cumsum(srt.softmax(-1), -1) > 1 - top_p
        pm[..., -1] = True
        srt = srt.masked_fill(~pm, float("-inf"))
        keep = keep & pm
    return torch.empty_like(srt).scatter_(-1, idx, srt), torch.empty_like(keep).scatter_(-1, idx, keep)


def _vlp_inputs(rc: RunCtx, cfg, with_grad=False):
    W = rc.world
    B, S, V = cfg["batch"], -(-cfg["seq"] // W) * W, cfg["vocab"]
    Vl = V // W
    logits = rc.randn(B, S, Vl)
    target = ((torch.arange(B * S, device=rc.device) * 17 + 3 + rc.trial) % V).view(B, S)
    gv = rc.rank * Vl + torch.arange(Vl, device=rc.device)
    logits = logits + (gv.view(1, 1, Vl) == target.unsqueeze(-1)).to(logits.dtype) * 8.0
    chunk = cfg.get("chunk", 0)
    if chunk:                                  # tokens per chunk (batch * chunk) must split evenly over the ranks
        chunk = -(-chunk // W) * W
    out = [logits, target, cfg["top_k"], cfg["top_p"], chunk]
    if with_grad:
        out.insert(2, torch.linspace(-1.0, 1.0, B * S, device=rc.device).view(B, S).to(rc.dtype))
    return tuple(out)


def _vp_to_seq(rc, x2d, ours):
    """[tokens, V/W] on every rank -> [tokens/W, V]: rank r receives token block r with the whole vocabulary."""
    if rc.world == 1:
        return x2d
    return rc.comm.all_to_all_permute(x2d.contiguous(), 0, 1) if ours else _a2a_ref(x2d, 0, 1, rc.world)


def _vlp_fwd_block(rc, logits2d, target_flat, top_k, top_p, ours):
    W, r = rc.world, rc.rank
    n = logits2d.shape[0] // W
    seq = _vp_to_seq(rc, logits2d, ours)
    filt, _ = _topk_topp(seq, top_k, top_p)
    lp = F.log_softmax(filt.float(), -1).gather(-1, target_flat[r * n:(r + 1) * n].unsqueeze(-1)).squeeze(-1)
    if W == 1:
        return lp
    return (rc.comm.all_gather(lp.contiguous()) if ours else _ag_ref(lp.contiguous(), W)).reshape(-1)


def _vlp_ref(rc, logits, target, top_k, top_p, chunk):
    B, S, Vl = logits.shape
    l2, t = logits.reshape(B * S, Vl), target.reshape(-1)
    step = B * chunk if chunk else B * S
    return torch.cat([_vlp_fwd_block(rc, l2[s:s + step], t[s:s + step], top_k, top_p, False) for s in range(0, B * S, step)]).view(B, S)


def _vlp_ours(rc, logits, target, top_k, top_p, chunk):
    """A token's result does not depend on which rank filters it, so all chunks share ONE exchange and ONE gather."""
    B, S, Vl = logits.shape
    return _vlp_fwd_block(rc, logits.reshape(B * S, Vl), target.reshape(-1), top_k, top_p, True).view(B, S)


_VLP_CFG = {"default": {"batch": 2, "seq": 8, "vocab": 256, "top_k": 10, "top_p": 0.9}, "small": {"batch": 1, "seq": 4, "vocab": 32, "top_k": 5, "top_p": 0.9},
            "large": {"batch": 4, "seq": 2048, "vocab": 131072, "top_k": 50, "top_p": 0.9}}
register(OpSpec(name="vocab_parallel_logprob_topk", problem_ids=(82,), group="wild", configs=_VLP_CFG,
                make_inputs=_vlp_inputs, reference=_vlp_ref, ours=_vlp_ours, atol=2e-2, rtol=2e-2))
register(OpSpec(name="vocab_parallel_logprob_topk_chunked", problem_ids=(83,), group="wild",
                configs={k: dict(v, chunk=2) for k, v in _VLP_CFG.items()},
                make_inputs=_vlp_inputs, reference=_vlp_ref, ours=_vlp_ours, atol=2e-2, rtol=2e-2))


def _vlpb_block(rc, logits2d, target_flat, grad_flat, top_k, top_p, ours):
    W, r = rc.world, rc.rank
    n = logits2d.shape[0] // W
    seq = _vp_to_seq(rc, logits2d, ours)
    filt, keep = _topk_topp(seq, top_k, top_p)
    g = -F.softmax(filt.float(), -1)
    g[torch.arange(n, device=g.device), target_flat[r * n:(r + 1) * n]] += 1.0
    g = g * grad_flat[r * n:(r + 1) * n].float().unsqueeze(-1) * keep
    if W == 1:
        return g
    return rc.comm.all_to_all_permute(g.contiguous(), 1, 0) if ours else _a2a_ref(g.contiguous(), 1, 0, W)


def _vlpb_ref(rc, logits, target, grad, top_k, top_p, chunk):
    B, S, Vl = logits.shape
    l2, t, g = logits.reshape(B * S, Vl), target.reshape(-1), grad.reshape(-1)
    step = B * chunk if chunk else B * S
    return torch.cat([_vlpb_block(rc, l2[s:s + step], t[s:s + step], g[s:s + step], top_k, top_p, False) for s in range(0, B * S, step)]).view(B, S, Vl)


def _vlpb_ours(rc, logits, target, grad, top_k, top_p, chunk):
    B, S, Vl = logits.shape
    return _vlpb_block(rc, logits.reshape(B * S, Vl), target.reshape(-1), grad.reshape(-1), top_k, top_p, True).view(B, S, Vl)


register(OpSpec(name="vocab_parallel_logprob_topk_backward", problem_ids=(84,), group="wild",
                configs={k: dict(v, chunk=2) for k, v in _VLP_CFG.items()},
                make_inputs=lambda rc, cfg: _vlp_inputs(rc, cfg, True), reference=_vlpb_ref, ours=_vlpb_ours, atol=2e-2, rtol=2e-2))


# =================================================================================================
# 85: distributed sample sort with exact rebalancing (reference/85_distributed_sample_sort.py)
# =================================================================================================
def _sort_inputs(rc: RunCtx, cfg):
    n = cfg["n_local"]
    if rc.trial % 4 == 3 and rc.rank % 2 == 1:
        n = 0
    vals = rc.randint(-50, 50, (n,)).to(rc.dtype) - rc.rank * max(1, n)
    return (vals, max(cfg["n_local"], 1) * rc.world)               # last: an upper bound of the global element count


def _target_counts(sizes: torch.Tensor, r: int, W: int) -> torch.Tensor:
    """How many of my (globally contiguous) elements go to each rank so that everyone ends with total/W (+1) elements."""
    total = sizes.sum()
    base, extra = total // W, total % W
    ranks = torch.arange(W, device=sizes.device)
    t_start = ranks * base + torch.minimum(ranks, extra)
    t_end = t_start + base + (ranks < extra).long()
    my_start = sizes[:r].sum()
    my_end = my_start + sizes[r]
    return (torch.minimum(t_end, my_end) - torch.maximum(t_start, my_start)).clamp(min=0)


def _sample_sort(rc, x, cap, ours):
    W, r = rc.world, rc.rank
    s = x.float().sort().values
    if W == 1:
        return s.to(x.dtype)
    dev = x.device
    def a2av(rows, counts, cap):
        if ours:
            out, _, total = rc.comm.all_to_all_v(rows.view(-1, 1).contiguous(), counts, cap)
            return out.view(-1), total
        out, _ = _a2av_ref(rows, counts)
        return out, None
    def gather1(t):
        return (rc.comm.all_gather(t.contiguous()) if ours else _ag_ref(t.contiguous(), W))
    n = s.numel()
    # W regular samples per rank (+inf where a rank has fewer elements), gathered and sorted: the splitters
    pos = ((torch.arange(W, device=dev) + 1) * n) // W - 1
    samp = torch.where(pos >= 0, s[pos.clamp(min=0)] if n > 0 else torch.zeros(W, device=dev), torch.full((W,), float("inf"), device=dev))
    alls = gather1(samp).reshape(-1).sort().values
    usable = torch.isfinite(alls).sum()
    sidx = ((torch.arange(1, W, device=dev) * usable) // W - 1).clamp(min=0)
    split = alls[sidx]
    bounds = torch.searchsorted(s, split, right=True)
    counts = torch.diff(torch.cat([torch.zeros(1, dtype=torch.long, device=dev), bounds, torch.tensor([n], device=dev)]))
    got, total = a2av(s, counts, cap)
    if not ours:
        m = got.sort().values
        sizes = gather1(torch.tensor([m.numel()], dtype=torch.int64, device=dev)).reshape(-1)
        out, _ = a2av(m, _target_counts(sizes, r, W), cap)
        return out.to(x.dtype)
    # ours: the received count never comes back to the host. The capacity buffer is sorted whole with +inf behind the
    # valid part, and the second exchange sends the first ``total`` rows of it (its send counts add up to ``total``).
    m = torch.where(torch.arange(cap, device=dev) < total, got, torch.full_like(got, float("inf"))).sort().values
    sizes = gather1(total.reshape(1).to(torch.int64)).reshape(-1)
    out, _, total2 = rc.comm.all_to_all_v(m.view(-1, 1).contiguous(), _target_counts(sizes, r, W), cap)
    return Ragged(out.view(-1).to(x.dtype), total2)


register(OpSpec(name="distributed_sample_sort", problem_ids=(85,), group="wild",
                configs={"default": {"n_local": 128}, "small": {"n_local": 16}, "large": {"n_local": 1 << 20}},
                make_inputs=_sort_inputs, reference=lambda rc, x, cap: _sample_sort(rc, x, cap, False), ours=lambda rc, x, cap: _sample_sort(rc, x, cap, True),
                atol=0, rtol=0))


# =================================================================================================
# 86: Newton-Schulz orthogonalisation of a column-sharded matrix (reference/86_tp_muon_orthogonalization.py)
# =================================================================================================
_NS_QUINTIC = ((4.0848, -6.8946, 2.9270), (3.9505, -6.3029, 2.6377), (3.7418, -5.5913, 2.3037), (2.8769, -3.1427, 1.2046),
               (2.8366, -3.0525, 1.2012))


def _muon_inputs(rc: RunCtx, cfg):
    cols_l = -(-cfg["cols"] // rc.world)
    return (rc.randn(cfg["rows"], cols_l) + 0.01 * rc.rank, cfg["steps"])


def _muon_ref(rc, x, steps):
    W = rc.world
    ar = _allreduce_ref if W > 1 else (lambda t: t)
    xw = x.float()
    xw = xw / torch.sqrt(ar((xw * xw).sum().reshape(1))).clamp_min(1e-7)
    for i in range(steps):
        a, b, c = _NS_QUINTIC[i % len(_NS_QUINTIC)]
        g = ar(xw @ xw.mT)
        xw = torch.addmm(xw, torch.addmm(g, g, g, alpha=c, beta=b), xw, alpha=1.0, beta=a)
    return xw.to(x.dtype)


def _muon_ours(rc, x, steps):
    """Gram matrix, its square and the update on the tcgen05 GEMM (bf16 operands, fp32 accumulation and fp32 all-reduce)."""
    W = rc.world
    ar = (lambda t: rc.comm.all_reduce(t)) if W > 1 else (lambda t: t)
    xw = x.float()
    xw = xw / torch.sqrt(ar((xw * xw).sum().reshape(1))).clamp_min(1e-7)
    fast = rc.dist.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.shape[0] % 8 == 0
    if fast:
        from ..ops import gemm_bf16, gemm_bf16_kn
    for i in range(steps):
        a, b, c = _NS_QUINTIC[i % len(_NS_QUINTIC)]
        if fast:
            # operands are split into a bf16 head and a bf16 remainder so that the products keep ~16 bits of mantissa
            hi = xw.to(torch.bfloat16)
            lo = (xw - hi.float()).to(torch.bfloat16)
            g = gemm_bf16(hi, hi, out_dtype=torch.float32)
            cross = gemm_bf16(hi, lo, out_dtype=torch.float32)
            g = ar((g + cross + cross.t()).contiguous())
            gh = g.to(torch.bfloat16)
            gl = (g - gh.float()).to(torch.bfloat16)
            gg = gemm_bf16(gh, gh, out_dtype=torch.float32)
            gc = gemm_bf16(gh, gl, out_dtype=torch.float32)
            upd = b * g + c * (gg + gc + gc.t())
            uh = upd.to(torch.bfloat16)
            ul = (upd - uh.float()).to(torch.bfloat16)
            xw = a * xw + gemm_bf16_kn(uh, hi, out_dtype=torch.float32) + gemm_bf16_kn(ul, hi, out_dtype=torch.float32) \
                + gemm_bf16_kn(uh, lo, out_dtype=torch.float32)
        else:
            g = ar((xw @ xw.mT).contiguous())
            xw = torch.addmm(xw, torch.addmm(g, g, g, alpha=c, beta=b), xw, alpha=1.0, beta=a)
    return xw.to(x.dtype)


register(OpSpec(name="muon_newton_schulz", problem_ids=(86,), group="wild",
                configs={"default": {"rows": 512, "cols": 512, "steps": 5}, "small": {"rows": 16, "cols": 32, "steps": 5}},
                make_inputs=_muon_inputs, reference=_muon_ref, ours=_muon_ours, atol=5e-3, rtol=2e-2))


# =================================================================================================
# 87: height-sharded conv2d with halo rows from the neighbours (reference/87_conv2d_boundary_exchange.py)
# =================================================================================================
def _c2_inputs(rc: RunCtx, cfg):
    C = cfg["channels"]
    return (rc.randn(1, C, cfg["local_h"], cfg["width"]), rc.randn(C, C, 3, 3, salt=1) * (1.0 / math.sqrt(9 * C)), rc.randn(C, salt=2) * 0.1)


def _c2(rc, x, w, bias, ours):
    W, r = rc.world, rc.rank
    if W == 1:
        return F.conv2d(x, w, bias, padding=1)
    edges = torch.stack([x[:, :, :1, :], x[:, :, -1:, :]], 0).contiguous()          # [2, 1, C, 1, width]: top row, bottom row
    zero = torch.zeros_like(edges[0])
    if ours:
        # only the two neighbouring rows are fetched (the all-gather moves every rank's rows to every rank)
        want = torch.tensor([max(r - 1, 0) * 2 + 1, min(r + 1, W - 1) * 2 + 0], device=x.device)
        got = rc.comm.row_gather(edges.view(2, -1), want).view(2, *edges.shape[1:])
        top, bot = (got[0] if r > 0 else zero), (got[1] if r < W - 1 else zero)
    else:
        alle = _ag_ref(edges, W)
        top, bot = (alle[r - 1][1] if r > 0 else zero), (alle[r + 1][0] if r < W - 1 else zero)
    return F.conv2d(torch.cat([top, x, bot], 2), w, bias, padding=(0, 1))


register(OpSpec(name="conv2d_halo", problem_ids=(87,), group="wild",
                configs={"default": {"channels": 1280, "local_h": 32, "width": 128}, "small": {"channels": 8, "local_h": 4, "width": 8}},
                make_inputs=_c2_inputs, reference=lambda rc, *a: _c2(rc, *a, ours=False), ours=lambda rc, *a: _c2(rc, *a, ours=True),
                atol=5e-2, rtol=3e-2))


# =================================================================================================
# 25: importance-sampling policy loss over a sharded batch (reference/25_importance_sampling_loss.py)
# =================================================================================================
def _isl_inputs(rc: RunCtx, cfg):
    M, N, V = cfg["tokens"], cfg["hidden"], cfg["vocab"]
    labels = rc.randint(0, V, (M,), salt=2)
    labels[::17] = -100
    return (rc.randn(M, N), rc.randn(V, N, std=1.0 / math.sqrt(N), shared=True, salt=1), labels, rc.randn(M, salt=3), rc.randn(M, salt=4))


def _isl_stats(ce, labels, old_lp, adv):
    valid = labels != -100
    new_lp = -ce
    delta = (new_lp - old_lp.float()).masked_fill(~valid, 0.0).clamp(-20.0, 20.0)
    ratio = torch.exp(delta)
    pg = -(ratio * adv.float()).masked_fill(~valid, 0.0)
    sums = torch.stack([valid.sum().float(), pg.sum(), ratio.masked_fill(~valid, 0.0).sum(), (ratio - delta - 1.0).masked_fill(~valid, 0.0).sum(),
                        ce.masked_fill(~valid, 0.0).sum()])
    mn = ratio.masked_fill(~valid, float("inf")).min()
    mx = ratio.masked_fill(~valid, float("-inf")).max()
    return new_lp, pg, sums, mn, mx


def _isl_finish(new_lp, pg, sums, mn, mx):
    nv = sums[0].clamp(min=1.0)
    return {"loss": sums[1] / nv, "per_token_logprobs": new_lp, "per_token_loss": pg,
            "metrics": torch.stack([sums[2] / nv, mn, mx, sums[3] / nv, sums[4] / nv])}


def _isl_ref(rc, hidden, weight, labels, old_lp, adv):
    ce = F.cross_entropy(F.linear(hidden, weight).float(), labels, ignore_index=-100, reduction="none")
    new_lp, pg, sums, mn, mx = _isl_stats(ce, labels, old_lp, adv)
    if rc.world > 1:
        for i in range(5):                                                   # one all-reduce per statistic, as the project does
            t = sums[i].clone(); dist.all_reduce(t); sums[i] = t
        dist.all_reduce(mn, op=dist.ReduceOp.MIN)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    return _isl_finish(new_lp, pg, sums, mn, mx)


def _isl_ours(rc, hidden, weight, labels, old_lp, adv):
    """LM-head GEMM on tcgen05, cross-entropy statistics in one pass over the logits, and the seven scalars (five sums, a
    minimum, a maximum) in ONE small gather instead of seven all-reduces."""
    if rc.dist.is_cuda and hidden.dtype == torch.bfloat16:
        from ..ops import ce_local_stats, gemm_bf16

        logits = gemm_bf16(hidden.contiguous(), weight.contiguous())
        st = ce_local_stats(logits, labels.clamp(min=0), 0)                   # [rows, 3]: max, sum exp(x - max), target logit
        ce = (torch.log(st[:, 1]) + st[:, 0] - st[:, 2]).masked_fill(labels == -100, 0.0)
    else:
        ce = F.cross_entropy(F.linear(hidden, weight).float(), labels, ignore_index=-100, reduction="none")
    new_lp, pg, sums, mn, mx = _isl_stats(ce, labels, old_lp, adv)
    if rc.world > 1:
        allv = rc.comm.all_gather(torch.cat([sums, mn.reshape(1), mx.reshape(1)]).contiguous())      # [W, 7]
        sums, mn, mx = allv[:, :5].sum(0), allv[:, 5].min(), allv[:, 6].max()
    return _isl_finish(new_lp, pg, sums, mn, mx)


register(OpSpec(name="importance_sampling_loss", problem_ids=(25,), group="wild",
                configs={"default": {"tokens": 1024, "hidden": 1024, "vocab": 32000}, "small": {"tokens": 32, "hidden": 16, "vocab": 64}},
                make_inputs=_isl_inputs, reference=_isl_ref, ours=_isl_ours, atol=5e-2, rtol=5e-2,
                cost=lambda cfg, W: Cost(flops=2.0 * cfg["tokens"] * cfg["hidden"] * cfg["vocab"])))


# =================================================================================================
# 73: vocabulary-parallel cross-entropy (reference/73_vocab_parallel_cross_entropy_loss.py)
# =================================================================================================
def _vce_inputs(rc: RunCtx, cfg):
    W = rc.world
    Vl = cfg["vocab"] // W
    return (rc.randn(cfg["batch"], cfg["seq"], Vl), rc.randint(0, Vl * W, (cfg["batch"], cfg["seq"]), shared=True, salt=1))


def _vce_ref(rc, logits, target):
    """Three all-reduces (max, target logit, sum of exponentials), fp32 math on a copy of the logits."""
    W, r = rc.world, rc.rank
    lg = logits.float()
    Vl = lg.shape[-1]
    ar = (lambda t, op=dist.ReduceOp.SUM: (dist.all_reduce(t, op=op), t)[1]) if W > 1 else (lambda t, op=None: t)
    mx = ar(lg.max(-1).values, dist.ReduceOp.MAX)
    lg = lg - mx.unsqueeze(-1)
    out_of_range = (target < r * Vl) | (target >= (r + 1) * Vl)
    local_t = (target - r * Vl).masked_fill(out_of_range, 0)
    pred = ar(lg.gather(-1, local_t.unsqueeze(-1)).squeeze(-1).masked_fill(out_of_range, 0.0))
    return torch.log(ar(torch.exp(lg).sum(-1))) - pred


def _vce_ours(rc, logits, target):
    if rc.dist.is_cuda and logits.dtype in (torch.bfloat16, torch.float32):
        from ..ops import vocab_parallel_cross_entropy

        return vocab_parallel_cross_entropy(logits, target, rc.comm)
    W, r = rc.world, rc.rank
    lg = logits.float()
    Vl = lg.shape[-1]
    mx = lg.max(-1).values
    se = torch.exp(lg - mx.unsqueeze(-1)).sum(-1)
    out_of_range = (target < r * Vl) | (target >= (r + 1) * Vl)
    tg = lg.gather(-1, (target - r * Vl).masked_fill(out_of_range, 0).unsqueeze(-1)).squeeze(-1).masked_fill(out_of_range, 0.0)
    st = torch.stack([mx, se, tg], -1)
    allst = rc.comm.all_gather(st.contiguous()) if W > 1 else st.unsqueeze(0)     # ONE packed exchange
    gmax = allst[..., 0].max(0).values
    return torch.log((allst[..., 1] * torch.exp(allst[..., 0] - gmax)).sum(0)) + gmax - allst[..., 2].sum(0)


register(OpSpec(name="vocab_parallel_cross_entropy", problem_ids=(73,), group="wild",
                configs={"default": {"batch": 8, "seq": 1024, "vocab": 512}, "small": {"batch": 2, "seq": 8, "vocab": 32},
                         "llama": {"batch": 1, "seq": 4096, "vocab": 128256}},
                make_inputs=_vce_inputs, reference=_vce_ref, ours=_vce_ours, atol=2e-2, rtol=2e-2,
                cost=lambda cfg, W: Cost(hbm_bytes=cfg["batch"] * cfg["seq"] * cfg["vocab"] / max(W, 1) * 2)))
