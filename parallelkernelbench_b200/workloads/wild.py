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
