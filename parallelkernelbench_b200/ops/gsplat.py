"""Gaussian-splat projection + redistribution to the camera owners (CUDA, symmetric heap)."""
from __future__ import annotations

import ctypes

import torch

from .. import _native as nv

HEADER_WORDS = 11


def gsplat_project_exchange(group, means, quats, scales, opacities, colors, viewmats_all, Ks_all, c_local: int, width: int,
                            height: int, eps2d: float = 0.3, near: float = 0.01, far: float = 1e10, gid_offset: int | None = None):
    """``viewmats_all`` [W*c_local, 4, 4] and ``Ks_all`` [W*c_local, 3, 3] hold every member's cameras in member order.
    Returns ``(records, count)``: ``records`` is an int32 ``[capacity, 11 + D]`` tensor of 32-bit words (camera id local
    to this rank, global Gaussian id, radius x, radius y as integers; means2d x/y, depth, three conic terms, opacity and
    D colour channels as float bits), ordered by (source member, camera, Gaussian id); ``count`` (int32 device scalar)
    is the number of valid rows. Replaces the pack + three list all-to-alls of
    reference/61_gsplat_3d_gaussian_splatting.py:320-450."""
    W, N, D = group.size, means.shape[0], colors.shape[1]
    f = lambda t: t.float().contiguous()  # noqa: E731
    means, quats, scales, opacities, colors = f(means), f(quats), f(scales), f(opacities), f(colors)
    V, K = f(viewmats_all).view(-1, 16), f(Ks_all).view(-1, 9)
    if V.shape[0] != W * c_local or K.shape[0] != W * c_local:
        raise ValueError("need the cameras of every member")
    heap = group.heap
    cap = W * N * c_local
    words = HEADER_WORDS + D
    cnt = heap.named(("gs_cnt", group.channel), (16,), torch.int32)
    recv = heap.named(("gs_recv", group.channel, cap, words), (cap, words), torch.int32)
    nblk = (N + 255) // 256
    blk_counts = torch.empty(W * c_local * nblk, dtype=torch.int32, device=means.device)
    count = torch.zeros((), dtype=torch.int32, device=means.device)
    nv.check(nv.cuda_lib().pkb_gsplat_project_exchange(
        group.ref, nv.ptr(means), nv.ptr(quats), nv.ptr(scales), nv.ptr(opacities), nv.ptr(colors), nv.ptr(V), nv.ptr(K), N, c_local, D,
        nv.c_float(float(width)), nv.c_float(float(height)), nv.c_float(eps2d), nv.c_float(near), nv.c_float(min(far, 3.0e38)),
        int(gid_offset if gid_offset is not None else group.rank_in_group * N), nv.ptr(blk_counts), ctypes.c_ulonglong(cnt.offset),
        ctypes.c_ulonglong(recv.offset), nv.c_ll(cap), nv.ptr(count), nv.current_stream()), "pkb_gsplat_project_exchange")
    nv.count_launch(3)
    return recv.local.clone(), count
