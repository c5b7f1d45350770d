"""Elementwise fp32 restatement of the Gaussian-splat projection stage.

The same math as reference/61_gsplat_3d_gaussian_splatting.py:128-317 (quaternion -> rotation, covariance,
world -> camera, perspective projection, conics, radii, culling), written as single elementwise operations in a fixed
order instead of einsums so that every intermediate has one well-defined rounding: the CUDA kernel performs the same
operations in the same order and the two agree bit for bit, which makes the discrete outputs (radii, which Gaussians
survive) comparable exactly.
"""
from __future__ import annotations

import torch


def _dot3(a0, b0, a1, b1, a2, b2):
    return (a0 * b0 + a1 * b1) + a2 * b2


def project(means, quats, scales, viewmats, Ks, width: int, height: int, eps2d: float = 0.3, near: float = 0.01, far: float = 1e10):
    """means [N,3], quats [N,4], scales [N,3], viewmats [C,4,4], Ks [C,3,3] (any float dtype; computed in fp32).
    Returns radii [C,N,2] int32, means2d [C,N,2], depths [C,N], conics [C,N,3]."""
    f = lambda t: t.float()  # noqa: E731
    mx, my, mz = f(means).unbind(-1)
    qw, qx, qy, qz = f(quats).unbind(-1)
    nq = torch.sqrt(((qw * qw + qx * qx) + qy * qy) + qz * qz).clamp(min=1e-12)
    qw, qx, qy, qz = qw / nq, qx / nq, qy / nq, qz / nq
    R = [[1 - 2 * (qy * qy + qz * qz), 2 * (qx * qy - qw * qz), 2 * (qx * qz + qw * qy)],
         [2 * (qx * qy + qw * qz), 1 - 2 * (qx * qx + qz * qz), 2 * (qy * qz - qw * qx)],
         [2 * (qx * qz - qw * qy), 2 * (qy * qz + qw * qx), 1 - 2 * (qx * qx + qy * qy)]]
    s = f(scales).unbind(-1)
    M = [[R[i][j] * s[j] for j in range(3)] for i in range(3)]
    Sg = [[_dot3(M[i][0], M[k][0], M[i][1], M[k][1], M[i][2], M[k][2]) for k in range(3)] for i in range(3)]      # [N] each
    V = f(viewmats)
    K = f(Ks)
    v = lambda i, j: V[:, i, j][:, None]  # noqa: E731  [C,1] against [N]
    t = [_dot3(v(i, 0), mx, v(i, 1), my, v(i, 2), mz) + v(i, 3) for i in range(3)]                                 # [C,N]
    T = [[_dot3(v(i, 0), Sg[0][j], v(i, 1), Sg[1][j], v(i, 2), Sg[2][j]) for j in range(3)] for i in range(3)]
    Cc = [[_dot3(T[i][0], v(l, 0), T[i][1], v(l, 1), T[i][2], v(l, 2)) for l in range(3)] for i in range(3)]
    fx, fy, cx, cy = K[:, 0, 0][:, None], K[:, 1, 1][:, None], K[:, 0, 2][:, None], K[:, 1, 2][:, None]
    w, h = float(width), float(height)
    tz = t[2]
    tz2 = tz * tz
    tanx, tany = (0.5 * w) / fx, (0.5 * h) / fy
    lxp, lxn = (w - cx) / fx + 0.3 * tanx, cx / fx + 0.3 * tanx
    lyp, lyn = (h - cy) / fy + 0.3 * tany, cy / fy + 0.3 * tany
    txc = tz * torch.minimum(torch.maximum(t[0] / tz, -lxn), lxp)
    tyc = tz * torch.minimum(torch.maximum(t[1] / tz, -lyn), lyp)
    J00, J02, J11, J12 = fx / tz, (-fx * txc) / tz2, fy / tz, (-fy * tyc) / tz2
    U0 = [J00 * Cc[0][j] + J02 * Cc[2][j] for j in range(3)]
    U1 = [J11 * Cc[1][j] + J12 * Cc[2][j] for j in range(3)]
    c00, c01 = U0[0] * J00 + U0[2] * J02, U0[1] * J11 + U0[2] * J12
    c10, c11 = U1[0] * J00 + U1[2] * J02, U1[1] * J11 + U1[2] * J12
    k = lambda i, j: K[:, i, j][:, None]  # noqa: E731
    m2x = _dot3(k(0, 0), t[0], k(0, 1), t[1], k(0, 2), tz) / tz
    m2y = _dot3(k(1, 0), t[0], k(1, 1), t[1], k(1, 2), tz) / tz
    aa, dd = c00 + eps2d, c11 + eps2d
    det = (aa * dd - c01 * c10).clamp(min=1e-10)
    conics = torch.stack([dd / det, (-(c01 + c10) / 2.0) / det, aa / det], -1)
    rx, ry = torch.ceil(3.33 * torch.sqrt(aa)), torch.ceil(3.33 * torch.sqrt(dd))
    ok = (tz > near) & (tz < far)
    rx, ry = torch.where(ok, rx, torch.zeros_like(rx)), torch.where(ok, ry, torch.zeros_like(ry))
    inside = ((m2x + rx) > 0) & ((m2x - rx) < w) & ((m2y + ry) > 0) & ((m2y - ry) < h)
    rx, ry = torch.where(inside, rx, torch.zeros_like(rx)), torch.where(inside, ry, torch.zeros_like(ry))
    return torch.stack([rx, ry], -1).int(), torch.stack([m2x, m2y], -1), tz, conics
