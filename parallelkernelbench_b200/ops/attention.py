"""Flash attention forward on tcgen05 (kernel: csrc/kernels/attention.cu).

Tensors are ``[batch, seq, heads, head_dim]`` bf16 (``head_dim`` 64 or 128), GQA when
``k.shape[2] < q.shape[2]``. ``q_segments`` / ``kv_segments`` describe where the rows sit in the
global sequence, which is how causal masks stay correct for context-parallel (zigzag) layouts.
"""
from __future__ import annotations

import ctypes
import math

import torch

from .. import _native as nv


class AttnDesc(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int32), ("sq", ctypes.c_int32), ("skv", ctypes.c_int32), ("hq", ctypes.c_int32),
                ("hkv", ctypes.c_int32), ("head_dim", ctypes.c_int32), ("causal", ctypes.c_int32), ("scale", ctypes.c_float),
                ("q_seg_rows", ctypes.c_int32), ("num_q_segs", ctypes.c_int32), ("q_seg_pos", ctypes.c_int32 * 16),
                ("num_kv_segs", ctypes.c_int32), ("kv_seg_row0", ctypes.c_int32 * 16), ("kv_seg_pos0", ctypes.c_int32 * 16),
                ("kv_seg_len", ctypes.c_int32 * 16), ("kv_seg_ready", ctypes.c_void_p), ("ready_epoch", ctypes.c_uint32),
                ("_pad", ctypes.c_uint32), ("budget_ns", ctypes.c_uint64), ("trace", ctypes.c_void_p),
                ("trace_capacity", ctypes.c_int32), ("_pad2", ctypes.c_int32)]


def flash_attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = False, scale: float | None = None,
                   q_segments: list[tuple[int, int]] | None = None, kv_segments: list[tuple[int, int, int]] | None = None,
                   kv_ready: torch.Tensor | None = None, ready_epoch: int = 0, return_lse: bool = True,
                   trace: torch.Tensor | None = None):
    """``q_segments``: list of (rows, global_pos0) runs, all runs the same number of rows.
    ``kv_segments``: list of (buffer_row0, global_pos0, length). Defaults: one run starting at 0.
    Returns ``(out, lse)`` with ``lse`` ``[batch, heads, sq]`` (natural log) or ``None``."""
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise TypeError("flash_attn_fwd expects bf16 tensors")
    B, sq, hq, D = q.shape
    _, skv, hkv, _ = k.shape
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        raise ValueError("q, k, v must be contiguous [batch, seq, heads, dim]")
    d = AttnDesc()
    d.batch, d.sq, d.skv, d.hq, d.hkv, d.head_dim = B, sq, skv, hq, hkv, D
    d.causal = 1 if causal else 0
    d.scale = float(scale if scale is not None else 1.0 / math.sqrt(D))
    q_segments = q_segments or [(sq, 0)]
    if len({r for r, _ in q_segments}) != 1 and len(q_segments) > 1:
        raise ValueError("all q runs must have the same number of rows")
    d.q_seg_rows, d.num_q_segs = q_segments[0][0], len(q_segments)
    for i, (_, pos) in enumerate(q_segments):
        d.q_seg_pos[i] = pos
    kv_segments = kv_segments or [(0, 0, skv)]
    d.num_kv_segs = len(kv_segments)
    for i, (row0, pos0, ln) in enumerate(kv_segments):
        d.kv_seg_row0[i], d.kv_seg_pos0[i], d.kv_seg_len[i] = row0, pos0, ln
    d.kv_seg_ready = kv_ready.data_ptr() if kv_ready is not None else None
    d.ready_epoch = ready_epoch
    if trace is not None:            # int64 buffer: [0] = record count, records of (role, event, tile, clock) from word 4
        d.trace, d.trace_capacity = trace.data_ptr(), (trace.numel() - 4) // 4
    out = torch.empty_like(q)
    lse = torch.empty((B, hq, sq), dtype=torch.float32, device=q.device) if return_lse else None
    nv.check(nv.cuda_lib().pkb_flash_attn_fwd(ctypes.byref(d), nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(out), nv.ptr(lse),
                                              nv.current_stream()), "pkb_flash_attn_fwd")
    nv.count_launch()
    return out, lse
