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
                ("kv_seg_len", ctypes.c_int32 * 16), ("kv_seg_flag", ctypes.c_int32 * 16), ("kv_seg_ready", ctypes.c_void_p), ("ready_epoch", ctypes.c_uint32),
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
        d.kv_seg_flag[i] = i
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


def zigzag_positions(world: int, rank: int, chunk: int) -> list[int]:
    """Global start positions of the two chunks a rank owns in the load-balanced causal layout:
    the sequence is cut into ``2 * world`` chunks and rank r holds chunks r and 2*world-1-r."""
    return [rank * chunk, (2 * world - 1 - rank) * chunk]


class RingAttention:
    """Context-parallel attention: every rank holds ``rows_local`` rows of one long sequence.

    One launch per forward: communication CTAs of the attention kernel push this rank's K and V into
    the peers' gather buffers while the attention CTAs start on the local rows and pick up remote
    segments as their counters arrive (reference behaviour: a Python loop of isend/irecv steps around
    a materialised-score attention, reference: reference/54_ring_attention.py:29-100).

    ``layout="zigzag"`` (causal load balance: two chunks per rank) or ``"contiguous"``.
    """

    def __init__(self, group, rows_local: int, hq: int, hkv: int, head_dim: int, layout: str = "zigzag",
                 comm_blocks: int = 8):
        W = group.size
        self.group, self.W, self.rows, self.hq, self.hkv, self.D = group, W, rows_local, hq, hkv, head_dim
        self.layout, self.comm_blocks = layout, comm_blocks
        self.segs = 2 if layout == "zigzag" else 1
        if rows_local % (self.segs * 128) != 0:
            raise ValueError("rows per rank must be a multiple of 128 per chunk")
        if W * self.segs > 16:
            raise ValueError("at most 16 KV segments (8 ranks in the zigzag layout)")
        self.seg_rows = rows_local // self.segs
        heap = group.heap
        self.k_gather = heap.empty((W * rows_local, hkv, head_dim), torch.bfloat16)
        self.v_gather = heap.empty((W * rows_local, hkv, head_dim), torch.bfloat16)
        self.flags = heap.empty((max(W * self.segs, 4),), torch.int32)
        self.flags.local.zero_()
        self.calls = 0
        self._fwd_kv = None        # (data_ptr, version) of the K and V the gather buffers currently hold

    def positions(self, rank_in_group: int) -> list[int]:
        if self.layout == "zigzag":
            return zigzag_positions(self.W, rank_in_group, self.seg_rows)
        return [rank_in_group * self.rows]

    @property
    def kv_slots(self):
        """Views of this rank's rows inside the gather buffers (write K, V there to skip the local copy)."""
        r = self.group.rank_in_group
        sl = slice(r * self.rows, (r + 1) * self.rows)
        return self.k_gather.local[sl], self.v_gather.local[sl]

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True, scale: float | None = None):
        """``q`` [rows, hq, d], ``k``/``v`` [rows, hkv, d] (this rank's rows). Returns ``(out, lse)``."""
        W, r = self.W, self.group.rank_in_group
        d = AttnDesc()
        d.batch, d.sq, d.skv, d.hq, d.hkv, d.head_dim = 1, self.rows, W * self.rows, self.hq, self.hkv, self.D
        d.causal = 1 if causal else 0
        d.scale = float(scale if scale is not None else 1.0 / math.sqrt(self.D))
        d.q_seg_rows, d.num_q_segs = self.seg_rows, self.segs
        for i, pos in enumerate(self.positions(r)):
            d.q_seg_pos[i] = pos
        # consumption order: local rows first, then the ranks whose pushes reach us first
        order = [(r - s) % W for s in range(W)]
        n = 0
        in_place = k.data_ptr() == self.kv_slots[0].data_ptr() and v.data_ptr() == self.kv_slots[1].data_ptr()
        for src in order:
            for sgi, pos in enumerate(self.positions(src)):
                d.kv_seg_row0[n] = src * self.rows + sgi * self.seg_rows
                d.kv_seg_pos0[n] = pos
                d.kv_seg_len[n] = self.seg_rows
                d.kv_seg_flag[n] = -1 if (src == r and in_place) else src * self.segs + sgi
                n += 1
        d.num_kv_segs = n
        self.calls += 1
        d.ready_epoch = self.calls
        out = torch.empty((self.rows, self.hq, self.D), dtype=torch.bfloat16, device=q.device)
        lse = torch.empty((1, self.hq, self.rows), dtype=torch.float32, device=q.device)
        if not in_place and W > 0:
            pass  # the communication CTAs copy the local rows into the gather buffers too
        nv.check(nv.cuda_lib().pkb_flash_attn_fwd_ring(
            ctypes.byref(d), self.group.ref, nv.ptr(q.contiguous()), nv.ptr(k.contiguous()), nv.ptr(v.contiguous()),
            ctypes.c_ulonglong(self.k_gather.offset), ctypes.c_ulonglong(self.v_gather.offset),
            ctypes.c_ulonglong(self.flags.offset), self.segs, self.seg_rows, self.comm_blocks, nv.ptr(out), nv.ptr(lse),
            nv.current_stream()), "pkb_flash_attn_fwd_ring")
        nv.count_launch()
        self._fwd_kv = (k.data_ptr(), v.data_ptr(), k._version, v._version)
        return out, lse

    __call__ = forward

    def backward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, lse: torch.Tensor, dout: torch.Tensor,
                 causal: bool = True, scale: float | None = None, fused: bool | None = None):
        """Gradients of :meth:`forward`. Returns ``(dq, dk, dv)`` in fp32 for this rank's rows.

        Fused form (default on GPUs; ``PKB_RING_BWD_UNFUSED=1`` or ``fused=False`` selects the other): K and V of the whole
        group are read from the gather buffers the forward call filled (nothing is gathered again when ``k`` / ``v`` are the
        tensors of the last forward call), and the backward kernel adds the dK / dV rows of every KV segment straight into
        the fp32 accumulator of the rank that owns the segment - ``red.global.add.v4.f32`` over peer pointers from its
        epilogue. Two barrier launches bracket it (accumulators zeroed everywhere before, all additions landed after). Per
        rank (W-1)/W of one fp32 dK + dV cross NVLink once, and no whole-sequence partial buffer is written or re-read
        (reference behaviour: a ring of send/recv steps around per-block gradients, reference/57_ring_attention_backward_dp.py:72-121).

        Unfused form: all-gather of K and V, single-GPU backward into fp32 partials for every row of the sequence, one
        reduce-scatter per tensor."""
        import os

        from . import collectives as C

        W, r = self.W, self.group.rank_in_group
        if fused is None:
            fused = os.environ.get("PKB_RING_BWD_UNFUSED") != "1"
        q_segments = [(self.seg_rows, pos) for pos in self.positions(r)]
        kv_segments = [(src * self.rows + sgi * self.seg_rows, pos, self.seg_rows) for src in range(W)
                       for sgi, pos in enumerate(self.positions(src))]
        if W > 1 and fused and q.is_cuda and q.dtype == torch.bfloat16:
            return self._backward_fused(q, k, v, out, lse, dout, causal, scale, q_segments, kv_segments)
        if W > 1:
            kg = C.all_gather(k.contiguous(), self.group).view(W * self.rows, self.hkv, self.D)
            vg = C.all_gather(v.contiguous(), self.group).view(W * self.rows, self.hkv, self.D)
        else:
            kg, vg = k, v
        dk_buf = dv_buf = None
        if W > 1:      # partial sums for every KV row of the group live in the heap: the reduce-scatter reads them in place
            heap = self.group.heap
            shape = (W * self.rows, self.hkv, self.D)
            dk_buf = heap.named(("ring_dk", self.group.channel, shape), shape, torch.float32).local
            dv_buf = heap.named(("ring_dv", self.group.channel, shape), shape, torch.float32).local
        dq, dkf, dvf = flash_attn_bwd(q, kg, vg, out, lse.reshape(self.hq, self.rows), dout, causal=causal, scale=scale,
                                      q_segments=q_segments, kv_segments=kv_segments, dk_out=dk_buf, dv_out=dv_buf)
        if W > 1:
            return dq, C.reduce_scatter(dkf, self.group), C.reduce_scatter(dvf, self.group)
        return dq, dkf, dvf

    def _backward_fused(self, q, k, v, out, lse, dout, causal, scale, q_segments, kv_segments):
        from . import collectives as C

        W, r = self.W, self.group.rank_in_group
        heap = self.group.heap
        same_kv = self._fwd_kv == (k.data_ptr(), v.data_ptr(), k._version, v._version)
        if not same_kv:
            # K / V are not what the last forward call gathered: gather them into the same buffers
            C.all_gather(k.contiguous(), self.group, out=self.k_gather.local.view(W, self.rows, self.hkv, self.D))
            C.all_gather(v.contiguous(), self.group, out=self.v_gather.local.view(W, self.rows, self.hkv, self.D))
        kg, vg = self.k_gather.local, self.v_gather.local
        shape = (self.rows, self.hkv, self.D)
        dk_acc = heap.named(("ring_dk_acc", self.group.channel, shape), shape, torch.float32)
        dv_acc = heap.named(("ring_dv_acc", self.group.channel, shape), shape, torch.float32)
        dk_acc.local.zero_()
        dv_acc.local.zero_()
        C.barrier(self.group)                                  # every accumulator is zero before any rank adds to it
        d = AttnDesc()
        d.batch, d.sq, d.skv, d.hq, d.hkv, d.head_dim = 1, self.rows, W * self.rows, self.hq, self.hkv, self.D
        d.causal = 1 if causal else 0
        d.scale = float(scale if scale is not None else 1.0 / math.sqrt(self.D))
        d.q_seg_rows, d.num_q_segs = q_segments[0][0], len(q_segments)
        for i, (_, pos) in enumerate(q_segments):
            d.q_seg_pos[i] = pos
        d.num_kv_segs = len(kv_segments)
        seg_bytes = self.seg_rows * self.hkv * self.D * 4
        dk_ptrs, dv_ptrs = (ctypes.c_ulonglong * 16)(), (ctypes.c_ulonglong * 16)()
        for i, (row0, pos0, ln) in enumerate(kv_segments):
            d.kv_seg_row0[i], d.kv_seg_pos0[i], d.kv_seg_len[i] = row0, pos0, ln
            src, sgi = divmod(i, self.segs)                   # kv_segments is rank-major, segment-minor
            owner = self.group.members[src]
            dk_ptrs[i] = (heap.base + owner * heap.stride + dk_acc.offset) + sgi * seg_bytes
            dv_ptrs[i] = (heap.base + owner * heap.stride + dv_acc.offset) + sgi * seg_bytes
        qc, oc, doc = (t.contiguous() for t in (q, out, dout))
        lsec = lse.reshape(1, self.hq, self.rows).float().contiguous()
        delta, lse2 = torch.empty_like(lsec), torch.empty_like(lsec)
        dq = torch.zeros((self.rows, self.hq, self.D), dtype=torch.float32, device=q.device)
        nv.check(nv.cuda_lib().pkb_flash_attn_bwd_scatter(ctypes.byref(d), nv.ptr(qc), nv.ptr(kg), nv.ptr(vg), nv.ptr(oc), nv.ptr(doc),
                                                          nv.ptr(lsec), nv.ptr(delta), nv.ptr(lse2), nv.ptr(dq), dk_ptrs, dv_ptrs,
                                                          nv.current_stream()), "pkb_flash_attn_bwd_scatter")
        nv.count_launch(2)
        C.barrier(self.group)                                  # all ranks' additions into this rank's rows have landed
        return dq, dk_acc.local, dv_acc.local


def flash_attn_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, lse: torch.Tensor, dout: torch.Tensor, *,
                   causal: bool, scale: float | None = None, q_pos0: int = 0,
                   q_segments: list[tuple[int, int]] | None = None, kv_segments: list[tuple[int, int, int]] | None = None,
                   dk_out: torch.Tensor | None = None, dv_out: torch.Tensor | None = None):
    """Attention backward from a saved forward. ``q, out, dout`` [Sq, Hq, D] (or [B, Sq, Hq, D]); ``k, v`` [Skv, Hkv, D]
    (or with the batch dimension); ``lse`` [Hq, Sq] (or [B, Hq, Sq]), natural log. Positions are described as in
    :func:`flash_attn_fwd`; without segment lists query row i sits at ``q_pos0 + i`` and key row j at j.
    ``dk_out`` / ``dv_out``: optional fp32 tensors shaped like k / v that receive the result (they are zero-filled here);
    a caller that reduces them over ranks passes symmetric-heap tensors so that the collective needs no staging copy.
    Returns fp32 ``(dq, dk, dv)`` shaped like q, k, v. bf16 inputs with head dimension 64 or 128 run on the tcgen05
    kernel (dK/dV accumulate in TMEM, dQ by fp32 vector reductions); anything else takes the PyTorch restatement."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    squeeze = q.dim() == 3
    if squeeze:
        q, k, v, out, dout, lse = (t.unsqueeze(0) for t in (q, k, v, out, dout, lse))
    B, sq, hq, _ = q.shape
    skv, hkv = k.shape[1], k.shape[2]
    q_segments = q_segments or [(sq, q_pos0)]
    kv_segments = kv_segments or [(0, 0, skv)]
    use_kernel = q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128)
    if not use_kernel:
        from ..refs.attention import attention_bwd_positions_ref

        q_pos = torch.cat([torch.arange(p0, p0 + r, device=q.device) for r, p0 in q_segments])
        kv_rows = torch.cat([torch.arange(r0, r0 + ln, device=q.device) for r0, _, ln in kv_segments])
        kv_pos = torch.cat([torch.arange(p0, p0 + ln, device=q.device) for _, p0, ln in kv_segments])
        dq = torch.empty(q.shape, dtype=torch.float32, device=q.device)
        dk = dk_out.view(k.shape).zero_() if dk_out is not None else torch.zeros(k.shape, dtype=torch.float32, device=q.device)
        dv = dv_out.view(v.shape).zero_() if dv_out is not None else torch.zeros(v.shape, dtype=torch.float32, device=q.device)
        step = max(1, min(sq, (1 << 26) // max(kv_rows.numel() * hq, 1)))        # bound the score matrix held at once
        for b in range(B):
            kb, vb = k[b][kv_rows], v[b][kv_rows]
            for s0 in range(0, sq, step):
                s1 = min(sq, s0 + step)
                a, bb, c = attention_bwd_positions_ref(q[b, s0:s1], kb, vb, out[b, s0:s1], lse[b][:, s0:s1], dout[b, s0:s1],
                                                       q_pos[s0:s1], kv_pos, causal, scale)
                dq[b, s0:s1] = a
                dk[b].index_add_(0, kv_rows, bb)
                dv[b].index_add_(0, kv_rows, c)
    else:
        d = AttnDesc()
        d.batch, d.sq, d.skv, d.hq, d.hkv, d.head_dim = B, sq, skv, hq, hkv, D
        d.causal, d.scale = (1 if causal else 0), float(scale)
        if len({r for r, _ in q_segments}) != 1:
            raise ValueError("all q runs must have the same number of rows")
        d.q_seg_rows, d.num_q_segs = q_segments[0][0], len(q_segments)
        for i, (_, pos) in enumerate(q_segments):
            d.q_seg_pos[i] = pos
        d.num_kv_segs = len(kv_segments)
        for i, (row0, pos0, ln) in enumerate(kv_segments):
            d.kv_seg_row0[i], d.kv_seg_pos0[i], d.kv_seg_len[i] = row0, pos0, ln
        qc, kc, vc, oc, doc = (t.contiguous() for t in (q, k, v, out, dout))
        lsec = lse.float().contiguous()
        delta = torch.empty_like(lsec)
        lse2 = torch.empty_like(lsec)
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        dk = dk_out.view(k.shape).zero_() if dk_out is not None else torch.zeros(k.shape, dtype=torch.float32, device=q.device)
        dv = dv_out.view(v.shape).zero_() if dv_out is not None else torch.zeros(v.shape, dtype=torch.float32, device=q.device)
        nv.check(nv.cuda_lib().pkb_flash_attn_bwd(ctypes.byref(d), nv.ptr(qc), nv.ptr(kc), nv.ptr(vc), nv.ptr(oc), nv.ptr(doc), nv.ptr(lsec),
                                                  nv.ptr(delta), nv.ptr(lse2), nv.ptr(dq), nv.ptr(dk), nv.ptr(dv), nv.current_stream()),
                 "pkb_flash_attn_bwd")
        nv.count_launch(2)
    if squeeze:
        return dq[0], dk[0], dv[0]
    return dq, dk, dv
