"""Expert-parallel MoE primitives (kernels: csrc/kernels/moe.cu, grouped GEMM in csrc/kernels/gemm.cu).

Everything stays on the device: the per-expert counts are all-gathered as a tiny tensor, the plan
kernel turns them into slot bases and grouped-GEMM offsets, the dispatch kernel writes rows straight
into the destination ranks' receive buffers, and the combine kernel pulls expert outputs back over
NVLink. The reference synchronises with the host three times per layer call
(reference: reference/31_fused_moe_fwd.py:60-101).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as nv
from ..parallel.symm_heap import SymmGroup


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, *, epilogue: str = "none",
                 out: torch.Tensor | None = None, block_n: int = 0) -> torch.Tensor:
    """Ragged GEMM: rows ``[offsets[e], offsets[e+1])`` of ``a[rows, K]`` times ``w[e]`` (``w`` is
    ``[G, N, K]``). ``offsets`` is an int32 device tensor ``[G+1]`` that the host never reads.
    ``epilogue="swiglu"`` expects interleaved (gate, up) rows in ``w`` and returns ``N/2`` columns."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.dim() != 3:
        raise TypeError("grouped_gemm expects bf16 a[rows, K] and w[G, N, K]")
    G, N, K = w.shape
    if a.shape[1] != K or a.stride(1) != 1 or not w.is_contiguous():
        raise ValueError("shape mismatch or non-contiguous operand")
    if offsets.dtype != torch.int32 or offsets.numel() != G + 1:
        raise ValueError("offsets must be int32 [G + 1]")
    n_out = N // 2 if epilogue == "swiglu" else N
    if out is None:
        out = torch.empty((a.shape[0], n_out), dtype=torch.bfloat16, device=a.device)
    epi = {"none": 0, "silu": 1, "swiglu": 4}[epilogue]
    nv.check(nv.cuda_lib().pkb_gemm_bf16_grouped(nv.ptr(a), nv.c_ll(a.stride(0)), nv.ptr(w), nv.c_ll(K), nv.ptr(out),
                                                 nv.c_ll(out.stride(0)), nv.ptr(offsets), G, a.shape[0], N, K, epi, block_n,
                                                 nv.current_stream()), "pkb_gemm_bf16_grouped")
    nv.count_launch()
    return out


def grouped_gemm_scatter(a: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, row_meta: torch.Tensor,
                         dest_ptrs: list[int], dest_pitch: int, block_n: int = 0) -> None:
    """Ragged GEMM like :func:`grouped_gemm` whose output row ``m`` is stored as row ``row_meta[m, 1]`` of the bf16 buffer at
    address ``dest_ptrs[row_meta[m, 0]]`` (``dest_pitch`` elements per row) - the buffers may be peers' symmetric memory, so
    the expert outputs travel home from the GEMM's epilogue."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.dim() != 3:
        raise TypeError("grouped_gemm_scatter expects bf16 a[rows, K] and w[G, N, K]")
    G, N, K = w.shape
    if a.shape[1] != K or a.stride(1) != 1 or not w.is_contiguous():
        raise ValueError("shape mismatch or non-contiguous operand")
    if offsets.dtype != torch.int32 or offsets.numel() != G + 1:
        raise ValueError("offsets must be int32 [G + 1]")
    if row_meta.dtype != torch.int32 or row_meta.shape[-1] != 2 or row_meta.shape[0] < a.shape[0] or not row_meta.is_contiguous():
        raise ValueError("row_meta must be a contiguous int32 [>= rows, 2] device tensor")
    if not dest_ptrs or len(dest_ptrs) > 8 or dest_pitch < N or dest_pitch % 8:
        raise ValueError("1..8 destination addresses and a row pitch >= N that is a multiple of 8")
    ptrs = (ctypes.c_ulonglong * len(dest_ptrs))(*dest_ptrs)
    nv.check(nv.cuda_lib().pkb_gemm_bf16_grouped_scatter(nv.ptr(a), nv.c_ll(a.stride(0)), nv.ptr(w), nv.c_ll(K), nv.c_ll(dest_pitch),
                                                         nv.ptr(offsets), G, a.shape[0], N, K, block_n, nv.ptr(row_meta), ptrs,
                                                         len(dest_ptrs), nv.current_stream()), "pkb_gemm_bf16_grouped_scatter")
    nv.count_launch()


def route_topk(logits: torch.Tensor, bias: torch.Tensor | None, top_k: int, counts: torch.Tensor | None = None):
    """Softmax over the experts, top-k and the per-expert histogram in one kernel (one warp per token).

    ``logits`` fp32 ``[T, E]`` (E <= 256), ``bias`` fp32 ``[E]`` or None. Returns ``(gates [T, k] fp32, idx [T, k] int32,
    counts [E] int32)``, the gates in descending order with ties going to the lower expert index - what
    ``torch.topk(torch.softmax(logits + bias, -1), k)`` returns (reference: reference/31_fused_moe_fwd.py:269-277)."""
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise TypeError("logits must be fp32 [T, E] with unit inner stride")
    T, E = logits.shape
    if E > 256 or not 1 <= top_k <= E:
        raise ValueError("at most 256 experts and 1 <= top_k <= E")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != E or not bias.is_contiguous()):
        raise TypeError("bias must be contiguous fp32 [E]")
    gates = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    idx = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
    if counts is None:
        counts = torch.empty(E, dtype=torch.int32, device=logits.device)
    nv.check(nv.cuda_lib().pkb_moe_route(nv.ptr(logits), nv.c_ll(logits.stride(0)), nv.ptr(bias), T, E, top_k, nv.ptr(gates),
                                         nv.ptr(idx), nv.ptr(counts), nv.current_stream()), "pkb_moe_route")
    nv.count_launch()
    return gates, idx, counts


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """``[..., I, H]`` gate and up weights -> ``[..., 2I, H]`` with rows (g0, u0, g1, u1, ...)."""
    return torch.stack([w_gate, w_up], dim=-2).reshape(*w_gate.shape[:-2], 2 * w_gate.shape[-2], w_gate.shape[-1]).contiguous()


class MoEExchange:
    """Dispatch / combine state of one expert-parallel group (buffers live in the symmetric heap)."""

    def __init__(self, group: SymmGroup, num_experts: int, hidden: int, max_tokens: int, top_k: int,
                 capacity_factor: float = 2.0, fp8: bool = True, push_combine: bool = False):
        W = group.size
        if num_experts % W != 0:
            raise ValueError("experts must divide evenly over the expert-parallel group")
        if fp8 and hidden % 128 != 0:
            raise ValueError("fp8 dispatch needs hidden % 128 == 0")
        self.group, self.E, self.El, self.hidden, self.top_k, self.fp8 = group, num_experts, num_experts // W, hidden, top_k, fp8
        self.capacity = int(max_tokens * top_k * capacity_factor + 127) // 128 * 128
        heap = group.heap
        self.payload_bytes = hidden if fp8 else hidden * 2
        self.scale_bytes = ((hidden // 128) * 4 + 15) // 16 * 16 if fp8 else 0
        self.recv_payload = heap.empty((self.capacity, self.payload_bytes), torch.uint8)
        self.recv_scales = heap.empty((self.capacity, max(self.scale_bytes, 16)), torch.uint8)
        # pull combine: the experts write their outputs to `y` (one row per received row) and the token owners pull them.
        # push combine: the dispatch also delivers (sender, assignment index) per row, the down GEMM's epilogue stores each
        # output row into row `assignment index` of the SENDER's `home` buffer, and the combine reads only local memory.
        self.push_combine = push_combine
        if push_combine:
            self.home = heap.empty((max_tokens * top_k, hidden), torch.bfloat16)
            self.recv_meta = heap.empty((self.capacity, 2), torch.int32)
            self.y = self.home
        else:
            self.y = heap.empty((self.capacity, hidden), torch.bfloat16)
        dev = self.y.local.device
        self.counts = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self.seg_base = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self.cursor = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self.offsets = torch.zeros(self.El + 1, dtype=torch.int32, device=dev)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=dev)
        self.slots = None

    # -- planning ------------------------------------------------------------------------------
    def plan(self, expert_idx: torch.Tensor, comm, counts_ready: bool = False) -> torch.Tensor:
        """``expert_idx`` int32 ``[T * k]``. Returns the all-gathered count matrix ``[W, E]`` (device).
        ``counts_ready``: ``self.counts`` already holds this rank's histogram (the fused router wrote it)."""
        lib = nv.cuda_lib()
        if not counts_ready:
            nv.check(lib.pkb_moe_histogram(nv.ptr(expert_idx), nv.c_ll(expert_idx.numel()), self.E, nv.ptr(self.counts),
                                           nv.current_stream()), "pkb_moe_histogram")
            nv.count_launch()
        all_counts = comm.all_gather(self.counts, self.group) if self.group.size > 1 else self.counts.unsqueeze(0)
        nv.check(lib.pkb_moe_plan(nv.ptr(all_counts), self.group.size, self.E, self.El, self.group.rank_in_group,
                                  nv.ptr(self.seg_base), nv.ptr(self.offsets), nv.ptr(self.cursor), nv.current_stream()),
                 "pkb_moe_plan")
        nv.count_launch()
        return all_counts

    # -- dispatch ------------------------------------------------------------------------------
    def dispatch(self, x: torch.Tensor, expert_idx: torch.Tensor, dequantize: bool = True):
        """Send every (token, k) row to its expert's rank. Returns the received rows as bf16
        ``[capacity, hidden]`` (rows ``[0, offsets[-1])`` are valid, expert-major); with
        ``dequantize=False`` (fp8 dispatch only) the received e4m3 bytes ``[capacity, hidden]`` and their fp32
        scales ``[capacity, >= hidden/128]`` instead, as views of the receive buffers."""
        from .elementwise import fp8_dequantize_1x128, fp8_quantize_1x128

        T = x.shape[0]
        self.slots = torch.empty(T * self.top_k, dtype=torch.int32, device=x.device)
        if self.fp8:
            payload, scales = fp8_quantize_1x128(x)
            if self.scale_bytes != scales.shape[1] * 4:
                pad = torch.zeros((T, self.scale_bytes // 4), dtype=torch.float32, device=x.device)
                pad[:, :scales.shape[1]] = scales
                scales = pad
        else:
            payload, scales = x.contiguous(), None
        nv.check(nv.cuda_lib().pkb_moe_dispatch_meta(
            self.group.ref, nv.ptr(payload), nv.ptr(scales), self.payload_bytes, self.scale_bytes, nv.ptr(expert_idx),
            nv.c_ll(T * self.top_k), self.top_k, self.El, nv.ptr(self.seg_base), nv.ptr(self.cursor), nv.ptr(self.slots),
            ctypes.c_ulonglong(self.recv_payload.offset), ctypes.c_ulonglong(self.recv_scales.offset), self.capacity,
            nv.ptr(self.overflow), ctypes.c_ulonglong(self.recv_meta.offset if self.push_combine else 0),
            nv.current_stream()), "pkb_moe_dispatch_meta")
        nv.count_launch()
        if self.fp8 and not dequantize:
            return self.recv_payload.local, self.recv_scales.local.view(torch.float32)
        if not dequantize:
            raise ValueError("dequantize=False needs the fp8 dispatch")
        if self.fp8:
            nblk = self.hidden // 128
            s = self.recv_scales.local.view(torch.float32)[:, :nblk]
            if s.shape[1] * 4 != self.scale_bytes:
                s = s.contiguous()
            # only the rows that arrived (offsets[-1], on the device) are converted: the buffer has capacity_factor x the mean
            return fp8_dequantize_1x128(self.recv_payload.local, s, torch.bfloat16, valid_rows=self.offsets[self.El:self.El + 1])
        return self.recv_payload.local.view(torch.bfloat16)

    def home_ptrs(self) -> list[int]:
        """Addresses of every member's ``home`` buffer, in group order (what ``recv_meta[:, 0]`` indexes)."""
        return [self.home.peer_ptr(r) for r in self.group.members]

    # -- combine -------------------------------------------------------------------------------
    def combine(self, expert_idx: torch.Tensor, gates: torch.Tensor, num_tokens: int) -> torch.Tensor:
        """``out[t] = sum_j gates[t, j] * y_owner[slot[t, j]]`` pulled over NVLink; ``self.y`` holds
        this rank's expert outputs."""
        out = torch.empty((num_tokens, self.hidden), dtype=torch.bfloat16, device=gates.device)
        if self.push_combine and num_tokens * self.top_k > self.home.local.shape[0]:
            raise ValueError("more tokens than the home buffer was sized for")
        nv.check(nv.cuda_lib().pkb_moe_combine_from(self.group.ref, ctypes.c_ulonglong(self.y.offset), nv.ptr(expert_idx),
                                                    nv.ptr(self.slots), nv.ptr(gates.contiguous().float()), nv.ptr(out),
                                                    nv.c_ll(num_tokens), self.top_k, self.hidden, self.El,
                                                    1 if self.push_combine else 0, nv.current_stream()),
                 "pkb_moe_combine_from")
        nv.count_launch()
        return out
