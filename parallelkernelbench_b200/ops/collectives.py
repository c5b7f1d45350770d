"""Collectives over the symmetric heap (kernels: csrc/kernels/collectives.cu).

Each function is one kernel launch: stage (unless the input already lives in the heap) -> in-kernel
barrier -> direct peer loads -> in-kernel barrier. Algorithm choice for all-reduce is by message
size: one-shot below ``ONE_SHOT_MAX_BYTES`` (latency bound: one barrier + one remote read of every
peer), NVLS in-switch reduction above it when the multicast mapping exists, otherwise two-shot.

They cover the bare-collective workloads of the reference (reference: reference/1_allreduce.py ...
reference/8_alltoall.py) and are the building blocks the composite ops call.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as nv
from .. import tuning
from ..parallel.symm_heap import SymmGroup, SymmTensor

ONE_SHOT_MAX_BYTES = 512 * 1024
LL_MAX_BYTES = 1024 * 1024        # data + epoch in one 8-byte store, no barrier (twice the bytes on the wire)
# the automatic choice stops earlier, at the table's ll_max_bytes (measured: 6.8 us vs NCCL 14.2 at 4 KiB, 9.4 vs 17.9 at 64 KiB,
# 23.6 vs 20.5 at 1 MiB)
_DT = {torch.bfloat16: 0, torch.float32: 1, torch.float64: 2, torch.float16: 3, torch.int32: 4, torch.int64: 5}
_OP = {"sum": 0, "max": 1, "min": 2}


def _lib():
    return nv.cuda_lib()


def _stage(group: SymmGroup, key: str, x: torch.Tensor, min_bytes: int = 0) -> tuple[int, int]:
    """Heap offset for ``x`` and how many bytes must be staged (0 when ``x`` is already in the heap)."""
    off = group.heap.contains(x)
    if off is not None and off % 16 == 0:
        return off, 0
    nbytes = max(x.numel() * x.element_size(), min_bytes)
    cap = 1 << max(12, (max(nbytes, 1) - 1).bit_length())
    buf = group.heap.named((key, group.channel), (cap,), torch.uint8)
    return buf.offset, x.numel() * x.element_size()


def _check(x: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        raise ValueError("symmetric-heap collectives need CUDA tensors")
    return x if x.is_contiguous() else x.contiguous()


def barrier(group: SymmGroup, blocks: int = 1) -> None:
    nv.check(_lib().pkb_coll_barrier(group.ref, blocks, nv.current_stream()), "pkb_coll_barrier")
    nv.count_launch()


def _ll_slots(group: SymmGroup, nbytes: int):
    """Slots of the no-barrier exchange for messages of up to ``nbytes`` (three size classes, each with its own epoch)."""
    cap_bytes = 64 * 1024 if nbytes <= 64 * 1024 else (256 * 1024 if nbytes <= 256 * 1024 else LL_MAX_BYTES)
    cap_units = cap_bytes // 4
    key = ("ll_slots", group.channel, cap_units)
    fresh = key not in group.heap._named
    buf = group.heap.named(key, (16 + 2 * group.size * cap_units * 8,), torch.uint8)
    if fresh:                           # epoch words must start at zero everywhere before the first exchange
        buf.local.zero_()
        barrier(group)
    return buf, cap_units


def all_reduce_(x: torch.Tensor, group: SymmGroup, max_blocks: int = 0) -> torch.Tensor:
    """In-place sum all-reduce of a tensor that lives in the symmetric heap (bf16 / fp32, whole-job group with a multicast
    mapping): every rank reduces its slice through the switch (``multimem.ld_reduce``) and writes the sums back to the
    same addresses on all ranks (``multimem.st``). No staging copy, no result buffer, no copy out - the message crosses
    HBM once for the read and once for the write, like NCCL's in-place form on registered buffers
    (reference: kernelgen/solutions_new_allreduce_parallelkittens.py:64-66 reduces in place the same way)."""
    off = group.heap.contains(x)
    if off is None or off % 16 != 0 or not x.is_contiguous():
        raise ValueError("all_reduce_ needs a contiguous, 16-byte aligned tensor allocated from the symmetric heap")
    if not (group.heap.mc_base != 0 and group.is_whole_heap and x.dtype in (torch.bfloat16, torch.float32)):
        raise RuntimeError("in-place all-reduce needs the multicast mapping, the whole-job group and bf16/fp32 data")
    nv.check(_lib().pkb_coll_allreduce_nvls(group.ref, _DT[x.dtype], nv.ptr(x), nv.c_ll(x.numel()), ctypes.c_ulonglong(off),
                                            ctypes.c_ulonglong(off), nv.ptr(None), 1, max_blocks, nv.current_stream()),
             "pkb_coll_allreduce_nvls")
    nv.count_launch()
    return x


def all_reduce(x: torch.Tensor, group: SymmGroup, op: str = "sum", out: torch.Tensor | None = None,
               algo: str = "auto", scale: float = 1.0, max_blocks: int = 0) -> torch.Tensor:
    x = _check(x)
    if x.dtype not in _DT:
        raise TypeError(f"unsupported dtype {x.dtype}")
    if out is None:
        out = torch.empty_like(x)
    n = x.numel()
    nbytes = n * x.element_size()
    nvls_ok = (group.heap.mc_base != 0 and group.is_whole_heap and op == "sum" and scale == 1.0
               and x.dtype in (torch.bfloat16, torch.float32))
    ll_ok = nbytes <= LL_MAX_BYTES and x.dtype in (torch.bfloat16, torch.float32) and group.size > 1
    if algo == "auto":
        # thresholds come from the tuning table (tuning/collectives_b200.json). Measured on B200 (device time under CUDA-graph
        # replay, 2 ranks, NCCL in brackets): the no-barrier exchange 6.7 us at 4 KiB (13.8), 9.0 us at 64 KiB (17.2); one-shot
        # 52.6 us at 16 MiB (59.0); two-shot 261 us at 128 MiB (285), the in-switch form 429 us there - with two ranks a peer
        # read costs the same as the switch reduction, so NVLS is used from four ranks on, where one-shot would read (W-1) copies
        algo = tuning.all_reduce_algo(nbytes, group.size, ll_ok=ll_ok, nvls_ok=nvls_ok)
    lib = _lib()
    if algo == "ll":
        if not ll_ok:
            raise RuntimeError("the latency-optimised all-reduce takes bf16/fp32 messages of at most 1 MiB on 2+ ranks")
        buf, cap_units = _ll_slots(group, nbytes)
        nv.check(lib.pkb_coll_allreduce_ll(group.ref, _DT[x.dtype], _OP[op], nv.ptr(x), nv.c_ll(n), ctypes.c_ulonglong(buf.offset),
                                           nv.c_ll(cap_units), nv.ptr(out), ctypes.c_double(scale), nv.current_stream()),
                 "pkb_coll_allreduce_ll")
        nv.count_launch()
        return out
    off, stage_bytes = _stage(group, "ar_in", x)
    if algo == "oneshot":
        nv.check(lib.pkb_coll_reduce(group.ref, _DT[x.dtype], _OP[op], nv.ptr(x),
                                     nv.c_ll(n if stage_bytes else 0), ctypes.c_ulonglong(off), nv.c_ll(0),
                                     nv.c_ll(n), nv.ptr(out), 1, ctypes.c_double(scale), max_blocks,
                                     nv.current_stream()), "pkb_coll_reduce")
    elif algo == "twoshot":
        res = group.heap.named(("ar_res", group.channel), (1 << max(12, (nbytes - 1).bit_length()),), torch.uint8)
        nv.check(lib.pkb_coll_allreduce_twoshot(group.ref, _DT[x.dtype], _OP[op], nv.ptr(x), nv.c_ll(n),
                                                ctypes.c_ulonglong(off), ctypes.c_ulonglong(res.offset),
                                                nv.ptr(out), 0 if stage_bytes else 1, ctypes.c_double(scale),
                                                max_blocks, nv.current_stream()), "pkb_coll_allreduce_twoshot")
    elif algo == "nvls":
        if not nvls_ok:
            raise RuntimeError("NVLS all-reduce not available for this call (needs multicast, sum, bf16/fp32, whole job)")
        res = group.heap.named(("ar_res", group.channel), (1 << max(12, (nbytes - 1).bit_length()),), torch.uint8)
        nv.check(lib.pkb_coll_allreduce_nvls(group.ref, _DT[x.dtype], nv.ptr(x), nv.c_ll(n),
                                             ctypes.c_ulonglong(off), ctypes.c_ulonglong(res.offset), nv.ptr(out),
                                             0 if stage_bytes else 1, max_blocks, nv.current_stream()),
                 "pkb_coll_allreduce_nvls")
    else:
        raise ValueError(f"unknown all-reduce algorithm {algo!r}")
    nv.count_launch()
    return out


def _nvls_ok(group: SymmGroup) -> bool:
    return group.heap.mc_base != 0 and group.is_whole_heap and group.size > 1


def reduce_scatter(x: torch.Tensor, group: SymmGroup, op: str = "sum", out: torch.Tensor | None = None,
                   scale: float = 1.0, algo: str = "auto") -> torch.Tensor:
    """``x`` is ``[W * n, ...]``; rank g receives the reduction of chunk g. ``algo``: ``"pull"`` (peer loads), ``"nvls"``
    (the switch adds: ``multimem.ld_reduce`` of this rank's slice; bf16 / fp32 sums on the whole-job group) or ``"auto"``
    (NVLS for slices of ``tuning.reduce_scatter_nvls_min`` bytes and more)."""
    x = _check(x)
    W = group.size
    if x.shape[0] % W != 0:
        raise ValueError("leading dimension must be divisible by the group size")
    n = x.numel() // W
    if out is None:
        out = torch.empty((x.shape[0] // W, *x.shape[1:]), dtype=x.dtype, device=x.device)
    nvls_fit = (_nvls_ok(group) and op == "sum" and scale == 1.0 and x.dtype in (torch.bfloat16, torch.float32)
                and (n * x.element_size()) % 16 == 0 and out.is_contiguous() and out.data_ptr() % 16 == 0)
    if algo == "nvls" and not nvls_fit:
        raise RuntimeError("NVLS reduce-scatter needs multicast, the whole-job group, a bf16/fp32 sum and 16-byte slices")
    if algo == "nvls" or (algo == "auto" and nvls_fit and n * x.element_size() >= tuning.reduce_scatter_nvls_min(W)):
        off, stage_bytes = _stage(group, "rs_in", x)
        nv.check(_lib().pkb_coll_reduce_scatter_nvls(group.ref, _DT[x.dtype], nv.ptr(x), nv.c_ll(n), ctypes.c_ulonglong(off),
                                                     nv.ptr(out), 0 if stage_bytes else 1, 0, nv.current_stream()),
                 "pkb_coll_reduce_scatter_nvls")
        nv.count_launch()
        return out
    off, stage_bytes = _stage(group, "rs_in", x)
    nv.check(_lib().pkb_coll_reduce(group.ref, _DT[x.dtype], _OP[op], nv.ptr(x),
                                    nv.c_ll(x.numel() if stage_bytes else 0), ctypes.c_ulonglong(off),
                                    nv.c_ll(n * group.rank_in_group), nv.c_ll(n), nv.ptr(out), 1,
                                    ctypes.c_double(scale), 0, nv.current_stream()), "pkb_coll_reduce")
    nv.count_launch()
    return out


def reduce(x: torch.Tensor, group: SymmGroup, dst: int = 0, op: str = "sum") -> torch.Tensor:
    """Sum to group member ``dst``; other members get their input back unchanged."""
    x = _check(x)
    is_root = group.rank_in_group == dst
    out = torch.empty_like(x) if is_root else x
    off, stage_bytes = _stage(group, "red_in", x)
    nv.check(_lib().pkb_coll_reduce(group.ref, _DT[x.dtype], _OP[op], nv.ptr(x),
                                    nv.c_ll(x.numel() if stage_bytes else 0), ctypes.c_ulonglong(off), nv.c_ll(0),
                                    nv.c_ll(x.numel()), nv.ptr(out), 1 if is_root else 0, ctypes.c_double(1.0), 0,
                                    nv.current_stream()), "pkb_coll_reduce")
    nv.count_launch()
    return out


def _gather_call(group, x, mask, in_base, member_stride, seg_bytes, out, out_stride, active, key):
    off, stage_bytes = _stage(group, key, x)
    nv.check(_lib().pkb_coll_gather(group.ref, nv.ptr(x), nv.c_ll(stage_bytes), ctypes.c_ulonglong(off),
                                    ctypes.c_uint(mask), nv.c_ll(in_base), nv.c_ll(member_stride),
                                    nv.c_ll(seg_bytes), nv.ptr(out), nv.c_ll(out_stride), 1 if active else 0, 0,
                                    nv.current_stream()), "pkb_coll_gather")
    nv.count_launch()


def all_gather(x: torch.Tensor, group: SymmGroup, out: torch.Tensor | None = None, algo: str = "auto") -> torch.Tensor:
    """Returns ``[W, *x.shape]`` (member order). ``algo``: ``"pull"`` (peer loads / TMA-bulk requests), ``"nvls"`` (every rank
    stores its shard once through the multicast mapping and the switch replicates it) or ``"auto"`` (NVLS for shards of
    ``tuning.all_gather_nvls_min`` bytes and more on the whole-job group)."""
    x = _check(x)
    W = group.size
    if out is None:
        out = torch.empty((W, *x.shape), dtype=x.dtype, device=x.device)
    nb = x.numel() * x.element_size()
    nvls_fit = _nvls_ok(group) and nb % 16 == 0 and x.data_ptr() % 16 == 0 and out.is_contiguous() and out.data_ptr() % 16 == 0
    if algo == "nvls" and not nvls_fit:
        raise RuntimeError("NVLS all-gather needs multicast, the whole-job group and 16-byte aligned shards")
    if algo == "nvls" or (algo == "auto" and nvls_fit and nb >= tuning.all_gather_nvls_min(W)):
        goff = group.heap.contains(out)
        direct = goff is not None and goff % 16 == 0          # the caller's result already lives in the heap: no copy out
        if not direct:
            cap = 1 << max(12, (W * nb - 1).bit_length())
            goff = group.heap.named(("ag_nvls", group.channel), (cap,), torch.uint8).offset
        nv.check(_lib().pkb_coll_allgather_nvls(group.ref, nv.ptr(x), nv.c_ll(nb), ctypes.c_ulonglong(goff),
                                                nv.ptr(None if direct else out), 0, nv.current_stream()), "pkb_coll_allgather_nvls")
        nv.count_launch()
        return out
    if W > 1 and 0 < nb <= tuning.all_gather_ll_max(W) and nb % 4 == 0 and x.data_ptr() % 4 == 0 and out.is_contiguous():
        buf, cap_units = _ll_slots(group, nb)
        nv.check(_lib().pkb_coll_allgather_ll(group.ref, nv.ptr(x), nv.c_ll(nb // 4), ctypes.c_ulonglong(buf.offset), nv.c_ll(cap_units),
                                              nv.ptr(out), nv.current_stream()), "pkb_coll_allgather_ll")
        nv.count_launch()
        return out
    _gather_call(group, x, (1 << W) - 1, 0, 0, nb, out, nb, True, "ag_in")
    return out


def all_to_all(x: torch.Tensor, group: SymmGroup, out: torch.Tensor | None = None, algo: str = "auto") -> torch.Tensor:
    """``x`` is ``[W, ...]``; ``out[g] = x_of_member_g[my index]``. ``algo``: ``"pull"`` (stage the input in the heap, receivers
    read their chunks from the peers), ``"push"`` (TMA bulk loads of the local input, TMA bulk stores into the receivers'
    buffers; no staging copy, and no copy out when ``out`` lives in the symmetric heap at the same offset on every member) or
    ``"auto"`` (push for chunks of ``tuning.all_to_all_push_min`` bytes and more)."""
    x = _check(x)
    W = group.size
    if x.shape[0] != W:
        raise ValueError("leading dimension must equal the group size")
    if out is None:
        out = torch.empty_like(x)
    chunk = x[0].numel() * x.element_size()
    push_fit = W > 1 and chunk % 16 == 0 and x.data_ptr() % 16 == 0 and out.is_contiguous() and out.data_ptr() % 16 == 0
    if algo == "push" and not push_fit:
        raise RuntimeError("the push all-to-all needs more than one member and 16-byte aligned chunks")
    goff = group.heap.contains(out) if push_fit else None
    direct = goff is not None and goff % 16 == 0              # the senders store straight into the caller's result
    # with a result outside the heap the push pays a local copy out of the receive buffer, so it takes over later
    push_min = tuning.all_to_all_push_min(W, direct=direct)
    if algo == "push" or (algo == "auto" and push_fit and chunk >= push_min):
        if not direct:
            cap = 1 << max(12, (W * chunk - 1).bit_length())
            goff = group.heap.named(("a2a_push", group.channel), (cap,), torch.uint8).offset
        nv.check(_lib().pkb_coll_all_to_all_push(group.ref, nv.ptr(x), nv.c_ll(chunk), ctypes.c_ulonglong(goff),
                                                 nv.ptr(None if direct else out), 0, nv.current_stream()), "pkb_coll_all_to_all_push")
        nv.count_launch()
        return out
    _gather_call(group, x, (1 << W) - 1, 0, chunk, chunk, out, chunk, True, "a2a_in")
    return out


def broadcast(x: torch.Tensor, group: SymmGroup, src: int = 0, algo: str = "auto") -> torch.Tensor:
    """Every member receives member ``src``'s tensor. ``algo``: ``"pull"`` (stage at the root, the others read it), ``"nvls"`` (the
    root stores once through the multicast mapping and the switch replicates it) or ``"auto"`` (NVLS from
    ``tuning.broadcast_nvls_min`` bytes on the whole-job group)."""
    x = _check(x)
    out = torch.empty_like(x)
    nb = x.numel() * x.element_size()
    nvls_fit = _nvls_ok(group) and nb % 16 == 0 and x.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
    if algo == "nvls" and not nvls_fit:
        raise RuntimeError("NVLS broadcast needs multicast, the whole-job group and a 16-byte aligned tensor")
    if algo == "nvls" or (algo == "auto" and nvls_fit and nb >= tuning.broadcast_nvls_min(group.size)):
        cap = 1 << max(12, (nb - 1).bit_length())
        boff = group.heap.named(("bc_nvls", group.channel), (cap,), torch.uint8).offset
        nv.check(_lib().pkb_coll_broadcast_nvls(group.ref, nv.ptr(x), nv.c_ll(nb), int(src), ctypes.c_ulonglong(boff), nv.ptr(out), 0,
                                                nv.current_stream()), "pkb_coll_broadcast_nvls")
        nv.count_launch()
        return out
    _gather_call(group, x, 1 << src, 0, 0, nb, out, nb, True, "bc_in")
    return out


def scatter(x: torch.Tensor, group: SymmGroup, src: int = 0) -> torch.Tensor:
    """Member ``src`` holds ``[W, ...]``; every member receives its chunk. All members pass a
    tensor of the full shape (only the root's content is used)."""
    x = _check(x)
    out = torch.empty_like(x[0])
    chunk = x[0].numel() * x.element_size()
    _gather_call(group, x, 1 << src, 0, chunk, chunk, out, chunk, True, "sc_in")
    return out


def gather(x: torch.Tensor, group: SymmGroup, dst: int = 0) -> torch.Tensor:
    """Member ``dst`` receives ``[W, *x.shape]``; the others get their input back."""
    x = _check(x)
    is_root = group.rank_in_group == dst
    W = group.size
    out = torch.empty((W, *x.shape), dtype=x.dtype, device=x.device) if is_root else x
    nb = x.numel() * x.element_size()
    _gather_call(group, x, (1 << W) - 1, 0, 0, nb, out, nb, is_root, "ga_in")
    return out


def row_gather(shard: torch.Tensor, ids: torch.Tensor, group: SymmGroup, resident: bool = False) -> torch.Tensor:
    """Lookup in a table sharded by rows over the group: ``out[i] = table[ids[i]]`` where member ``g`` owns rows
    ``[g * S, (g + 1) * S)`` and ``shard`` is this member's ``[S, ...]`` slice. Rows are fetched with direct peer loads,
    so no request/reply exchange is needed (the reference does three all-to-alls: reference/10_embedding_lookup.py).
    ``resident=True``: ``shard`` lives in the symmetric heap and has not changed since the last barrier - no staging,
    no barriers."""
    shard = _check(shard)
    idc = ids.contiguous().view(-1).to(torch.int64)
    S = shard.shape[0]
    row_bytes = (shard.numel() // max(S, 1)) * shard.element_size()
    if resident:
        off = group.heap.contains(shard)
        if off is None:
            raise ValueError("resident=True needs a shard allocated in the symmetric heap")
        stage_bytes = 0
    else:
        off, stage_bytes = _stage(group, "rowgather_in", shard)
    out = torch.empty((idc.numel(), *shard.shape[1:]), dtype=shard.dtype, device=shard.device)
    nv.check(_lib().pkb_coll_row_gather(group.ref, nv.ptr(shard), nv.c_ll(stage_bytes), ctypes.c_ulonglong(off), nv.ptr(idc),
                                        nv.c_ll(idc.numel()), nv.c_ll(S), nv.c_ll(row_bytes), nv.ptr(out), 0 if resident else 1,
                                        0, nv.current_stream()), "pkb_coll_row_gather")
    nv.count_launch()
    return out.view(*ids.shape, *shard.shape[1:])


def _collapse(shape, in_st, out_st):
    """Merge adjacent dimensions that are contiguous in both layouts; returns lists (outermost first)."""
    dims = [(n, a, b) for n, a, b in zip(shape, in_st, out_st) if n != 1]
    merged: list[list[int]] = []
    for n, a, b in dims:
        if merged and merged[-1][1] == a * n and merged[-1][2] == b * n:
            merged[-1] = [merged[-1][0] * n, a, b]
        else:
            merged.append([n, a, b])
    return merged


def all_to_all_permute(x: torch.Tensor, group: SymmGroup, scatter_dim: int, gather_dim: int) -> torch.Tensor:
    """Split ``x`` along ``scatter_dim`` into W parts, send part g to member g, and concatenate what arrives along
    ``gather_dim`` - in one launch, with the layout change done by the peer loads themselves (the reference chunks,
    exchanges a list and concatenates: reference/33_ulysses_all_to_all_tensor_primitive.py:9-22)."""
    x = _check(x)
    W, r = group.size, group.rank_in_group
    sd, gd = scatter_dim % x.ndim, gather_dim % x.ndim
    if x.shape[sd] % W != 0:
        raise ValueError("scatter dimension must be divisible by the group size")
    es = x.element_size()
    box = list(x.shape)
    box[sd] //= W
    out_shape = list(box)
    out_shape[gd] *= W
    out = torch.empty(out_shape, dtype=x.dtype, device=x.device)
    in_st = [s * es for s in x.stride()]
    out_st = [s * es for s in out.stride()]
    m = _collapse(box, in_st, out_st)
    inner = es
    if m and m[-1][1] == es and m[-1][2] == es:
        inner = m[-1][0] * es
        m = m[:-1]
    if len(m) > 3:
        raise ValueError("layout change needs more than three strided dimensions")
    while len(m) < 3:
        m.insert(0, [1, 0, 0])
    ext = (ctypes.c_longlong * 3)(*[d[0] for d in m])
    ist = (ctypes.c_longlong * 3)(*[d[1] for d in m])
    ost = (ctypes.c_longlong * 3)(*[d[2] for d in m])
    off, stage_bytes = _stage(group, "a2ap_in", x)
    nv.check(_lib().pkb_coll_a2a_permute(group.ref, nv.ptr(x), nv.c_ll(stage_bytes), ctypes.c_ulonglong(off),
                                         nv.c_ll(box[sd] * in_st[sd]), ext, ist, nv.c_ll(box[gd] * out_st[gd]), ost,
                                         nv.c_ll(inner), nv.ptr(out), 0, nv.current_stream()), "pkb_coll_a2a_permute")
    nv.count_launch()
    return out


def all_to_all_v(x: torch.Tensor, send_counts: torch.Tensor, group: SymmGroup, out_capacity_rows: int,
                 send_offsets: torch.Tensor | None = None, max_send_rows: int | None = None):
    """Variable all-to-all of rows. ``x`` is ``[rows, ...]`` grouped by destination, ``send_counts``
    an int64 device tensor ``[W]``. Returns ``(out[out_capacity_rows, ...], recv_counts[W], total[1])``;
    counts stay on the device - there is no host round trip (the reference pays one ``.tolist()``
    per exchange, reference: reference/31_fused_moe_fwd.py:60-101). ``out_capacity_rows`` and
    ``max_send_rows`` (default: ``out_capacity_rows``) must be the same on every rank: they size the
    symmetric staging buffer."""
    x = _check(x)
    W = group.size
    if send_counts.dtype != torch.int64 or send_counts.numel() != W:
        raise ValueError("send_counts must be int64 [W]")
    if send_offsets is None:
        send_offsets = torch.cumsum(send_counts, 0) - send_counts
    rows = x.shape[0]
    row_elems = 1
    for d in x.shape[1:]:
        row_elems *= int(d)
    row_bytes = row_elems * x.element_size()
    max_send_rows = out_capacity_rows if max_send_rows is None else max_send_rows
    if rows > max_send_rows:
        raise ValueError(f"{rows} rows to send exceed max_send_rows={max_send_rows}")
    cap = 1 << max(12, (max(max_send_rows * row_bytes, 1) - 1).bit_length())
    stage = group.heap.named(("a2av_in", group.channel), (cap,), torch.uint8)
    meta = group.heap.named(("a2av_meta", group.channel), (2 * 16,), torch.int64)
    out = torch.empty((out_capacity_rows, *x.shape[1:]), dtype=x.dtype, device=x.device)
    recv_counts = torch.empty(W, dtype=torch.int64, device=x.device)
    total = torch.empty(1, dtype=torch.int64, device=x.device)
    nv.check(_lib().pkb_coll_all_to_all_v(group.ref, nv.ptr(x), nv.c_ll(rows), nv.c_ll(row_bytes),
                                          nv.ptr(send_counts), nv.ptr(send_offsets.contiguous()),
                                          ctypes.c_ulonglong(stage.offset), ctypes.c_ulonglong(meta.offset),
                                          nv.ptr(out), nv.c_ll(out_capacity_rows), nv.ptr(recv_counts),
                                          nv.ptr(total), 0, nv.current_stream()), "pkb_coll_all_to_all_v")
    nv.count_launch()
    return out, recv_counts, total


__all__ = ["barrier", "all_reduce", "reduce_scatter", "reduce", "all_gather", "all_to_all", "broadcast",
           "scatter", "gather", "all_to_all_v", "SymmTensor", "SymmGroup"]
