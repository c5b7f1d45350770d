"""CPU twin of the symmetric heap (native part: csrc/runtime/host_shm.cpp).

Ranks are processes of one host sharing a POSIX shared-memory segment; the collectives follow the
same stage -> barrier -> read peers -> barrier protocol as the CUDA kernels, with ``std::atomic``
flags. It exists for machines without a GPU (the gloo plumbing configuration) and for fault
injection on the host: ``drop_signals`` / ``delay_ms`` make a rank misbehave, and every wait is
bounded, so survivors get a :class:`HostCollectiveTimeout` naming the missing peer.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np
import torch
import torch.distributed as dist

from .. import _native as nv

_DT = {torch.bfloat16: 0, torch.float32: 1, torch.float64: 2, torch.int32: 4, torch.int64: 5}
_OP = {"sum": 0, "max": 1, "min": 2}
CTRL_BYTES = 1 << 20


class HostCollectiveTimeout(RuntimeError):
    def __init__(self, msg: str, missing_peer: int):
        super().__init__(msg)
        self.missing_peer = missing_peer


class HostGroup:
    def __init__(self, heap: "HostHeap", members: list[int], channel: int):
        self.heap = heap
        self.members = list(members)
        self.size = len(members)
        self.channel = channel
        self.rank_in_group = members.index(heap.rank) if heap.rank in members else -1
        self.c_members = (ctypes.c_int * len(members))(*members)


class HostHeap:
    def __init__(self, handle: int, name: str, rank: int, world: int, nbytes: int, timeout_ms: int):
        self.handle, self.name, self.rank, self.world, self.nbytes = handle, name, rank, world, nbytes
        self.timeout_ms = timeout_ms
        self._top = CTRL_BYTES
        self._next_channel = 0
        self._groups: dict = {}
        self.world_group = self.group(list(range(world)))

    @classmethod
    def create(cls, ctx=None, nbytes: int = 64 << 20, name: str | None = None, rank: int | None = None,
               world: int | None = None, timeout_ms: int = 30000) -> "HostHeap":
        lib = nv.host_lib()
        lib.pkbh_heap_local.restype = ctypes.c_void_p
        lib.pkbh_heap_peer.restype = ctypes.c_void_p
        if ctx is not None:
            rank, world = ctx.rank, ctx.world
        if name is None:
            tok = [f"/pkb200_{os.getpid()}_{os.environ.get('MASTER_PORT', '0')}"] if rank == 0 else [None]
            if world > 1:
                dist.broadcast_object_list(tok, src=0)
            name = tok[0]
        h = lib.pkbh_heap_create(name.encode(), rank, world, ctypes.c_longlong(nbytes), timeout_ms)
        if h < 0:
            raise RuntimeError("pkbh_heap_create failed: " + lib.pkbh_last_error().decode())
        return cls(h, name, rank, world, nbytes, timeout_ms)

    def close(self) -> None:
        if self.handle is not None:
            nv.host_lib().pkbh_heap_close(self.handle, 1 if self.rank == 0 else 0)
            self.handle = None

    def group(self, members: list[int]) -> HostGroup:
        key = tuple(members)
        if key not in self._groups:
            self._groups[key] = HostGroup(self, list(members), self._next_channel)
            self._next_channel += 1
        return self._groups[key]

    def _raw_alloc(self, nbytes: int) -> int:
        off = (self._top + 63) // 64 * 64
        if off + nbytes > self.nbytes:
            raise MemoryError("host heap exhausted")
        self._top = off + nbytes
        return off

    def alloc_bytes(self, nbytes: int) -> int:
        from . import guards

        if not guards.enabled():
            return self._raw_alloc(nbytes)
        if getattr(self, "_guards", None) is None:
            base = nv.host_lib().pkbh_heap_local(self.handle)

            def fill(off, n):
                ctypes.memset(base + off, guards.PATTERN, n)

            def first_bad(off, n):
                raw = ctypes.string_at(base + off, n)
                if raw == bytes([guards.PATTERN]) * n:
                    return -1
                return next(i for i, b in enumerate(raw) if b != guards.PATTERN)

            self._guards = guards.GuardBook(fill, first_bad, align=64)
        return self._guards.allocate(self._raw_alloc, nbytes)

    def check_guards(self, raise_on_violation: bool = True) -> list[dict]:
        """Allocations of this rank's heap whose guard bands were overwritten (empty without ``PKB_HEAP_GUARD=1``)."""
        from . import guards

        book = getattr(self, "_guards", None)
        bad = book.check() if book is not None else []
        if bad and raise_on_violation:
            raise guards.GuardViolation(bad)
        return bad

    # fault injection (host side only)
    def drop_signals(self, count: int) -> None:
        nv.host_lib().pkbh_debug_drop_signals(self.handle, count)

    def delay_ms(self, ms: int) -> None:
        nv.host_lib().pkbh_debug_delay_ms(self.handle, ms)

    # ------------------------------------------------------------------ collectives
    def _raise(self, rc: int, what: str) -> None:
        if rc == 0:
            return
        lib = nv.host_lib()
        msg = lib.pkbh_last_error().decode()
        if rc == 2:
            raise HostCollectiveTimeout(f"{what}: {msg}", lib.pkbh_last_missing_peer(self.handle))
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")

    def _scratch(self, nbytes: int) -> int:
        key = "_scratch_buf"
        cur = getattr(self, key, None)
        if cur is None or cur[1] < nbytes:
            cap = 1 << max(12, (max(nbytes, 1) - 1).bit_length())
            cur = (self.alloc_bytes(cap), cap)
            setattr(self, key, cur)
        return cur[0]

    def barrier(self, group: HostGroup | None = None, timeout_ms: int | None = None) -> None:
        g = group or self.world_group
        rc = nv.host_lib().pkbh_barrier(self.handle, g.c_members, g.size, g.channel, timeout_ms or self.timeout_ms)
        self._raise(rc, "barrier")

    def _reduce(self, x, g, op, in_base, n, out, active, scale, timeout_ms):
        x = x.contiguous()
        off = self._scratch(x.numel() * x.element_size())
        rc = nv.host_lib().pkbh_reduce(self.handle, g.c_members, g.size, g.channel, _DT[x.dtype], _OP[op],
                                       ctypes.c_void_p(x.data_ptr()), ctypes.c_longlong(x.numel()),
                                       ctypes.c_ulonglong(off), ctypes.c_longlong(in_base), ctypes.c_longlong(n),
                                       ctypes.c_void_p(out.data_ptr()), 1 if active else 0, ctypes.c_double(scale),
                                       timeout_ms or self.timeout_ms)
        self._raise(rc, "reduce")
        return out

    def all_reduce(self, x: torch.Tensor, group: HostGroup | None = None, op: str = "sum", scale: float = 1.0,
                   timeout_ms: int | None = None) -> torch.Tensor:
        g = group or self.world_group
        return self._reduce(x, g, op, 0, x.numel(), torch.empty_like(x), True, scale, timeout_ms)

    def reduce_scatter(self, x: torch.Tensor, group: HostGroup | None = None, op: str = "sum",
                       timeout_ms: int | None = None) -> torch.Tensor:
        g = group or self.world_group
        n = x.numel() // g.size
        out = torch.empty((x.shape[0] // g.size, *x.shape[1:]), dtype=x.dtype)
        return self._reduce(x, g, op, n * g.rank_in_group, n, out, True, 1.0, timeout_ms)

    def _gather(self, x, g, mask, member_stride, seg_bytes, out, active, timeout_ms):
        x = x.contiguous()
        off = self._scratch(x.numel() * x.element_size())
        rc = nv.host_lib().pkbh_gather(self.handle, g.c_members, g.size, g.rank_in_group, g.channel,
                                       ctypes.c_void_p(x.data_ptr()), ctypes.c_longlong(x.numel() * x.element_size()),
                                       ctypes.c_ulonglong(off), ctypes.c_uint(mask), ctypes.c_longlong(0),
                                       ctypes.c_longlong(member_stride), ctypes.c_longlong(seg_bytes),
                                       ctypes.c_void_p(out.data_ptr()), ctypes.c_longlong(seg_bytes),
                                       1 if active else 0, timeout_ms or self.timeout_ms)
        self._raise(rc, "gather")
        return out

    def all_gather(self, x: torch.Tensor, group: HostGroup | None = None, timeout_ms: int | None = None) -> torch.Tensor:
        g = group or self.world_group
        out = torch.empty((g.size, *x.shape), dtype=x.dtype)
        return self._gather(x, g, (1 << g.size) - 1, 0, x.numel() * x.element_size(), out, True, timeout_ms)

    def all_to_all(self, x: torch.Tensor, group: HostGroup | None = None, timeout_ms: int | None = None) -> torch.Tensor:
        g = group or self.world_group
        chunk = x[0].numel() * x.element_size()
        return self._gather(x, g, (1 << g.size) - 1, chunk, chunk, torch.empty_like(x), True, timeout_ms)

    def broadcast(self, x: torch.Tensor, src: int = 0, group: HostGroup | None = None,
                  timeout_ms: int | None = None) -> torch.Tensor:
        g = group or self.world_group
        return self._gather(x, g, 1 << src, 0, x.numel() * x.element_size(), torch.empty_like(x), True, timeout_ms)

    def local_view(self, offset: int, nbytes: int) -> np.ndarray:
        base = nv.host_lib().pkbh_heap_local(self.handle)
        return np.ctypeslib.as_array((ctypes.c_uint8 * nbytes).from_address(base + offset))
