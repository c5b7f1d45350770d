"""Python side of the symmetric heap (native part: csrc/runtime/symm_heap.cu).

``SymmetricHeap.create(ctx)`` is collective over all ranks of the job. It allocates this rank's
slab with CUDA virtual memory management, passes the slab's file descriptor to every peer over
abstract unix sockets (``SCM_RIGHTS``), maps all slabs at ``base + rank * stride`` and - when the
GPUs support it and it is asked for - binds the slabs to one NVSwitch multicast object so kernels
can use ``multimem`` instructions.

This is our own replacement for the two external runtimes the reference wraps for kernel authors:
torch's ``_symmetric_memory`` (reference: kernelgen/solution_new_add_cuda.py:70-106) and
ThunderKittens' ``TKParallelTensor`` with its cache keyed by shape/dtype
(reference: utils/parallelkittens_runtime.py:14-72).

Allocation is a bump allocator; every rank must allocate in the same order so that offsets agree.
``named(key, ...)`` caches buffers by key, so steady-state calls reuse their staging space.
"""
from __future__ import annotations

import ctypes
import os
import socket
import struct
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import _native as nv
from ..utils import env as _env

CTRL_BYTES = 1 << 20        # control space at the start of every slab (barrier flags, epochs)
MAX_WORLD = 16
NUM_CHANNELS = 32
_ALIGN = 1024


class SymmCtxStruct(ctypes.Structure):
    _fields_ = [("base", ctypes.c_uint64), ("stride", ctypes.c_uint64), ("mc_base", ctypes.c_uint64),
                ("rank", ctypes.c_int32), ("world", ctypes.c_int32), ("gsize", ctypes.c_int32),
                ("grank", ctypes.c_int32), ("members", ctypes.c_int32 * 16), ("channel", ctypes.c_int32),
                ("_pad", ctypes.c_int32), ("budget_ns", ctypes.c_uint64)]


class _RawCudaBuffer:
    """Exposes a raw device range through ``__cuda_array_interface__`` so torch can wrap it."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        self._owner = owner


@dataclass
class SymmTensor:
    """A tensor that exists at the same heap offset on every rank."""
    heap: "SymmetricHeap"
    offset: int
    local: torch.Tensor

    @property
    def nbytes(self) -> int:
        return self.local.numel() * self.local.element_size()

    def peer_ptr(self, rank: int) -> int:
        return self.heap.base + rank * self.heap.stride + self.offset

    def peer(self, rank: int) -> torch.Tensor:
        """View of rank ``rank``'s copy (readable and writable over NVLink)."""
        return self.heap._view(self.peer_ptr(rank), self.local.shape, self.local.dtype)

    def mc_ptr(self) -> int:
        return self.heap.mc_base + self.offset if self.heap.mc_base else 0


class SymmGroup:
    """A set of ranks sharing one control channel of the heap (one per process group)."""

    def __init__(self, heap: "SymmetricHeap", members: list[int], channel: int):
        self.heap = heap
        self.members = list(members)
        self.channel = channel
        self.size = len(members)
        self.rank_in_group = members.index(heap.rank) if heap.rank in members else -1
        s = SymmCtxStruct()
        s.base, s.stride, s.mc_base = heap.base, heap.stride, heap.mc_base
        s.rank, s.world = heap.rank, heap.world
        s.gsize, s.grank = self.size, max(self.rank_in_group, 0)
        for i, m in enumerate(members):
            s.members[i] = m
        s.channel = channel
        s.budget_ns = _env.wait_budget_ns()
        self.struct = s

    @property
    def ref(self):
        return ctypes.byref(self.struct)

    @property
    def is_whole_heap(self) -> bool:
        return self.size == self.heap.world

    def set_wait_budget_ms(self, ms: float) -> None:
        self.struct.budget_ns = int(ms * 1e6)


class SymmetricHeap:
    def __init__(self, ctx, handle: int, nbytes: int, base: int, stride: int, mc_base: int):
        self.ctx = ctx
        self.rank, self.world = ctx.rank, ctx.world
        self.handle = handle
        self.nbytes = nbytes
        self.base, self.stride, self.mc_base = base, stride, mc_base
        self._top = CTRL_BYTES
        self._named: dict = {}
        self._next_channel = 0
        self._groups: dict = {}
        self.world_group = self.group(list(range(self.world)))

    # ------------------------------------------------------------------ creation / teardown
    @classmethod
    def create(cls, ctx, nbytes: int | None = None, multicast: bool | None = None) -> "SymmetricHeap":
        lib = nv.cuda_lib()
        lib.pkb_heap_round_size.restype = ctypes.c_longlong
        for f in (lib.pkb_heap_base, lib.pkb_heap_stride, lib.pkb_heap_mc_base):
            f.restype = ctypes.c_ulonglong
        if nbytes is None:
            nbytes = int(float(os.environ.get("PKB_HEAP_GIB", "1")) * (1 << 30))
        if multicast is None:
            multicast = os.environ.get("PKB_NVLS", "1") not in ("0", "")
        multicast = bool(multicast) and ctx.world > 1 and lib.pkb_heap_multicast_supported() == 1
        # every rank must agree on multicast availability
        if ctx.world > 1:
            flag = torch.tensor([1 if multicast else 0], device=ctx.device, dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            multicast = bool(flag.item())
        size = lib.pkb_heap_round_size(ctypes.c_longlong(nbytes), ctx.world, 1 if multicast else 0)
        if size <= 0:
            raise RuntimeError("pkb_heap_round_size failed: " + (lib.pkb_last_error() or b"").decode())
        fd = ctypes.c_int(-1)
        handle = lib.pkb_heap_create(ctypes.c_longlong(size), ctx.rank, ctx.world, ctypes.byref(fd))
        if handle < 0:
            raise RuntimeError("pkb_heap_create failed: " + (lib.pkb_last_error() or b"").decode())
        if ctx.world > 1:
            fds = _exchange_fds(ctx, fd.value, tag="slab")
            for peer, pfd in fds.items():
                nv.check(lib.pkb_heap_import_peer(handle, peer, pfd), "pkb_heap_import_peer")
                os.close(pfd)
            if multicast:
                mfd = ctypes.c_int(-1)
                if ctx.rank == 0:
                    nv.check(lib.pkb_heap_mc_create(handle, ctypes.byref(mfd)), "pkb_heap_mc_create")
                got = _broadcast_fd(ctx, mfd.value, tag="mc")
                if ctx.rank != 0:
                    nv.check(lib.pkb_heap_mc_import(handle, got), "pkb_heap_mc_import")
                    os.close(got)
                nv.check(lib.pkb_heap_mc_add_device(handle), "pkb_heap_mc_add_device")
                ctx.barrier()
                nv.check(lib.pkb_heap_mc_bind(handle), "pkb_heap_mc_bind")
            ctx.barrier()
        heap = cls(ctx, handle, int(size), int(lib.pkb_heap_base(handle)), int(lib.pkb_heap_stride(handle)),
                   int(lib.pkb_heap_mc_base(handle)))
        return heap

    def close(self) -> None:
        if self.handle is None:
            return
        torch.cuda.synchronize()
        if self.world > 1 and dist.is_initialized():
            try:
                self.ctx.barrier()
            except Exception:
                pass
        nv.cuda_lib().pkb_heap_destroy(self.handle)
        self.handle = None

    # ------------------------------------------------------------------ groups
    def group(self, members: list[int]) -> SymmGroup:
        """Control channel for a rank subset. Collective: all ranks call it in the same order."""
        key = tuple(members)
        if key not in self._groups:
            if self._next_channel >= NUM_CHANNELS:
                raise RuntimeError("out of symmetric-heap control channels")
            self._groups[key] = SymmGroup(self, list(members), self._next_channel)
            self._next_channel += 1
        return self._groups[key]

    def group_for(self, pg) -> SymmGroup:
        """The :class:`SymmGroup` matching a torch process group (``None`` = the whole job)."""
        if pg is None or pg is dist.group.WORLD:
            return self.world_group
        return self.group(dist.get_process_group_ranks(pg))

    # ------------------------------------------------------------------ allocation
    def _view(self, ptr: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = max(n * torch.empty((), dtype=dtype).element_size(), 1)
        raw = torch.as_tensor(_RawCudaBuffer(ptr, nbytes, self), device=self.ctx.device)
        return raw.view(dtype)[:n].view(*shape) if n > 0 else torch.empty(shape, dtype=dtype, device=self.ctx.device)

    def _raw_alloc(self, nbytes: int) -> int:
        off = (self._top + _ALIGN - 1) // _ALIGN * _ALIGN
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {nbytes} bytes at {off}, heap has {self.nbytes} "
                              f"(set PKB_HEAP_GIB)")
        self._top = off + nbytes
        return off

    def alloc_bytes(self, nbytes: int) -> int:
        from . import guards

        if not guards.enabled():
            return self._raw_alloc(nbytes)
        if getattr(self, "_guards", None) is None:
            local = self.base + self.rank * self.stride

            def fill(off, n):
                self._view(local + off, (n,), torch.uint8).fill_(guards.PATTERN)

            def first_bad(off, n):
                bad = (self._view(local + off, (n,), torch.uint8) != guards.PATTERN).nonzero()
                return int(bad[0]) if bad.numel() else -1

            self._guards = guards.GuardBook(fill, first_bad, align=_ALIGN)
        return self._guards.allocate(self._raw_alloc, nbytes)

    def check_guards(self, raise_on_violation: bool = True) -> list[dict]:
        """Allocations of this rank's heap whose guard bands were overwritten (empty without ``PKB_HEAP_GUARD=1``).
        Synchronises the device."""
        from . import guards

        book = getattr(self, "_guards", None)
        if book is None:
            return []
        torch.cuda.synchronize()
        bad = book.check()
        if bad and raise_on_violation:
            raise guards.GuardViolation(bad)
        return bad

    def empty(self, shape, dtype=torch.bfloat16) -> SymmTensor:
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)))
        n = 1
        for s in shape:
            n *= s
        nbytes = (n * torch.empty((), dtype=dtype).element_size() + 15) // 16 * 16
        off = self.alloc_bytes(max(nbytes, 16))
        return SymmTensor(self, off, self._view(self.base + self.rank * self.stride + off, shape, dtype))

    def named(self, key, shape, dtype=torch.bfloat16) -> SymmTensor:
        """Cached allocation: the same key returns the same buffer (grown if a larger one is asked)."""
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)))
        cur = self._named.get(key)
        if cur is not None and cur.local.dtype == dtype and tuple(cur.local.shape) == shape:
            return cur
        need = 1
        for s in shape:
            need *= s
        need *= torch.empty((), dtype=dtype).element_size()
        if cur is not None and cur.nbytes >= need:
            t = SymmTensor(self, cur.offset, self._view(self.base + self.rank * self.stride + cur.offset, shape, dtype))
            return t
        t = self.empty(shape, dtype)
        self._named[key] = t
        return t

    def mark(self) -> int:
        return self._top

    def release(self, mark: int) -> None:
        """Free everything allocated after ``mark`` (stack discipline; drops named buffers above it)."""
        self._top = mark
        self._named = {k: v for k, v in self._named.items() if v.offset < mark}

    def contains(self, t: torch.Tensor) -> int | None:
        """Heap offset of a local tensor that lives in this rank's slab, else ``None``."""
        p = t.data_ptr()
        lo = self.base + self.rank * self.stride
        if lo <= p < lo + self.nbytes:
            return p - lo
        return None


# ---------------------------------------------------------------------------------------------
# file-descriptor passing
# ---------------------------------------------------------------------------------------------

def _job_token(ctx) -> str:
    obj = [f"{os.getpid()}_{os.environ.get('MASTER_PORT', '0')}"] if ctx.rank == 0 else [None]
    if ctx.world > 1:
        dist.broadcast_object_list(obj, src=0)
    return obj[0]


def _sock_name(token: str, tag: str, rank: int) -> bytes:
    return b"\0pkb200_" + f"{token}_{tag}_{rank}".encode()


def _exchange_fds(ctx, fd: int, tag: str) -> dict[int, int]:
    """All-to-all of one file descriptor per rank. Returns {peer: received fd}."""
    token = _job_token(ctx)
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(_sock_name(token, tag, ctx.rank))
    srv.listen(ctx.world + 4)
    srv.settimeout(120)
    ctx.barrier()
    outs = []
    for peer in range(ctx.world):
        if peer == ctx.rank:
            continue
        c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        c.settimeout(120)
        c.connect(_sock_name(token, tag, peer))
        socket.send_fds(c, [struct.pack("i", ctx.rank)], [fd])
        outs.append(c)
    got: dict[int, int] = {}
    for _ in range(ctx.world - 1):
        conn, _addr = srv.accept()
        conn.settimeout(120)
        msg, fds, _flags, _a = socket.recv_fds(conn, 16, 1)
        got[struct.unpack("i", msg[:4])[0]] = fds[0]
        conn.close()
    ctx.barrier()
    for c in outs:
        c.close()
    srv.close()
    return got


def _broadcast_fd(ctx, fd: int, tag: str) -> int:
    """Rank 0 sends one descriptor to every other rank; returns the received fd (or ``fd`` on rank 0)."""
    token = _job_token(ctx)
    if ctx.rank != 0:
        srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        srv.bind(_sock_name(token, tag, ctx.rank))
        srv.listen(4)
        srv.settimeout(120)
    ctx.barrier()
    result = fd
    if ctx.rank == 0:
        for peer in range(1, ctx.world):
            c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            c.settimeout(120)
            c.connect(_sock_name(token, tag, peer))
            socket.send_fds(c, [b"mc"], [fd])
            c.close()
    else:
        conn, _addr = srv.accept()
        conn.settimeout(120)
        _msg, fds, _flags, _a = socket.recv_fds(conn, 16, 1)
        result = fds[0]
        conn.close()
        srv.close()
    ctx.barrier()
    return result
