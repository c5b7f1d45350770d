"""Per-rank distributed context: one process per GPU, ``torch.distributed`` for the plumbing.

``init_context()`` reads the torchrun environment (``RANK``, ``LOCAL_RANK``, ``WORLD_SIZE``,
``MASTER_ADDR``, ``MASTER_PORT``), binds the process to its GPU and creates the default process
group - NCCL on GPUs (with ``device_id`` so peer access is set up eagerly), gloo on CPU-only
machines. Without a torchrun environment it falls back to a single-rank group so the same code runs
as a plain script. Replaces the four identical per-backend initialisers of the reference
(reference: utils/init_and_finalize_backends.py:13-100).
"""
from __future__ import annotations

import datetime
import os
import socket
from dataclasses import dataclass, field

import torch
import torch.distributed as dist


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@dataclass
class DistContext:
    rank: int
    world: int
    local_rank: int
    device: torch.device
    backend: str
    owns_group: bool = True
    _heap: object = field(default=None, repr=False)

    @property
    def is_cuda(self) -> bool:
        return self.device.type == "cuda"

    def barrier(self) -> None:
        if self.world > 1:
            if self.is_cuda:
                dist.barrier(device_ids=[self.device.index])
            else:
                dist.barrier()

    def heap(self):
        """The symmetric heap of this job (created on first use; collective over all ranks)."""
        if self._heap is None:
            if self.is_cuda:
                from .symm_heap import SymmetricHeap

                self._heap = SymmetricHeap.create(self)
            else:
                from .host_heap import HostHeap

                self._heap = HostHeap.create(self)
        return self._heap

    def finalize(self) -> None:
        if self._heap is not None:
            self._heap.close()
            self._heap = None
        if self.owns_group and dist.is_initialized():
            try:
                if self.is_cuda:
                    torch.cuda.synchronize()
                dist.destroy_process_group()
            except Exception:  # teardown must never mask the real failure
                pass


def init_context(backend: str | None = None, timeout_s: float = 600.0) -> DistContext:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available() and backend != "gloo"
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    if use_cuda:
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
    else:
        device = torch.device("cpu")
    owns = False
    if not dist.is_initialized():
        if "MASTER_ADDR" not in os.environ:
            os.environ["MASTER_ADDR"] = "127.0.0.1"
        if "MASTER_PORT" not in os.environ:
            os.environ["MASTER_PORT"] = str(_free_port())
        kwargs = dict(backend=backend, init_method="env://", rank=rank, world_size=world,
                      timeout=datetime.timedelta(seconds=timeout_s))
        if use_cuda:
            kwargs["device_id"] = device
        dist.init_process_group(**kwargs)
        owns = True
    return DistContext(rank=rank, world=world, local_rank=local_rank, device=device, backend=backend,
                       owns_group=owns)
