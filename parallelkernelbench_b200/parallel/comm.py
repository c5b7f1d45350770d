"""One collective interface for op implementations, backed by our own transports.

``Comm`` is what the "ours" side of every workload calls instead of ``torch.distributed``: on GPUs it
dispatches to the symmetric-heap kernels (:mod:`parallelkernelbench_b200.ops.collectives`), on a
CPU-only machine to the shared-memory twin (:mod:`parallelkernelbench_b200.parallel.host_heap`) that
runs the same protocol. Groups are given as a torch process group, a list of global ranks, or
``None`` for the whole job. Layout conventions follow ``torch.distributed``'s tensor collectives:
``all_gather`` returns ``[W, *shape]``, ``reduce_scatter`` and ``all_to_all`` split dimension 0.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class Comm:
    def __init__(self, ctx):
        self.ctx = ctx
        self.heap = ctx.heap()
        self.is_cuda = ctx.is_cuda
        if self.is_cuda:
            from ..ops import collectives as C

            self._C = C

    # ------------------------------------------------------------------ groups
    def group(self, g=None):
        if g is None:
            return self.heap.world_group
        if isinstance(g, (list, tuple)):
            return self.heap.group(list(g))
        if hasattr(g, "members") and hasattr(g, "channel"):
            return g
        if g is dist.group.WORLD:
            return self.heap.world_group
        return self.heap.group(dist.get_process_group_ranks(g))

    def size(self, g=None) -> int:
        return self.group(g).size

    def rank(self, g=None) -> int:
        return self.group(g).rank_in_group

    # ------------------------------------------------------------------ collectives
    def barrier(self, group=None) -> None:
        g = self.group(group)
        if self.is_cuda:
            self._C.barrier(g)
        else:
            self.heap.barrier(g)

    def all_reduce(self, x: torch.Tensor, op: str = "sum", group=None, scale: float = 1.0, algo: str = "auto") -> torch.Tensor:
        g = self.group(group)
        if self.is_cuda:
            return self._C.all_reduce(x, g, op=op, scale=scale, algo=algo).view(x.shape)
        return self.heap.all_reduce(x, g, op=op, scale=scale).view(x.shape)

    def all_gather(self, x: torch.Tensor, group=None) -> torch.Tensor:
        g = self.group(group)
        if self.is_cuda:
            return self._C.all_gather(x, g)
        return self.heap.all_gather(x, g)

    def all_gather_cat(self, x: torch.Tensor, dim: int = 0, group=None) -> torch.Tensor:
        """Concatenate the members' tensors along ``dim`` (``all_gather`` + a local permutation)."""
        out = self.all_gather(x, group)
        if dim == 0:
            return out.reshape(-1, *x.shape[1:])
        return torch.cat(list(out.unbind(0)), dim=dim)

    def reduce_scatter(self, x: torch.Tensor, op: str = "sum", group=None, scale: float = 1.0) -> torch.Tensor:
        g = self.group(group)
        if self.is_cuda:
            return self._C.reduce_scatter(x, g, op=op, scale=scale)
        y = self.heap.reduce_scatter(x, g, op=op)
        return y * scale if scale != 1.0 else y

    def all_to_all(self, x: torch.Tensor, group=None) -> torch.Tensor:
        g = self.group(group)
        if self.is_cuda:
            return self._C.all_to_all(x, g)
        return self.heap.all_to_all(x, g)

    def all_to_all_permute(self, x: torch.Tensor, scatter_dim: int, gather_dim: int, group=None) -> torch.Tensor:
        """Split along ``scatter_dim``, exchange, concatenate along ``gather_dim`` (sequence <-> head exchange)."""
        g = self.group(group)
        W = self.size(group)
        if W == 1:
            return x.contiguous()
        if self.is_cuda:
            return self._C.all_to_all_permute(x, g, scatter_dim, gather_dim)
        parts = torch.stack([c.contiguous() for c in x.chunk(W, dim=scatter_dim)])
        got = self.heap.all_to_all(parts, g)
        return torch.cat(list(got.unbind(0)), dim=gather_dim).contiguous()

    def row_gather(self, shard: torch.Tensor, ids: torch.Tensor, group=None) -> torch.Tensor:
        """Lookup in a table sharded by rows over the group."""
        g = self.group(group)
        if self.size(group) == 1:
            return shard[ids]
        if self.is_cuda:
            return self._C.row_gather(shard, ids, g)
        W = self.size(group)
        table = self.heap.all_gather(shard.contiguous(), g).reshape(W * shard.shape[0], *shard.shape[1:])
        return table[ids]

    def broadcast(self, x: torch.Tensor, src: int = 0, group=None) -> torch.Tensor:
        g = self.group(group)
        if self.is_cuda:
            return self._C.broadcast(x, g, src=src)
        return self.heap.broadcast(x, src=src, group=g)

    def reduce(self, x: torch.Tensor, dst: int = 0, op: str = "sum", group=None) -> torch.Tensor:
        g = self.group(group)
        if self.is_cuda:
            return self._C.reduce(x, g, dst=dst, op=op)
        y = self.heap.all_reduce(x, g, op=op)
        return y if g.rank_in_group == dst else x

    def scatter(self, x: torch.Tensor, src: int = 0, group=None) -> torch.Tensor:
        g = self.group(group)
        if self.is_cuda:
            return self._C.scatter(x, g, src=src)
        full = self.heap.broadcast(x, src=src, group=g)
        return full[g.rank_in_group].clone()

    def gather(self, x: torch.Tensor, dst: int = 0, group=None) -> torch.Tensor:
        g = self.group(group)
        if self.is_cuda:
            return self._C.gather(x, g, dst=dst)
        full = self.heap.all_gather(x, g)
        return full if g.rank_in_group == dst else x

    def all_to_all_v(self, x: torch.Tensor, send_counts: torch.Tensor, out_capacity_rows: int, group=None,
                     max_send_rows: int | None = None):
        """Rows of ``x`` grouped by destination; returns ``(out, recv_counts, total)`` with device-side counts.
        ``out_capacity_rows`` and ``max_send_rows`` (an upper bound of ``x.shape[0]`` over all ranks; default: the output
        capacity) must be the same on every rank."""
        g = self.group(group)
        if self.is_cuda:
            return self._C.all_to_all_v(x, send_counts.to(torch.int64), g, out_capacity_rows, max_send_rows=max_send_rows)
        # CPU twin: exchange the count matrix, then one padded all-to-all
        W = g.size
        counts = self.heap.all_gather(send_counts.to(torch.int64), g)          # [W, W]
        recv = counts[:, g.rank_in_group].contiguous()
        cap = max(int(counts.max().item()), 1)
        padded = x.new_zeros((W, cap, *x.shape[1:]))
        offs = torch.cumsum(send_counts, 0) - send_counts
        for d in range(W):
            n = int(send_counts[d])
            padded[d, :n] = x[int(offs[d]):int(offs[d]) + n]
        got = self.heap.all_to_all(padded, g)
        out = x.new_zeros((out_capacity_rows, *x.shape[1:]))
        pos = 0
        for s in range(W):
            n = int(recv[s])
            take = max(0, min(n, out_capacity_rows - pos))
            out[pos:pos + take] = got[s, :take]
            pos += n
        return out, recv, torch.tensor([pos], dtype=torch.int64)
