"""Two-level device meshes in Megatron rank order.

``Mesh2D(world, inner, ...)`` splits ``world`` ranks into ``outer x inner`` with the *inner*
dimension varying fastest (rank = outer_idx * inner + inner_idx). Every rank must construct the
mesh with the same arguments because ``dist.new_group`` is collective. This one class covers the
pairs the workloads need: TP x CP, CP x PP, CP x DP, TP x FSDP, EP x EP-FSDP, polar x azimuth
(reference builders: utils/input_output_tensors.py:110-263).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch.distributed as dist


def factor_two_level(world: int, prefer_inner: int = 2) -> tuple[int, int]:
    """(outer, inner) with inner = the largest divisor of ``world`` that is <= prefer_inner."""
    inner = 1
    for d in range(1, prefer_inner + 1):
        if world % d == 0:
            inner = d
    return world // inner, inner


def inner_groups(world: int, inner: int) -> list[list[int]]:
    return [list(range(o * inner, (o + 1) * inner)) for o in range(world // inner)]


def outer_groups(world: int, inner: int) -> list[list[int]]:
    return [list(range(i, world, inner)) for i in range(inner)]


@dataclass
class Mesh2D:
    world: int
    inner: int
    rank: int
    inner_name: str = "inner"
    outer_name: str = "outer"
    inner_group: object = None
    outer_group: object = None

    @property
    def outer(self) -> int:
        return self.world // self.inner

    @property
    def inner_rank(self) -> int:
        return self.rank % self.inner

    @property
    def outer_rank(self) -> int:
        return self.rank // self.inner

    @property
    def inner_ranks(self) -> list[int]:
        return inner_groups(self.world, self.inner)[self.outer_rank]

    @property
    def outer_ranks(self) -> list[int]:
        return outer_groups(self.world, self.inner)[self.inner_rank]

    @classmethod
    def build(cls, world: int, inner: int, rank: int, inner_name: str = "inner", outer_name: str = "outer",
              create_groups: bool = True) -> "Mesh2D":
        if world % inner != 0:
            raise ValueError(f"inner size {inner} does not divide world {world}")
        m = cls(world=world, inner=inner, rank=rank, inner_name=inner_name, outer_name=outer_name)
        if create_groups and dist.is_initialized() and world > 1:
            for ranks in inner_groups(world, inner):
                g = dist.new_group(ranks)
                if rank in ranks:
                    m.inner_group = g
            for ranks in outer_groups(world, inner):
                g = dist.new_group(ranks)
                if rank in ranks:
                    m.outer_group = g
        return m
