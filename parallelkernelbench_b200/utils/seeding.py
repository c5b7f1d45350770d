"""Deterministic seeding of op inputs.

One integer seed per (op, rank, trial), so reference and candidate see bitwise-identical inputs
and a different trial changes every tensor (same role as reference:
utils/input_output_tensors.py:57-59, with a string op name instead of a numeric problem id).
"""
from __future__ import annotations

import zlib

import torch


def seed_for(op_name: str, rank: int, trial: int = 0) -> int:
    return (zlib.crc32(op_name.encode()) % 1_000_000) * 1009 + rank * 7919 + trial * 1_000_003 + 42


def seeded_generator(op_name: str, rank: int, trial: int = 0, device: str | torch.device = "cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed_for(op_name, rank, trial))
    return g
