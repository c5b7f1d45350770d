"""Worked examples shown in the prompt: for an op, the reference is printed next to a solution file that passes
``launch eval --solution``. They play the role of the reference's in-context pairs (reference:
kernelgen/solutions_ex_allreduce.py:1-33 next to kernelgen/solutions_new_allreduce_parallelkittens.py:180-210, and
kernelgen/solutions_ex_alltoall.py:1-56 next to kernelgen/solutions_new_alltoall_parallelkittens.py), written against
this package's own interface instead of an external kernel library."""
from __future__ import annotations

from pathlib import Path

_DIR = Path(__file__).resolve().parent

# op name -> example file (each defines solution(rc, *inputs) for that op)
EXAMPLES = {
    "allreduce": "allreduce_symmetric_heap.py",
    "alltoall": "alltoall_symmetric_heap.py",
    "gemm_allreduce": "gemm_allreduce_two_kernels.py",
    "tp_rmsnorm": "tp_rmsnorm_own_kernel.py",
}


def example_path(op: str) -> Path:
    return _DIR / EXAMPLES[op]


def example_source(op: str) -> str:
    return example_path(op).read_text()
