"""Thin Python wrappers over the hand-written sm_100a kernels (one module per kernel family)."""
from .gemm import gemm_bf16, linear_bf16  # noqa: F401
from .norm import rmsnorm, sum_rmsnorm  # noqa: F401
