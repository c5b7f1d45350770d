"""Thin Python wrappers over the hand-written sm_100a kernels (one module per kernel family)."""
from .gemm import gemm_bf16, gemm_bf16_kn, gemm_bf16_tn, linear_bf16  # noqa: F401
from .norm import rmsnorm, sum_rmsnorm  # noqa: F401
from .elementwise import (ce_backward, rmsnorm_bwd, swiglu_bwd, swiglu_fwd,  # noqa: F401
                          adam_step, ce_finalize, ce_local_stats, fp8_dequantize_1x128, fp8_quantize_1x128,  # noqa: F401
                          ln_bwd_colreduce, rope, tp_rmsnorm, vocab_parallel_cross_entropy)
