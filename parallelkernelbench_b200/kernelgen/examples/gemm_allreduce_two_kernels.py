"""Example solution for the op `gemm_allreduce` (row-parallel linear layer): the tcgen05 GEMM of this package, then the
symmetric-heap all-reduce - two launches, no NCCL, no cuBLAS. The weight arrives as [K, N]; the kernel wants one output
feature per row ([N, K]), so the re-laid-out copy is cached across calls (weights do not change between them)."""
import torch

_cache = {}


def solution(rc, a, b):
    if not a.is_cuda or a.dtype != torch.bfloat16 or a.shape[1] % 8 != 0:
        return rc.comm.all_reduce((a.float() @ b.float()).to(a.dtype))       # CPU ranks / odd shapes: plain PyTorch product
    from parallelkernelbench_b200.ops import gemm_bf16

    key = (b.data_ptr(), tuple(b.shape))
    w = _cache.get(key)
    if w is None:
        w = _cache[key] = b.t().contiguous()
    return rc.comm.all_reduce(gemm_bf16(a.contiguous(), w))
