"""A candidate's own CUDA source is compiled for sm_100a (nvcc cross-compiles without a GPU), cached, and loadable; the
package's device headers are on its include path."""
import ctypes

import pytest

SRC = r'''
#include "pkb/ptx.cuh"
#include "pkb/symm.cuh"

__global__ void scale_kernel(float* x, float a, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] *= a;
}

extern "C" int candidate_answer() { return 42 + (int)sizeof(pkb::SymmCtx) * 0; }

extern "C" int candidate_scale(float* x, float a, long long n, void* stream) {
  scale_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, a, n);
  return (int)cudaGetLastError();
}
'''


def test_compile_cache_and_load(tmp_path, monkeypatch):
    from parallelkernelbench_b200.utils import cuda_ext

    monkeypatch.setenv("PKB_EXT_DIR", str(tmp_path))
    monkeypatch.setattr(cuda_ext, "_loaded", {})
    lib = cuda_ext.compile_cuda_module(SRC, name="cand")
    assert lib.candidate_answer() == 42 and hasattr(lib, "candidate_scale")
    built = list(tmp_path.glob("cand_*/cand.so"))
    assert len(built) == 1
    stamp = built[0].stat().st_mtime_ns
    assert cuda_ext.compile_cuda_module(SRC, name="cand") is lib                      # in-process cache
    monkeypatch.setattr(cuda_ext, "_loaded", {})
    lib2 = cuda_ext.compile_cuda_module(SRC, name="cand")                              # on-disk cache: no rebuild
    assert isinstance(lib2, ctypes.CDLL) and built[0].stat().st_mtime_ns == stamp
    with pytest.raises(RuntimeError, match="nvcc failed"):
        cuda_ext.compile_cuda_module("this is not CUDA", name="broken")
