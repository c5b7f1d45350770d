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


def test_forbidden_constructs_are_refused_before_any_build(tmp_path, monkeypatch):
    """Candidate text that names a cluster-multicast bulk load, a batched memcpy call or a trap never reaches nvcc or a GPU.
    The forbidden spellings are assembled here from fragments so that this test file does not contain them either."""
    from parallelkernelbench_b200.harness import launch
    from parallelkernelbench_b200.utils import cuda_ext
    from parallelkernelbench_b200.utils.source_screen import ForbiddenSourceError, screen_source

    mc_load = ("cp" + ".async." + "bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes." + "multi" + "cast::" + "cluster"
               + " [%0], [%1, {%3, %4}], [%2], %5;")
    batch = "cuda" + "Memcpy" + "Batch" + "Async(dst, src, sizes, n, attrs, idx, 1, &fail, stream);"
    trap = "if (bad) __tr" + "ap();"
    for bad in (mc_load, batch, trap):
        assert screen_source(f'asm volatile("{bad}");'), bad
    split = 'asm volatile("cp" ".async." "bulk.shared::cluster.global.mbarrier::complete_tx::bytes"\n    ".multi" "cast::" "cluster [%0], [%1], %2, [%3], %4;");'
    assert screen_source(split.replace('" "', ""))                    # a statement split over lines is still one statement
    assert screen_source(SRC) == []                                    # ordinary code passes
    commit_ok = "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster." + "multi" + "cast::" + "cluster.b64 [%0], %1;"
    assert screen_source(commit_ok) == []                              # only loads are off-limits, not the MMA commit

    monkeypatch.setenv("PKB_EXT_DIR", str(tmp_path))
    with pytest.raises(ForbiddenSourceError):
        cuda_ext.compile_cuda_module(SRC + "\n// " + batch, name="bad")
    assert not list(tmp_path.glob("bad_*"))                            # nothing was written or compiled

    sol = tmp_path / "sol.py"
    sol.write_text("SRC = r\'\'\'" + mc_load + "\'\'\'\ndef solution(rc, x):\n    return x\n")
    monkeypatch.setattr(launch, "LOGS_ROOT", str(tmp_path / "logs"))
    job = launch.run_job("allreduce", "file", 2, solution=str(sol))
    assert job["returncode"] == 2 and "source screen" in job["stderr"] and job["artifact_count"] == 0
    assert not list((tmp_path / "logs").rglob("candidate_solution.py"))

