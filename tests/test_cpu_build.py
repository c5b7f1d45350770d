"""The build entry point works on a machine without a GPU and leaves loadable libraries in-tree."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_build_entry_point_and_symbols():
    import __graft_entry__ as g

    g.build()
    from parallelkernelbench_b200 import _native as nv

    lib = nv.cuda_lib()
    for sym in ("pkb_gemm_bf16", "pkb_gemm_bf16_pair", "pkb_rmsnorm_bf16", "pkb_coll_reduce", "pkb_coll_gather",
                "pkb_coll_allreduce_nvls", "pkb_tp_ag_gemm", "pkb_tp_gemm_rs_rmsnorm", "pkb_heap_create"):
        assert hasattr(lib, sym), sym
    assert nv.host_lib().pkbh_ctrl_bytes() == 1 << 20


def test_missing_library_raises_loudly(monkeypatch, tmp_path):
    from parallelkernelbench_b200 import _native as nv

    monkeypatch.setattr(nv, "_LIB_DIR", tmp_path)
    monkeypatch.setattr(nv, "_cuda", None)
    try:
        nv.cuda_lib()
    except nv.NativeLibraryError as e:
        assert "Build it" in str(e)
    else:
        raise AssertionError("a missing kernel library must not be silently ignored")


def test_jitter_variant_builds_and_is_selected_by_env(monkeypatch):
    """The timing-perturbation build (-DPKB_JITTER) is a second library with the same entry points; PKB_JITTER=1 loads it."""
    import ctypes

    from parallelkernelbench_b200 import _native as nv
    from parallelkernelbench_b200 import build

    assert set(build.VARIANTS) == {"jitter", "bounds"}
    path = build.build_variant("jitter")
    assert path.exists() and path.name == "libpkb200_cuda_jitter.so"
    lib = ctypes.CDLL(str(path))
    for sym in ("pkb_coll_reduce", "pkb_coll_allreduce_ll", "pkb_tp_ag_gemm", "pkb_moe_dispatch", "pkb_flash_attn_fwd"):
        assert hasattr(lib, sym), sym
    seen = []
    monkeypatch.setenv("PKB_JITTER", "1")
    monkeypatch.setattr(nv, "_cuda", None)
    monkeypatch.setattr(nv, "_load", lambda p, what: seen.append(p.name) or lib)
    nv.cuda_lib()
    assert seen == ["libpkb200_cuda_jitter.so"]
    monkeypatch.delenv("PKB_JITTER")
    monkeypatch.setenv("PKB_DEBUG_BOUNDS", "1")
    monkeypatch.setattr(nv, "_cuda", None)
    nv.cuda_lib()
    assert seen[-1] == "libpkb200_cuda_bounds.so"
    monkeypatch.setattr(nv, "_cuda", None)


def test_example_script_compiles_and_declines_politely_without_a_gpu():
    import subprocess

    path = os.path.join(ROOT, "examples", "tp_mlp_block.py")
    compile(open(path).read(), path, "exec")
    import torch

    if not torch.cuda.is_available():
        r = subprocess.run([sys.executable, path], capture_output=True, text=True, timeout=300)
        assert r.returncode == 2 and "needs CUDA" in r.stderr
