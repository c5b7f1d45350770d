"""tcgen05 GEMM against a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, w, bias=None, act="none", alpha=1.0):
    y = alpha * (a.float() @ w.float().t())
    if bias is not None:
        y = y + bias.float()
    if act.endswith("silu"):
        y = torch.nn.functional.silu(y)
    return y


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 64), (256, 512, 256), (1024, 1024, 1024),
                                    (100, 72, 40), (129, 257, 136), (1, 128, 64), (2048, 3584, 512)])
@pytest.mark.parametrize("block_n", [128, 256])
def test_gemm_matches_fp32_reference(M, N, K, block_n):
    from parallelkernelbench_b200.ops import gemm_bf16

    g = torch.Generator(device="cuda").manual_seed(1234 + M + N + K)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, generator=g)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16, generator=g) * 0.05
    out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm_bf16(a, w, out=out, block_n=block_n)
    ref = _ref(a, w)
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 512, 1024), (300, 520, 136), (1000, 72, 40), (2048, 3584, 512)])
def test_pair_gemm_matches_reference_and_single_cta_kernel(M, N, K):
    from parallelkernelbench_b200.ops import gemm_bf16

    g = torch.Generator(device="cuda").manual_seed(99 + M)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, generator=g)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16, generator=g) * 0.05
    out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm_bf16(a, w, out=out, mode="pair")
    torch.testing.assert_close(out.float(), _ref(a, w), atol=2e-2, rtol=2e-2)
    assert torch.equal(out, gemm_bf16(a, w, mode="single"))
    out32 = gemm_bf16(a, w, mode="pair", out_dtype=torch.float32, epilogue="silu")
    torch.testing.assert_close(out32, _ref(a, w, act="silu"), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("epilogue", ["none", "silu", "bias", "bias_silu"])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_epilogues(epilogue, out_dtype):
    from parallelkernelbench_b200.ops import gemm_bf16

    M, N, K = 384, 640, 320
    g = torch.Generator(device="cuda").manual_seed(7)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, generator=g)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16, generator=g) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16, generator=g) if "bias" in epilogue else None
    out = gemm_bf16(a, w, bias=bias, epilogue=epilogue, alpha=0.5, out_dtype=out_dtype)
    ref = _ref(a, w, bias, epilogue, 0.5)
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)


def test_gemm_is_deterministic_and_leaves_guard_bands_alone():
    from parallelkernelbench_b200.ops import gemm_bf16

    M, N, K = 300, 520, 1024
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    # output embedded in a larger buffer whose border must stay untouched
    buf = torch.full((M + 16, N + 16), 7.0, device="cuda", dtype=torch.bfloat16)
    out = buf[8:8 + M, 8:8 + N]
    gemm_bf16(a, w, out=out)
    first = out.clone()
    for _ in range(10):
        gemm_bf16(a, w, out=out)
        assert torch.equal(out, first)
    border = buf.clone()
    border[8:8 + M, 8:8 + N] = 7.0
    assert torch.all(border == 7.0)


def test_large_k_accumulation():
    from parallelkernelbench_b200.ops import gemm_bf16

    M, N, K = 256, 256, 8192
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
    out = gemm_bf16(a, w)
    torch.testing.assert_close(out.float(), _ref(a, w), atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 384, 512), (300, 200, 136), (520, 712, 328), (4096, 4096, 1024)])
def test_gemm_with_row_major_kn_weight(M, N, K):
    from parallelkernelbench_b200.ops.gemm import gemm_bf16_kn

    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16) * 0.05
    out = gemm_bf16_kn(a, b)
    torch.testing.assert_close(out.float(), a.float() @ b.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (384, 512, 1000), (4096, 1024, 4096), (264, 648, 200)])
def test_gemm_transposed_a_for_weight_gradients(M, N, K):
    from parallelkernelbench_b200.ops import gemm_bf16_tn

    a = torch.randn(K, M, device="cuda", dtype=torch.bfloat16) * 0.1
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16) * 0.1
    out = gemm_bf16_tn(a, b, out_dtype=torch.float32)
    torch.testing.assert_close(out, a.float().t() @ b.float(), atol=3e-2, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("epilogue", ["none", "swiglu"])
@pytest.mark.parametrize("pair", ["1", "0"])
def test_grouped_gemm_uneven_groups(epilogue, pair):
    """Ragged GEMM (one weight matrix per row group) with an empty group, groups that end inside a 256-row tile and rows behind
    the last group, on the CTA-pair kernel and on the one-CTA-per-tile kernel (selected by a variable read once per process,
    hence the child process), against per-group fp32 products."""
    import os
    import subprocess
    import sys

    if os.environ.get("PKB_TEST_GROUPED_CHILD") != "1":
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        r = subprocess.run([sys.executable, "-m", "pytest", os.path.abspath(__file__), "-x", "-q", "-k",
                            f"test_grouped_gemm_uneven_groups and {epilogue} and {pair}"], cwd=root, capture_output=True, text=True,
                           timeout=600, env={**os.environ, "PKB_TEST_GROUPED_CHILD": "1", "PKB_GROUPED_PAIR": pair})
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-1500:]
        return
    from parallelkernelbench_b200.ops.moe import grouped_gemm

    torch.manual_seed(3)
    counts = [300, 0, 513, 128, 77, 256]
    G, N, K = len(counts), 512, 320
    rows = sum(counts) + 40                                  # rows behind the last group are never touched
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
    a = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(G, N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    n_out = N // 2 if epilogue == "swiglu" else N
    out = torch.full((rows, n_out), 7.0, device="cuda", dtype=torch.bfloat16)
    grouped_gemm(a, w, off, epilogue=epilogue, out=out)
    torch.cuda.synchronize()
    lo = 0
    for e, c in enumerate(counts):
        acc = a[lo:lo + c].float() @ w[e].float().t()
        ref = torch.nn.functional.silu(acc[:, 0::2]) * acc[:, 1::2] if epilogue == "swiglu" else acc
        assert torch.allclose(out[lo:lo + c].float(), ref, atol=2e-2, rtol=2e-2), (e, (out[lo:lo + c].float() - ref).abs().max())
        lo += c
    assert bool((out[lo:] == 7.0).all())                     # untouched
