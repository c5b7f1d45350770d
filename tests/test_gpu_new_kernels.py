"""Block-scaled fp8 GEMM (dense, grouped, SwiGLU and re-quantising epilogues) against the fp32 PyTorch restatement
of the same arithmetic on dequantised operands; the fused router; the fused GEMM + all-reduce / + all-gather and GEMV +
all-gather kernels against their two-launch forms; the MoE layer with fp8 experts and with the combine pushed from the down
GEMM's epilogue; the debug builds (timing perturbation, checked heap bases, guard bands); checkpoint resume."""
import os

import pytest
import torch

pytestmark = [pytest.mark.gpu]


def _operands(M, N, K, groups=0, seed=0):
    from parallelkernelbench_b200.refs.gemm_fp8 import quantize_rows_1x128, quantize_weight_128x128

    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(M, K, device="cuda", generator=g) * torch.rand(M, 1, device="cuda", generator=g) * 4   # rows of different magnitude
    w = torch.randn((groups, N, K) if groups else (N, K), device="cuda", generator=g) * 0.05
    return quantize_rows_1x128(a), quantize_weight_128x128(w)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 1024), (300, 384, 512), (4096, 2048, 2048)])
def test_dense_matches_dequantised_product(M, N, K):
    from parallelkernelbench_b200.ops.gemm_fp8 import gemm_fp8_blockscaled
    from parallelkernelbench_b200.refs.gemm_fp8 import gemm_fp8_blockscaled_ref

    (a8, sa), (w8, sb) = _operands(M, N, K)
    out = torch.full((M + 8, N), float("nan"), device="cuda", dtype=torch.bfloat16)      # rows past M must stay untouched
    gemm_fp8_blockscaled(a8, sa, w8, sb, out=out[:M])
    ref = gemm_fp8_blockscaled_ref(a8, sa, w8, sb)
    torch.testing.assert_close(out[:M].float(), ref.float(), rtol=1e-2, atol=1e-2 * ref.float().abs().max().item())
    assert torch.isnan(out[M:]).all()


def test_grouped_swiglu_and_requantise_feed_a_second_gemm():
    from parallelkernelbench_b200.ops.gemm_fp8 import gemm_fp8_blockscaled
    from parallelkernelbench_b200.refs.gemm_fp8 import dequantize_rows_1x128, gemm_fp8_blockscaled_ref

    G, H, I = 6, 512, 256
    counts = torch.tensor([130, 0, 128, 5, 257, 64])
    offsets = torch.zeros(G + 1, dtype=torch.int32)
    offsets[1:] = counts.cumsum(0)
    M = int(offsets[-1]) + 40                                            # spare rows after the last group
    (a8, sa), (w8, sb) = _operands(M, 2 * I, H, groups=G, seed=1)
    off_d = offsets.cuda()

    h_ref = gemm_fp8_blockscaled_ref(a8, sa, w8, sb, offsets, "swiglu")
    h = gemm_fp8_blockscaled(a8, sa, w8, sb, offsets=off_d, epilogue="swiglu")
    rows = int(offsets[-1])
    torch.testing.assert_close(h[:rows].float(), h_ref[:rows].float(), rtol=2e-2, atol=2e-2 * h_ref.float().abs().max().item())

    h8, hs = gemm_fp8_blockscaled(a8, sa, w8, sb, offsets=off_d, epilogue="swiglu_quant")
    h8_ref, hs_ref = gemm_fp8_blockscaled_ref(a8, sa, w8, sb, offsets, "swiglu_quant")
    back, back_ref = dequantize_rows_1x128(h8[:rows], hs[:rows]), dequantize_rows_1x128(h8_ref[:rows], hs_ref[:rows])
    torch.testing.assert_close(back, back_ref, rtol=0.14, atol=2e-2 * back_ref.abs().max().item())   # one e4m3 step where bf16 rounding differs

    (_, _), (w8d, sbd) = _operands(1, H, I, groups=G, seed=2)
    y = gemm_fp8_blockscaled(h8, hs, w8d, sbd, offsets=off_d)
    y_ref = gemm_fp8_blockscaled_ref(h8, hs, w8d, sbd, offsets)
    torch.testing.assert_close(y[:rows].float(), y_ref[:rows].float(), rtol=1e-2, atol=1e-2 * y_ref.float().abs().max().item())


def test_moe_layer_with_fp8_experts_matches_its_reference():
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=1", "--master-addr", "127.0.0.1",
           "--master-port", "29671", os.path.join(root, "tests/mp/all_ops_worker.py"), "--ops", "moe_layer", "--config", "fp8_experts"]
    r = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "TOTAL_FAILS 0" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def _all_ops(nproc, port, *args, env=None):
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(root, "tests/mp/all_ops_worker.py"), *args]
    r = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600, env={**os.environ, **(env or {})})
    assert r.returncode == 0 and "TOTAL_FAILS 0" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.parametrize("nproc", [1, 2])
def test_fused_gemm_allreduce_matches_gemm_then_allreduce(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    _all_ops(nproc, 29672 + nproc, "--ops", "gemm_allreduce", "--config", "default", env={"PKB_FUSED_GEMM_AR": "1"})
    _all_ops(nproc, 29676 + nproc, "--ops", "gemm_allreduce", "--config", "large", env={"PKB_FUSED_GEMM_AR": "1"})


@pytest.mark.parametrize("E,k", [(8, 2), (64, 6), (256, 8), (100, 3)])
def test_fused_router_matches_softmax_topk_bincount(E, k):
    from parallelkernelbench_b200.ops.moe import route_topk

    g = torch.Generator(device="cuda").manual_seed(E)
    logits = torch.randn(777, E, device="cuda", generator=g) * 2
    bias = torch.randn(E, device="cuda", generator=g) * 0.1
    logits[5, :] = 0.25                                    # a row of exact ties: the lowest indices must win, in order
    for b in (None, bias):
        if b is not None:
            logits[5, :] = 0.25 - b                        # keep the tie after the bias is added
        gates, idx, counts = route_topk(logits, b, k)
        ref_g, ref_i = torch.topk(torch.softmax(logits + (0 if b is None else b), dim=-1), k, dim=-1)
        torch.testing.assert_close(gates, ref_g, rtol=1e-5, atol=1e-7)
        rows = torch.ones(777, dtype=torch.bool, device="cuda")
        rows[5] = False                                    # torch.topk leaves the order among exact ties unspecified
        assert torch.equal(idx[rows].long(), ref_i[rows])
        if b is None:
            assert idx[5].tolist() == list(range(k))
        assert torch.equal(counts.long(), torch.bincount(idx.view(-1).long(), minlength=E))


def test_moe_layer_with_fused_router():
    _all_ops(1, 29681, "--ops", "moe_layer", "--config", "default", env={"PKB_FUSED_ROUTER": "1"})


@pytest.mark.parametrize("nproc", [1, 2])
def test_fused_gemm_allgather_matches_gemm_then_allgather(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    _all_ops(nproc, 29684 + nproc, "--ops", "gemm_allgather", "--config", "default", env={"PKB_FUSED_GEMM_AG": "1"})
    _all_ops(nproc, 29688 + nproc, "--ops", "gemm_allgather", "--config", "large", env={"PKB_FUSED_GEMM_AG": "1"})


@pytest.mark.parametrize("nproc", [1, 2])
def test_moe_layer_with_expert_outputs_pushed_home_by_the_down_gemm(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    _all_ops(nproc, 29692 + nproc, "--ops", "moe_layer", "--config", "default", env={"PKB_PUSH_COMBINE": "1"})
    _all_ops(nproc, 29696 + nproc, "--ops", "moe_layer", "--config", "fp8_experts", env={"PKB_PUSH_COMBINE": "1"})


def test_fsdp_llama_resumes_from_sharded_checkpoint():
    """Not a kernel: the engine's per-rank checkpoint (fp32 master, Adam moments, fp8 wire copy, head, step count)."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=1", "--master-addr", "127.0.0.1",
           "--master-port", "29699", os.path.join(root, "tests/mp/llama_worker.py"), "--resume-check"]
    r = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "TOTAL_FAILS 0" in r.stdout and "-> same" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_collectives_and_tp_mlp_under_the_timing_perturbation_build():
    """Random pauses around every signal and wait (PKB_JITTER=1 loads the -DPKB_JITTER library): results must not change."""
    import subprocess
    import sys

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not os.path.exists(os.path.join(root, "parallelkernelbench_b200/_lib/libpkb200_cuda_jitter.so")):
        pytest.skip("build it with: python -m parallelkernelbench_b200.build --jitter")
    for i, script in enumerate(("tests/mp/collectives_worker.py", "tests/mp/tp_mlp_worker.py", "tests/mp/moe_worker.py")):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
               "--master-port", str(29660 + i), os.path.join(root, script)]
        r = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=900, env={**os.environ, "PKB_JITTER": "1"})
        assert r.returncode == 0 and "TOTAL_FAILS 0" in r.stdout, script + r.stdout[-3000:] + r.stderr[-3000:]


def test_collectives_and_moe_under_the_checked_build_record_no_violation():
    """PKB_DEBUG_BOUNDS=1 loads the -DPKB_DEBUG_BOUNDS library: correct code must leave the status block clean."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not os.path.exists(os.path.join(root, "parallelkernelbench_b200/_lib/libpkb200_cuda_bounds.so")):
        pytest.skip("build it with: python -m parallelkernelbench_b200.build --debug-bounds")
    n = 2 if torch.cuda.device_count() >= 2 else 1
    for i, script in enumerate(("tests/mp/collectives_worker.py", "tests/mp/moe_worker.py")):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
               "--master-port", str(29664 + i), os.path.join(root, script)]
        r = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=900, env={**os.environ, "PKB_DEBUG_BOUNDS": "1"})
        assert r.returncode == 0 and "TOTAL_FAILS 0" in r.stdout, script + r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.parametrize("nproc", [1, 2])
def test_fused_gemv_allgather_matches_gemv_then_allgather(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    _all_ops(nproc, 29652 + nproc, "--ops", "gemv_decode", "--config", "default", "--trials", "3", env={"PKB_FUSED_GEMV_AG": "1"})
    _all_ops(nproc, 29656 + nproc, "--ops", "gemv_decode", "--config", "llama", env={"PKB_FUSED_GEMV_AG": "1"})


def test_speculative_single_pass_softmax_is_bit_identical_to_the_two_pass_form(tmp_path):
    """PKB_FA_SPEC=1 changes how often S is read from TMEM, not which offsets the exponentials use: outputs must be equal bit
    for bit, and the ordinary forward tests must pass with it."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    files = {}
    for name, env in (("two_pass", {}), ("spec", {"PKB_FA_SPEC": "1"})):
        files[name] = str(tmp_path / f"{name}.pt")
        r = subprocess.run([sys.executable, os.path.join(root, "tests/mp/fa_variant_worker.py"), files[name]], cwd=root,
                           capture_output=True, text=True, timeout=600, env={**os.environ, **env})
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    a, b = torch.load(files["two_pass"]), torch.load(files["spec"])
    for k in a:
        assert torch.equal(a[k], b[k]), k
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(root, "tests/test_gpu_attention.py"), "-x", "-q", "-k",
                        "matches_reference or zigzag_rank"], cwd=root, capture_output=True, text=True, timeout=900,
                       env={**os.environ, "PKB_FA_SPEC": "1"})
    assert r.returncode == 0, r.stdout[-3000:]


def test_own_kernel_example_solution_matches_on_gpu():
    """The worked example that compiles its own CUDA kernels at first use, evaluated like any candidate file."""
    from parallelkernelbench_b200.harness import launch
    from parallelkernelbench_b200.kernelgen.examples import example_path

    s = launch.eval_op("tp_rmsnorm", 1, trials=1, solution=str(example_path("tp_rmsnorm")), timeout_s=600)
    assert s["all_ok"], s["trials"][-1]


def test_fsdp_llama_step_through_the_harness():
    """The engine as a registry op: ours against the PyTorch + NCCL implementation of the same engine, first step's loss."""
    from parallelkernelbench_b200.harness import launch

    s = launch.eval_op("fsdp_llama_step", 1, trials=1, config="default", timeout_s=900)
    assert s["all_ok"], s["trials"][-1]


@pytest.mark.parametrize("op", ["allreduce", "alltoall", "tp_mlp", "moe_layer"])
def test_ops_leave_the_guard_bands_of_the_symmetric_heap_intact(op):
    """PKB_HEAP_GUARD=1 brackets every symmetric allocation with pattern-filled bands; the worker checks them after the run."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    n = 2 if torch.cuda.device_count() >= 2 else 1
    r = subprocess.run([sys.executable, "-m", "parallelkernelbench_b200.harness.launch", "run", "--op", op, "--impl", "ours", "--nproc", str(n),
                        "--config", "small"], cwd=root, capture_output=True, text=True, timeout=600, env={**os.environ, "PKB_HEAP_GUARD": "1"})
    assert r.returncode == 0 and "dry run ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("state_dtype", [torch.bfloat16, torch.float32])
def test_fused_zero_adam_step_matches_the_formula_on_one_rank(state_dtype):
    """One rank: the reduction and the gather degenerate to local moves, the arithmetic is the whole of it."""
    from parallelkernelbench_b200.ops.optim import ZeroAdamStep
    from parallelkernelbench_b200.parallel import init_context

    os.environ.setdefault("PKB_HEAP_GIB", "0.25")
    ctx = init_context()
    try:
        part = 8 * 1000 + 8
        g = torch.Generator(device="cuda").manual_seed(3)
        op = ZeroAdamStep(ctx.heap().world_group, part)
        grad = torch.randn(part, device="cuda", generator=g).to(torch.bfloat16)
        p0 = (torch.randn(part, device="cuda", generator=g) * 0.2).to(state_dtype)
        m0 = (torch.randn(part, device="cuda", generator=g) * 0.01).to(state_dtype)
        v0 = (torch.rand(part, device="cuda", generator=g) * 0.01).to(state_dtype)
        lr, b1, b2, eps, wd, step, gs = 1e-2, 0.9, 0.95, 1e-8, 0.1, 3, 0.5
        op.grad_buffer.copy_(grad)
        p, m, v = p0.clone(), m0.clone(), v0.clone()
        full = op.step(p, m, v, lr=lr, beta1=b1, beta2=b2, eps=eps, step=step, weight_decay=wd, grad_scale=gs)
        gf = grad.float() * gs
        m_ref = b1 * m0.float() + (1 - b1) * gf
        v_ref = b2 * v0.float() + (1 - b2) * gf * gf
        upd = (m_ref / (1 - b1 ** step)) / ((v_ref / (1 - b2 ** step)).sqrt() + eps)
        p_ref = p0.float() - lr * upd - lr * wd * p0.float()
        tol = dict(atol=1e-5, rtol=1e-5) if state_dtype == torch.float32 else dict(atol=1e-2, rtol=1e-2)
        torch.testing.assert_close(p.float(), p_ref, **tol)
        torch.testing.assert_close(m.float(), m_ref, **tol)
        torch.testing.assert_close(v.float(), v_ref, **tol)
        torch.testing.assert_close(full.float(), p_ref, atol=1e-2, rtol=1e-2)      # the gathered copy is bf16
    finally:
        ctx.finalize()


def test_fused_quantise_and_rope_pushes_match_their_two_step_forms_on_one_rank():
    """One rank: the gather is a local store, what is checked is the arithmetic and the layout of the gathered buffers."""
    from parallelkernelbench_b200.ops import fp8_quantize_1x128, rope
    from parallelkernelbench_b200.ops.fused_push import Fp8QuantAllGather, RopeAllGather
    from parallelkernelbench_b200.parallel import init_context

    os.environ.setdefault("PKB_HEAP_GIB", "0.25")
    ctx = init_context()
    try:
        group = ctx.heap().world_group
        g = torch.Generator(device="cuda").manual_seed(9)
        x = (torch.randn(37, 384, device="cuda", generator=g) * torch.rand(37, 1, device="cuda", generator=g) * 5).to(torch.bfloat16)
        x[3] = 0                                                     # an all-zero block keeps scale 1
        y, s = Fp8QuantAllGather(group, tuple(x.shape))(x)
        y_ref, s_ref = fp8_quantize_1x128(x)
        assert torch.equal(y[0], y_ref) and torch.equal(s[0], s_ref)

        b, t, hq, hk, d = 2, 24, 4, 2, 64
        q = torch.randn(b, t, hq, d, device="cuda", generator=g).to(torch.bfloat16)
        k = torch.randn(b, t, hk, d, device="cuda", generator=g).to(torch.bfloat16)
        ang = torch.rand(b, t, d, device="cuda", generator=g) * 6.28
        cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
        qg, kg = RopeAllGather(group, b, t, hq, hk, d)(q, k, cos, sin)
        torch.testing.assert_close(qg, rope(q, cos, sin), atol=1e-2, rtol=1e-2)
        torch.testing.assert_close(kg, rope(k, cos, sin), atol=1e-2, rtol=1e-2)
    finally:
        ctx.finalize()
