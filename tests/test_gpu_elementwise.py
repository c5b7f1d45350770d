"""Elementwise kernels against plain PyTorch fp32 restatements of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_rope_matches_rotate_half():
    from parallelkernelbench_b200.ops import rope

    x = torch.randn(4, 37, 8, 64, device="cuda", dtype=torch.bfloat16)
    ang = torch.rand(4, 37, 32, device="cuda") * 6.28
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    y = rope(x, cos, sin)
    xf = x.float()
    rot = torch.cat([-xf[..., 32:], xf[..., :32]], -1)
    ref = xf * cos.to(torch.bfloat16).float().unsqueeze(-2) + rot * sin.to(torch.bfloat16).float().unsqueeze(-2)
    torch.testing.assert_close(y.float(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fp8_quant_dequant_round_trip(dtype):
    from parallelkernelbench_b200.ops import fp8_dequantize_1x128, fp8_quantize_1x128

    x = torch.randn(64, 1024, device="cuda", dtype=dtype) * 3
    x[3, 128:256] = 0                                    # an all-zero block keeps scale 1
    y, s = fp8_quantize_1x128(x)
    xb = x.float().view(64, 8, 128)
    s_ref = xb.abs().amax(-1) / 448.0
    s_ref = torch.where(s_ref == 0, torch.ones_like(s_ref), s_ref)
    torch.testing.assert_close(s, s_ref, rtol=1e-6, atol=0)
    y_ref = (xb / s_ref.unsqueeze(-1)).to(torch.float8_e4m3fn).view(64, 1024)
    assert (y.view(torch.float8_e4m3fn).float() - y_ref.float()).abs().max() <= 32.0   # at most one fp8 ulp at the top
    assert (y.view(torch.float8_e4m3fn).float() != y_ref.float()).float().mean() < 0.01
    back = fp8_dequantize_1x128(y, s, torch.float32)
    torch.testing.assert_close(back, x.float(), atol=2e-3, rtol=0.07)   # e4m3: 3 mantissa bits, subnormals near zero
    y2, s2 = fp8_quantize_1x128(x, pow2_scales=True)
    assert torch.all(torch.log2(s2) == torch.log2(s2).round())


@pytest.mark.parametrize("decoupled", [True, False])
def test_adam_matches_torch_optimizer(decoupled):
    from parallelkernelbench_b200.ops import adam_step

    n = 10007
    p0 = torch.randn(n, device="cuda")
    p = p0.clone(); m = torch.zeros(n, device="cuda"); v = torch.zeros(n, device="cuda")
    ref_p = torch.nn.Parameter(p0.clone())
    opt_cls = torch.optim.AdamW if decoupled else torch.optim.Adam
    opt = opt_cls([ref_p], lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        ref_p.grad = g.clone()
        opt.step()
        adam_step(p, m, v, g, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, step=step, weight_decay=0.1, decoupled=decoupled, p_bf16=pb)
    torch.testing.assert_close(p, ref_p.data, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(pb.float(), p, atol=1e-2, rtol=1e-2)


def test_cross_entropy_stats_single_rank_equals_torch():
    from parallelkernelbench_b200.ops import ce_finalize, ce_local_stats

    logits = torch.randn(50, 1000, device="cuda", dtype=torch.bfloat16) * 4
    tgt = torch.randint(0, 1000, (50,), device="cuda")
    halves = [ce_local_stats(logits[:, :512].contiguous(), tgt, 0), ce_local_stats(logits[:, 512:].contiguous(), tgt, 512)]
    loss = ce_finalize(torch.stack(halves))
    ref = torch.nn.functional.cross_entropy(logits.float(), tgt, reduction="none")
    torch.testing.assert_close(loss, ref, atol=2e-3, rtol=2e-3)


def test_layernorm_backward_column_reduce():
    from parallelkernelbench_b200.ops import ln_bwd_colreduce

    xh = torch.randn(1000, 333, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(1000, 333, device="cuda", dtype=torch.bfloat16)
    dg, db = ln_bwd_colreduce(xh, dy)
    torch.testing.assert_close(dg, (dy.float() * xh.float()).sum(0), atol=1e-2, rtol=1e-3)
    torch.testing.assert_close(db, dy.float().sum(0), atol=1e-2, rtol=1e-3)
