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
    # scales and payload bytes equal PyTorch's evaluation of the same formula on the GPU bit for bit: the scale is amax times the
    # rounded reciprocal of 448 (how a tensor divided by a Python scalar is computed there), the quotient is correctly rounded
    assert torch.equal(s, s_ref)
    y_ref = (xb / s_ref.unsqueeze(-1)).to(torch.float8_e4m3fn).view(64, 1024)
    assert torch.equal(y.view(torch.uint8), y_ref.view(torch.uint8))
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


def test_fsdp_adamw_fp8_matches_dequant_sum_then_adamw():
    """fp8 slices + scales -> summed gradient -> AdamW -> re-quantised weights, against plain fp32 PyTorch."""
    from parallelkernelbench_b200.ops import fp8_dequantize_1x128, fp8_quantize_1x128
    from parallelkernelbench_b200.ops.quant import fsdp_adamw_fp8

    torch.manual_seed(5)
    W, n = 4, 128 * 257
    grads = [torch.randn(n, device="cuda") * 0.01 for _ in range(W)]
    qs = [fp8_quantize_1x128(g.view(-1, 128)) for g in grads]
    payload = torch.stack([q.view(-1) for q, _ in qs])
    scales = torch.stack([s.view(-1) for _, s in qs])
    gsum = sum(fp8_dequantize_1x128(q, s, torch.float32).view(-1) for q, s in qs) / W
    p = torch.randn(n, device="cuda") * 0.02
    m, v = torch.randn(n, device="cuda") * 1e-3, torch.rand(n, device="cuda") * 1e-5
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    q_out = torch.empty(n, dtype=torch.uint8, device="cuda")
    s_out = torch.empty(n // 128, device="cuda")
    pb = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    lr, b1, b2, eps, wd, step = 1e-3, 0.9, 0.95, 1e-8, 0.1, 3
    fsdp_adamw_fp8(payload, scales, p, m, v, q_out, s_out, lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd,
                   grad_scale=1.0 / W, step=step, p_bf16=pb)
    pr.mul_(1 - lr * wd)
    mr.mul_(b1).add_(gsum, alpha=1 - b1)
    vr.mul_(b2).addcmul_(gsum, gsum, value=1 - b2)
    pr.addcdiv_(mr / (1 - b1 ** step), (vr / (1 - b2 ** step)).sqrt() + eps, value=-lr)
    torch.testing.assert_close(p, pr, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(m, mr, rtol=1e-5, atol=1e-9)
    torch.testing.assert_close(v, vr, rtol=1e-5, atol=1e-12)
    torch.testing.assert_close(pb.float(), pr, rtol=1e-2, atol=1e-4)
    back = fp8_dequantize_1x128(q_out.view(-1, 128), s_out.view(-1, 1), torch.float32).view(-1)
    torch.testing.assert_close(back, pr, rtol=0.07, atol=2e-3)


def test_swiglu_forward_backward_match_autograd():
    from parallelkernelbench_b200.ops import swiglu_bwd, swiglu_fwd

    torch.manual_seed(6)
    gu = torch.randn(300, 2 * 1024, device="cuda", dtype=torch.bfloat16)
    da = torch.randn(300, 1024, device="cuda", dtype=torch.bfloat16)
    ref_in = gu.float().requires_grad_()
    ref = torch.nn.functional.silu(ref_in[:, :1024]) * ref_in[:, 1024:]
    ref.backward(da.float())
    torch.testing.assert_close(swiglu_fwd(gu).float(), ref.detach(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(swiglu_bwd(gu, da).float(), ref_in.grad, rtol=2e-2, atol=3e-2)


@pytest.mark.parametrize("H", [512, 4096, 8192])
def test_rmsnorm_backward_matches_autograd(H):
    from parallelkernelbench_b200.ops import rmsnorm_bwd

    torch.manual_seed(7)
    rows, eps = 777, 1e-5
    x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16)
    g = (1.0 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
    dy = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16)
    xr, gr = x.float().requires_grad_(), g.float().requires_grad_()
    y = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + eps) * gr
    y.backward(dy.float())
    dx, dg = rmsnorm_bwd(x, g, dy, eps)
    torch.testing.assert_close(dx.float(), xr.grad, rtol=2e-2, atol=3e-2)
    torch.testing.assert_close(dg, gr.grad, rtol=1e-2, atol=2e-1)


def test_cross_entropy_backward_matches_autograd():
    from parallelkernelbench_b200.ops import ce_backward

    torch.manual_seed(8)
    rows, V, start = 64, 1024, 512                      # this "rank" owns vocabulary [512, 1536) of 2048
    full = torch.randn(rows, 2048, device="cuda")
    tgt = torch.randint(0, 2048, (rows,), device="cuda")
    lse = torch.logsumexp(full, -1)
    ref = (torch.softmax(full, -1) - torch.nn.functional.one_hot(tgt, 2048).float())[:, start:start + V] / rows
    got = ce_backward(full[:, start:start + V].to(torch.bfloat16), lse, tgt, start, 1.0 / rows)
    torch.testing.assert_close(got.float(), ref, rtol=3e-2, atol=2e-4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_clip_grad_norm_kernels_match_torch(dtype):
    from parallelkernelbench_b200.ops.quant import clip_grad_norm_

    torch.manual_seed(9)
    grads = [torch.randn(n, device="cuda", dtype=dtype) for n in (1000, 77, 4096 * 33, 5, 1 << 20, 300, 12, 64, 999, 2048)]   # two batches
    scales = [1.0, 0.5, 1.0, 1.0, 0.25, 1.0, 1.0, 2.0, 1.0, 1.0]
    ref = [g.float() * s for g, s in zip(grads, scales)]
    total = torch.sqrt(sum((r * r).sum() for r in ref))
    for max_norm in (1.0, 1e9):
        mine = [g.clone() for g in grads]
        norm = clip_grad_norm_(mine, max_norm, pre_scale=scales)
        coef = min(max_norm / float(total), 1.0)
        torch.testing.assert_close(norm, total, rtol=2e-3, atol=1e-3)
        for got, r in zip(mine, ref):
            torch.testing.assert_close(got.float(), r * coef, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-6)


@pytest.mark.gpu
def test_fp8_dequant_stops_at_the_device_side_row_count():
    from parallelkernelbench_b200.ops import fp8_dequantize_1x128, fp8_quantize_1x128

    x = torch.randn(96, 512, device="cuda", dtype=torch.bfloat16)
    y, s = fp8_quantize_1x128(x)
    full = fp8_dequantize_1x128(y, s, torch.bfloat16)
    valid = torch.tensor([37], dtype=torch.int32, device="cuda")
    part = fp8_dequantize_1x128(y, s, torch.bfloat16, valid_rows=valid)
    assert torch.equal(part[:37], full[:37])
    assert torch.allclose(full.float(), x.float(), atol=0.3, rtol=0.07)
