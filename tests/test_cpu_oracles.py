"""The fp32 restatements that GPU kernels are checked against are themselves checked here, on CPU, against independent
formulations (autograd, einsum algebra, brute force)."""
import math

import torch


def test_attention_backward_formula_matches_autograd():
    from parallelkernelbench_b200.refs.attention import attention_bwd_positions_ref, attention_positions_ref

    torch.manual_seed(0)
    Sq, Skv, Hq, Hkv, D = 24, 40, 4, 2, 8
    q, k, v = torch.randn(Sq, Hq, D, requires_grad=True), torch.randn(Skv, Hkv, D, requires_grad=True), torch.randn(Skv, Hkv, D, requires_grad=True)
    dout = torch.randn(Sq, Hq, D)
    q_pos, kv_pos = torch.arange(16, 16 + Sq), torch.arange(Skv)
    for causal in (False, True):
        for t in (q, k, v):
            t.grad = None
        out, lse = attention_positions_ref(q, k, v, q_pos, kv_pos, causal, D ** -0.5)
        out.backward(dout)
        dq, dk, dv = attention_bwd_positions_ref(q.detach(), k.detach(), v.detach(), out.detach(), lse.detach(), dout, q_pos, kv_pos,
                                                 causal, D ** -0.5)
        torch.testing.assert_close(dq, q.grad, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(dk, k.grad, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(dv, v.grad, rtol=1e-4, atol=1e-5)


def test_gaussian_projection_restatement_matches_matrix_algebra():
    """quaternion -> R, covariance R S^2 R^T, world -> camera, Jacobian projection, conics and radii written as matrix
    products (the way the splatting literature states them) against the elementwise fixed-order restatement."""
    from parallelkernelbench_b200.refs.gsplat import project

    torch.manual_seed(1)
    N, C, W, H = 200, 3, 96, 64
    means = torch.stack([(torch.rand(N) - 0.5) * 8.0, (torch.rand(N) - 0.5) * 8.0, torch.rand(N) * 2 + 2], -1)   # some fall outside
    quats, scales = torch.randn(N, 4), torch.rand(N, 3) * 0.05
    view = torch.eye(4).repeat(C, 1, 1)
    view[:, 0, 3] = torch.tensor([0.0, 0.1, -0.2])
    ang = 0.1
    view[2, :3, :3] = torch.tensor([[math.cos(ang), 0, math.sin(ang)], [0, 1, 0], [-math.sin(ang), 0, math.cos(ang)]])
    K = torch.eye(3).repeat(C, 1, 1)
    K[:, 0, 0] = K[:, 1, 1] = 0.8 * min(W, H)
    K[:, 0, 2], K[:, 1, 2] = W / 2, H / 2
    radii, m2, depth, conics = project(means, quats, scales, view, K, W, H)

    qn = torch.nn.functional.normalize(quats, dim=-1)
    w, x, y, z = qn.unbind(-1)
    R = torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y), 2 * (x * y + w * z), 1 - 2 * (x * x + z * z),
                     2 * (y * z - w * x), 2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)], -1).view(N, 3, 3)
    M = R * scales[:, None, :]
    cov = M @ M.transpose(1, 2)
    Rc, t = view[:, :3, :3], view[:, :3, 3]
    mc = torch.einsum("cij,nj->cni", Rc, means) + t[:, None, :]
    cc = torch.einsum("cij,njk,clk->cnil", Rc, cov, Rc)
    tz = mc[..., 2]
    fx, fy, cx, cy = K[:, 0, 0, None], K[:, 1, 1, None], K[:, 0, 2, None], K[:, 1, 2, None]
    lim_xp, lim_xn = (W - cx) / fx + 0.3 * 0.5 * W / fx, cx / fx + 0.3 * 0.5 * W / fx
    lim_yp, lim_yn = (H - cy) / fy + 0.3 * 0.5 * H / fy, cy / fy + 0.3 * 0.5 * H / fy
    tx = tz * torch.minimum(torch.maximum(mc[..., 0] / tz, -lim_xn), lim_xp)
    ty = tz * torch.minimum(torch.maximum(mc[..., 1] / tz, -lim_yn), lim_yp)
    O = torch.zeros_like(tz)
    J = torch.stack([fx / tz, O, -fx * tx / tz ** 2, O, fy / tz, -fy * ty / tz ** 2], -1).view(C, N, 2, 3)
    cov2 = J @ cc @ J.transpose(-1, -2)
    ref_m2 = torch.einsum("cij,cnj->cni", K[:, :2, :3], mc) / tz[..., None]
    cov2 = cov2 + torch.eye(2) * 0.3
    det = (cov2[..., 0, 0] * cov2[..., 1, 1] - cov2[..., 0, 1] * cov2[..., 1, 0]).clamp(min=1e-10)
    ref_con = torch.stack([cov2[..., 1, 1] / det, -(cov2[..., 0, 1] + cov2[..., 1, 0]) / 2 / det, cov2[..., 0, 0] / det], -1)
    torch.testing.assert_close(m2, ref_m2, rtol=1e-4, atol=1e-3)
    torch.testing.assert_close(depth, tz, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(conics, ref_con, rtol=2e-3, atol=1e-4)
    ref_rx = torch.ceil(3.33 * torch.sqrt(cov2[..., 0, 0]))
    visible = radii[..., 0] > 0
    assert visible.any() and (~visible).any()                     # the scene has both culled and surviving Gaussians
    assert ((radii[..., 0].float() - ref_rx)[visible].abs() <= 1).all()   # ceil may flip on last-bit differences


def test_segment_permute_first_seen_unique_and_target_counts():
    from parallelkernelbench_b200.workloads.wild import _first_seen_unique, _segment_permute, _target_counts

    data = torch.arange(10)
    seg = torch.tensor([3, 0, 2, 5])
    out = _segment_permute(data, seg, torch.tensor([3, 0, 2, 1]))
    assert out.tolist() == [5, 6, 7, 8, 9, 0, 1, 2, 3, 4]
    new, allnodes = _first_seen_unique(torch.tensor([7, 3]), torch.tensor([3, 9, 7, 9, 1]))
    assert allnodes.tolist() == [7, 3, 9, 1] and new.tolist() == [9, 1]
    sizes = torch.tensor([5, 0, 7, 1])                              # 13 elements over 4 ranks -> 4, 3, 3, 3
    sent = torch.stack([_target_counts(sizes, r, 4) for r in range(4)])
    assert sent.sum(0).tolist() == [4, 3, 3, 3] and sent.sum(1).tolist() == sizes.tolist()


def test_permuting_all_to_all_descriptor_reproduces_chunk_and_cat():
    """The (extents, strides, offsets) handed to the permuting all-to-all kernel, executed here by a plain Python copy loop
    over byte buffers, must give what chunk -> exchange -> cat gives."""
    from parallelkernelbench_b200.ops.collectives import _collapse

    torch.manual_seed(2)
    W = 4
    for shape, sd, gd in [((8, 6), 0, 1), ((2, 3, 8, 5), 2, 1), ((2, 4, 8, 5), 1, 2), ((4, 4, 3), 0, 0), ((3, 8, 2, 2), 1, 3)]:
        xs = [torch.randn(*shape) for _ in range(W)]
        want = [torch.cat([xs[s].chunk(W, dim=sd)[r] for s in range(W)], dim=gd).contiguous() for r in range(W)]
        for r in range(W):
            box = list(shape)
            box[sd] //= W
            out_shape = list(box)
            out_shape[gd] *= W
            out = torch.empty(out_shape)
            es = 4
            in_st = [s * es for s in xs[0].stride()]
            out_st = [s * es for s in out.stride()]
            m = _collapse(box, in_st, out_st)
            inner = es
            if m and m[-1][1] == es and m[-1][2] == es:
                inner = m[-1][0] * es
                m = m[:-1]
            assert len(m) <= 3
            while len(m) < 3:
                m.insert(0, [1, 0, 0])
            in_rank_off, out_member_off = box[sd] * in_st[sd], box[gd] * out_st[gd]
            ob = out.view(-1).numpy().view("uint8")
            for g in range(W):
                ib = xs[g].contiguous().view(-1).numpy().view("uint8")
                for i0 in range(m[0][0]):
                    for i1 in range(m[1][0]):
                        for i2 in range(m[2][0]):
                            so = r * in_rank_off + i0 * m[0][1] + i1 * m[1][1] + i2 * m[2][1]
                            do = g * out_member_off + i0 * m[0][2] + i1 * m[1][2] + i2 * m[2][2]
                            ob[do:do + inner] = ib[so:so + inner]
            assert torch.equal(out, want[r]), (shape, sd, gd, r)


def test_block_scaled_fp8_restatement():
    """Quantisers invert within one e4m3 step, the block-scaled product equals the per-K-block scaled sum the kernel
    forms, and the grouped form equals one dense product per group."""
    from parallelkernelbench_b200.refs.gemm_fp8 import (dequantize_rows_1x128, dequantize_weight_128x128, gemm_fp8_blockscaled_ref,
                                                        quantize_rows_1x128, quantize_weight_128x128)

    torch.manual_seed(3)
    M, N, K = 70, 256, 384
    a, w = torch.randn(M, K) * 3, torch.randn(N, K) * 0.1
    a[5, 128:256] = 0
    a8, sa = quantize_rows_1x128(a)
    w8, sb = quantize_weight_128x128(w)
    assert a8.dtype == torch.uint8 and sa.shape == (M, K // 128) and sb.shape == (N // 128, K // 128) and sa[5, 1] == 1.0
    torch.testing.assert_close(dequantize_rows_1x128(a8, sa), a, rtol=0.07, atol=3 * 448 * 2 ** -9 / 448)
    torch.testing.assert_close(dequantize_weight_128x128(w8, sb), w, rtol=0.07, atol=1e-3)
    assert dequantize_rows_1x128(a8, sa).abs().amax() <= a.abs().amax() * (1 + 1e-6)       # amax maps to +-448 exactly

    # the sum the kernel forms: one unscaled e4m3 product per 128-deep K block, scaled and accumulated in fp32
    af, wf = a8.view(torch.float8_e4m3fn).float(), w8.view(torch.float8_e4m3fn).float()
    acc = torch.zeros(M, N)
    for kb in range(K // 128):
        part = af[:, kb * 128:(kb + 1) * 128] @ wf[:, kb * 128:(kb + 1) * 128].t()
        acc += part * sa[:, kb:kb + 1] * sb[:, kb].repeat_interleave(128)[None, :]
    ref = gemm_fp8_blockscaled_ref(a8, sa, w8, sb)
    torch.testing.assert_close(ref.float(), acc.to(torch.bfloat16).float(), rtol=1e-2, atol=1e-2)

    G = 3
    wg8, sbg = quantize_weight_128x128(torch.randn(G, N, K) * 0.1)
    offsets = torch.tensor([0, 20, 20, 64], dtype=torch.int32)
    out = gemm_fp8_blockscaled_ref(a8, sa, wg8, sbg, offsets)
    torch.testing.assert_close(out[:20], gemm_fp8_blockscaled_ref(a8[:20], sa[:20], wg8[0], sbg[0]))
    torch.testing.assert_close(out[20:64], gemm_fp8_blockscaled_ref(a8[20:64], sa[20:64], wg8[2], sbg[2]))
    assert out[64:].abs().max() == 0
    h8, hs = gemm_fp8_blockscaled_ref(a8, sa, wg8, sbg, offsets, "swiglu_quant")
    h = gemm_fp8_blockscaled_ref(a8, sa, wg8, sbg, offsets, "swiglu")
    assert h8.shape == (M, N // 2) and hs.shape == (M, N // 256)
    torch.testing.assert_close(dequantize_rows_1x128(h8, hs), h.float(), rtol=0.07, atol=1e-3 * h.float().abs().max().item() + 1e-6)


def test_moe_reference_with_fp8_experts_stays_close_to_bf16_experts():
    from parallelkernelbench_b200.refs.moe import moe_reference

    torch.manual_seed(4)
    T, H, I, E, k = 96, 256, 128, 4, 2
    x = torch.randn(T, H).to(torch.bfloat16)
    wr = (torch.randn(E, H) * 0.05).to(torch.bfloat16)
    wg, wu, wd = [(torch.randn(*s) * 0.05).to(torch.bfloat16) for s in ((E, I, H), (E, I, H), (E, H, I))]
    base = moe_reference(x, wr, None, wg, wu, wd, E, k, fp8_dispatch=True).float()
    q = moe_reference(x, wr, None, wg, wu, wd, E, k, fp8_dispatch=True, fp8_experts=True).float()
    err = (q - base).abs().max() / base.abs().max()
    assert 0 < err < 0.1, err


def test_fsdp_llama_sharded_checkpoint_round_trip_on_cpu():
    """2 steps in one go against 1 step, save, restore into a fresh engine, 1 step: same losses and the same master weights
    (PyTorch implementation of the engine, one CPU rank)."""
    import tempfile

    from parallelkernelbench_b200.models.llama import FSDPLlama, LlamaConfig
    from parallelkernelbench_b200.parallel import init_context

    ctx = init_context()
    cfg = LlamaConfig(layers=2, hidden=64, ffn=128, heads=4, kv_heads=2, vocab=256, seq=32)
    torch.manual_seed(0)
    tok = [torch.randint(0, 256, (32,)) for _ in range(2)]
    tgt = [torch.randint(0, 256, (32,)) for _ in range(2)]
    a = FSDPLlama(ctx, cfg, impl="torch")
    la = [float(a.step(tok[i], tgt[i])) for i in range(2)]
    b = FSDPLlama(ctx, cfg, impl="torch")
    lb0 = float(b.step(tok[0], tgt[0]))
    with tempfile.TemporaryDirectory() as d:
        path = b.save_sharded(d)
        assert path.endswith("rank_0_of_1.pt")
        c = FSDPLlama(ctx, cfg, impl="torch")
        assert c.load_sharded(d) == 1
        other = FSDPLlama(ctx, LlamaConfig(layers=2, hidden=64, ffn=256, heads=4, kv_heads=2, vocab=256, seq=32), impl="torch")
        try:
            other.load_sharded(d)
        except ValueError as e:
            assert "ffn" in str(e)
        else:
            raise AssertionError("a checkpoint of another config must be refused")
    lc1 = float(c.step(tok[1], tgt[1]))
    assert la[0] == lb0 and la[1] == lc1 and a.steps == c.steps == 2
    assert torch.equal(a.units[1].master, c.units[1].master) and torch.equal(a.head_master, c.head_master)
    assert torch.equal(a.embed.m, c.embed.m)


def test_push_combine_index_plan_reproduces_the_direct_sum():
    """Index logic of the MoE way home when the down GEMM's epilogue pushes rows: the dispatch delivers (sender, assignment
    index) with every row, the expert rank stores output row r at row `assignment index` of the sender's buffer, and the
    sender sums gates[t, j] * home[t * k + j]. Emulated with plain tensors for W ranks against the direct per-token sum."""
    torch.manual_seed(5)
    W, T, k, E, H = 3, 10, 2, 6, 4
    el = E // W
    f = lambda e, x: x * (e + 1) + 0.5 * e                                   # "expert e" as a cheap function of the row  # noqa: E731
    xs = [torch.randn(T, H) for _ in range(W)]
    idx = [torch.stack([torch.randperm(E)[:k] for _ in range(T)]) for _ in range(W)]
    gates = [torch.rand(T, k) for _ in range(W)]
    # dispatch: every rank appends its rows to the receive buffer of the expert's owner, expert-major, with the metadata
    recv = [[[] for _ in range(el)] for _ in range(W)]
    for s in range(W):
        for i in range(T * k):
            t, e = i // k, int(idx[s].view(-1)[i])
            recv[e // el][e % el].append((xs[s][t], s, i))
    home = [torch.full((T * k, H), float("nan")) for _ in range(W)]
    for r in range(W):                                                       # grouped GEMM with the row-scatter epilogue
        for le in range(el):
            for row, src, i in recv[r][le]:
                home[src][i] = f(r * el + le, row)
    for s in range(W):                                                       # local combine
        out = (gates[s].view(-1, 1) * home[s]).view(T, k, H).sum(1)
        want = torch.stack([sum(gates[s][t, j] * f(int(idx[s][t, j]), xs[s][t]) for j in range(k)) for t in range(T)])
        torch.testing.assert_close(out, want)
        assert not torch.isnan(home[s]).any()                                # every assignment came home exactly once
