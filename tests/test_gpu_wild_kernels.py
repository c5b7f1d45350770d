"""Numerics of the small project-derived compute kernels against plain PyTorch restatements of the same formulas."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nb,n", [(3, 1024), (2, 250), (2, 77), (1, 1)])
def test_kalman_block_step_matches_the_library_products(nb, n):
    from parallelkernelbench_b200.ops.wild import kalman_block_step

    g = torch.Generator(device="cuda").manual_seed(5 + n)
    H = torch.randn(nb, n, 1, dtype=torch.float64, device="cuda", generator=g) * 0.05
    w = torch.randn(nb, n, 1, dtype=torch.float64, device="cuda", generator=g)
    P = torch.eye(n, dtype=torch.float64, device="cuda").repeat(nb, 1, 1) + 0.01 * torch.randn(nb, n, n, dtype=torch.float64, device="cuda", generator=g)
    err = torch.randn(1, dtype=torch.float64, device="cuda", generator=g).reshape(())
    lam = 0.98
    P_in, w_in = P.clone(), w.clone()
    w_new, P_new = kalman_block_step(H, err, w, P, lam)
    K = torch.bmm(P, H)
    A = 1.0 / (lam + torch.bmm(H.transpose(1, 2), K)).sum()
    w_ref = w + A * err * K
    P_ref = (1.0 / lam) * (P - A * torch.bmm(K, K.transpose(1, 2)))
    torch.testing.assert_close(w_new, w_ref, atol=1e-12, rtol=1e-11)
    torch.testing.assert_close(P_new, P_ref, atol=1e-12, rtol=1e-11)
    assert torch.equal(P, P_in) and torch.equal(w, w_in)                 # the inputs are left alone
    # the denominator summed elsewhere (two ranks with the same data double it)
    w2, P2 = kalman_block_step(H, err, w, P, lam, all_reduce=lambda s: s * 2)
    A2 = A / 2
    torch.testing.assert_close(w2, w + A2 * err * K, atol=1e-12, rtol=1e-11)
    torch.testing.assert_close(P2, (1.0 / lam) * (P - A2 * torch.bmm(K, K.transpose(1, 2))), atol=1e-12, rtol=1e-11)
    again = kalman_block_step(H, err, w, P, lam)
    assert torch.equal(again[0], w_new) and torch.equal(again[1], P_new)  # fixed summation order: bit-reproducible


@pytest.mark.parametrize("B,P", [(1024, 16384), (40, 1000), (7, 33), (1, 4)])
def test_sinkhorn_knopp_matches_the_matrix_rewriting_form(B, P):
    from parallelkernelbench_b200.ops.wild import sinkhorn_coldot, sinkhorn_knopp, sinkhorn_rowdot

    g = torch.Generator(device="cuda").manual_seed(B + P)
    t = torch.randn(B, P, device="cuda", generator=g) * 0.05
    temp, iters = 0.07, 3
    E = torch.exp(t.double() / temp)
    r = torch.rand(P, device="cuda", generator=g) + 0.5
    c = torch.rand(B, device="cuda", generator=g) + 0.5
    torch.testing.assert_close(sinkhorn_rowdot(t, r, temp).double(), E @ r.double(), atol=0, rtol=2e-5)
    torch.testing.assert_close(sinkhorn_coldot(t, c, temp).double(), E.t() @ c.double(), atol=0, rtol=2e-5)

    def rewrite(world):                       # the reference's loop in fp64; `world` identical shards stand in for the ranks
        q = E.t().clone()
        total = float(B * world)
        q /= q.sum() * world
        for _ in range(iters):
            q /= q.sum(dim=1, keepdim=True) * world
            q /= P
            q /= q.sum(dim=0, keepdim=True)
            q /= total
        return (q * total).t().contiguous()

    out = sinkhorn_knopp(t, temp, iters)
    torch.testing.assert_close(out.double(), rewrite(1), atol=1e-9, rtol=1e-4)
    out2 = sinkhorn_knopp(t, temp, iters, all_reduce=lambda x: x * 2)
    torch.testing.assert_close(out2.double(), rewrite(2), atol=1e-9, rtol=1e-4)
    assert torch.equal(out, sinkhorn_knopp(t, temp, iters))               # fixed summation orders: bit-reproducible


@pytest.mark.parametrize("R,N,k,classes", [(32, 2048, 200, 1000), (5, 300, 7, 10), (3, 4096, 4096, 50), (2, 2, 1, 3)])
def test_knn_topk_matches_library_topk_and_votes(R, N, k, classes):
    from parallelkernelbench_b200.ops.wild import knn_merge_votes, knn_topk_local

    g = torch.Generator(device="cuda").manual_seed(R * N + k)
    sim = torch.randn(R, N, device="cuda", generator=g)
    labels = torch.randint(0, classes, (1, N), device="cuda", generator=g)
    top, idx = sim.topk(k, dim=1)
    lab = labels.expand(R, -1).gather(1, idx)
    votes = torch.zeros(R, classes, device="cuda").scatter_add_(1, lab, torch.ones_like(top)) / k
    s1, v1 = knn_topk_local(sim, labels, k, classes)
    assert torch.equal(s1, top)                                       # a selection: the values are the inputs themselves
    torch.testing.assert_close(v1, votes, atol=1e-6, rtol=1e-6)
    pairs = knn_topk_local(sim, labels, k)
    assert torch.equal(pairs[..., 0], top) and torch.equal(pairs[..., 1].long().sort(1).values, lab.sort(1).values)
    # merge of W candidate lists, laid out [W, Q, k, 2] as the exchange delivers them
    W, kk = 4, min(k, 4096 // 4)
    lists = torch.stack([torch.randn(R, kk, device="cuda", generator=g), torch.randint(0, classes, (R, kk), device="cuda", generator=g).float()], -1)
    lists = torch.stack([lists + 0.001 * s for s in range(W)])        # [W, R, kk, 2]; labels shifted too, rounded again below
    lists[..., 1] = lists[..., 1].round().clamp(0, classes - 1)
    s_all = lists[..., 0].permute(1, 0, 2).reshape(R, W * kk)
    l_all = lists[..., 1].permute(1, 0, 2).reshape(R, W * kk).long()
    km = min(k, W * kk)
    top2, ti = s_all.topk(km, dim=1)
    lab2 = l_all.gather(1, ti)
    votes2 = torch.zeros(R, classes, device="cuda").scatter_add_(1, lab2, torch.ones_like(top2)) / km
    s2, v2 = knn_merge_votes(lists, km, classes)
    assert torch.equal(s2, top2)
    torch.testing.assert_close(v2, votes2, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("n,H,W", [(9, 256, 256), (5, 8, 8), (1, 8, 4), (24, 64, 32)])
def test_mask_iou_suppression_matches_the_matrix_form(n, H, W):
    from parallelkernelbench_b200.ops.wild import mask_iou_suppress

    g = torch.Generator(device="cuda").manual_seed(n * H + W)
    base = torch.randn(-(-n // 3), H, W, device="cuda", generator=g)
    masks = base.repeat_interleave(3, 0)[:n].clone()
    masks = masks + 0.35 * torch.randn(masks.shape, device="cuda", generator=g)      # groups of three heavily overlapping masks
    last = torch.randint(-1, 4, (n,), device="cuda", generator=g)
    for thr in (0.7, 0.4):
        for reverse in (False, True):
            b = (masks > 0).flatten(1).float()
            inter = b @ b.t()
            area = b.sum(1)
            iou = inter / (area[:, None] + area[None, :] - inter).clamp_min(1.0)
            over = torch.triu(iou >= thr, diagonal=1)
            li, lj = last.view(n, 1), last.view(1, n)
            cmp = torch.lt if reverse else torch.gt
            want = (over & cmp(li, lj) & (lj > -1)).any(1) | (over & cmp(lj, li) & (li > -1)).any(0)
            got = mask_iou_suppress(masks, last, thr, reverse)
            assert torch.equal(got, want), (thr, reverse, got.tolist(), want.tolist())


@pytest.mark.parametrize("B,W,r", [(128, 4, 2), (8, 1, 0), (700, 2, 1), (3, 3, 0)])
def test_siglip_loss_epilogue_matches_logsigmoid_sum(B, W, r):
    import torch.nn.functional as F

    from parallelkernelbench_b200.ops.wild import siglip_loss_from_products

    g = torch.Generator(device="cuda").manual_seed(B * 7 + W)
    prod = torch.randn(B, W * B, device="cuda", generator=g) * 0.6
    scale, bias = 10.0, -10.0
    logits = (scale * prod.double() + bias)
    sign = -torch.ones_like(logits)
    idx = torch.arange(B, device="cuda")
    sign[idx, r * B + idx] = 1.0
    want = -F.logsigmoid(sign * logits).sum() / B
    got = siglip_loss_from_products(prod, scale, bias, r * B)
    torch.testing.assert_close(got.double(), want, atol=1e-5, rtol=2e-5)
    assert torch.equal(got, siglip_loss_from_products(prod, scale, bias, r * B))
