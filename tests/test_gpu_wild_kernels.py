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
