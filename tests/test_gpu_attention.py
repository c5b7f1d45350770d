"""tcgen05 flash attention forward against a plain fp32 PyTorch restatement."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, q_pos, kv_pos, causal, scale):
    """q [B,Sq,Hq,D], k/v [B,Skv,Hkv,D]; positions are 1-D tensors of global positions."""
    B, Sq, Hq, D = q.shape
    Hkv = k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, dim=1)
    s = torch.einsum("bhqd,bhkd->bhqk", qf, kf) * scale
    if causal:
        mask = kv_pos[None, :] > q_pos[:, None]
        s = s.masked_fill(mask[None, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p)
    return torch.einsum("bhqk,bhkd->bhqd", p, vf).permute(0, 2, 1, 3), lse


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [128, 384, 300])
def test_flash_attention_matches_reference(D, causal, S):
    from parallelkernelbench_b200.ops.attention import flash_attn_fwd

    B, Hq, Hkv = 2, 8, 2
    g = torch.Generator(device="cuda").manual_seed(S + D)
    q = torch.randn(B, S, Hq, D, device="cuda", dtype=torch.bfloat16, generator=g)
    k = torch.randn(B, S, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    v = torch.randn(B, S, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    out, lse = flash_attn_fwd(q, k, v, causal=causal)
    pos = torch.arange(S, device="cuda")
    ref, ref_lse = _ref(q, k, v, pos, pos, causal, 1.0 / math.sqrt(D))
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(lse, ref_lse, atol=2e-2, rtol=1e-3)


def test_flash_attention_segments_model_a_zigzag_rank():
    """Rank 1 of 4 in a zigzag layout: q chunks 1 and 6 (of 8), KV buffer holding all 8 chunks in rank order."""
    from parallelkernelbench_b200.ops.attention import flash_attn_fwd

    C, W, r, Hq, Hkv, D = 256, 4, 1, 4, 2, 128
    g = torch.Generator(device="cuda").manual_seed(11)
    full_q = torch.randn(1, 2 * W * C, Hq, D, device="cuda", dtype=torch.bfloat16, generator=g)
    full_k = torch.randn(1, 2 * W * C, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    full_v = torch.randn(1, 2 * W * C, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    chunks = lambda t, idx: torch.cat([t[:, c * C:(c + 1) * C] for c in idx], dim=1).contiguous()  # noqa: E731
    q = chunks(full_q, [r, 2 * W - 1 - r])
    order = [c for rr in range(W) for c in (rr, 2 * W - 1 - rr)]          # buffer layout: rank-major, two chunks each
    k, v = chunks(full_k, order), chunks(full_v, order)
    out, lse = flash_attn_fwd(q, k, v, causal=True, q_segments=[(C, r * C), (C, (2 * W - 1 - r) * C)],
                              kv_segments=[(i * C, c * C, C) for i, c in enumerate(order)])
    pos = torch.arange(2 * W * C, device="cuda")
    ref, ref_lse = _ref(full_q, full_k, full_v, pos, pos, True, 1.0 / math.sqrt(D))
    ref = chunks(ref, [r, 2 * W - 1 - r])
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
    assert torch.equal(out, flash_attn_fwd(q, k, v, causal=True, q_segments=[(C, r * C), (C, (2 * W - 1 - r) * C)],
                                           kv_segments=[(i * C, c * C, C) for i, c in enumerate(order)])[0])


@pytest.mark.parametrize("case", [
    dict(B=1, sq=256, skv=256, hq=4, hkv=2, D=128, causal=False),
    dict(B=1, sq=256, skv=256, hq=4, hkv=2, D=128, causal=True),
    dict(B=2, sq=384, skv=384, hq=2, hkv=2, D=64, causal=True),
    dict(B=1, sq=200, skv=333, hq=3, hkv=1, D=128, causal=False),
    dict(B=1, sq=1024, skv=1024, hq=8, hkv=2, D=128, causal=True),
])
def test_flash_attention_backward_matches_fp32_reference(case):
    """dq, dk, dv of the tcgen05 backward kernel against the explicit fp32 formula, from the forward kernel's own out / lse."""
    from parallelkernelbench_b200.ops.attention import flash_attn_bwd, flash_attn_fwd
    from parallelkernelbench_b200.refs.attention import attention_bwd_positions_ref

    B, sq, skv, hq, hkv, D, causal = (case[k] for k in ("B", "sq", "skv", "hq", "hkv", "D", "causal"))
    torch.manual_seed(3)
    q = torch.randn(B, sq, hq, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, skv, hkv, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, skv, hkv, D, device="cuda", dtype=torch.bfloat16)
    dout = torch.randn(B, sq, hq, D, device="cuda", dtype=torch.bfloat16)
    out, lse = flash_attn_fwd(q, k, v, causal=causal)
    dq, dk, dv = flash_attn_bwd(q, k, v, out, lse, dout, causal=causal)
    torch.cuda.synchronize()
    q_pos, kv_pos = torch.arange(sq, device="cuda"), torch.arange(skv, device="cuda")
    for b in range(B):
        rq, rk, rv = attention_bwd_positions_ref(q[b], k[b], v[b], out[b], lse[b], dout[b], q_pos, kv_pos, causal, D ** -0.5)
        for name, got, ref in (("dq", dq[b], rq), ("dk", dk[b], rk), ("dv", dv[b], rv)):
            err = (got - ref).abs().max().item()
            tol = 2e-2 * max(ref.abs().max().item(), 1.0)
            assert err <= tol, f"{name} batch {b}: max err {err} > {tol} ({case})"


def test_flash_attention_backward_zigzag_segments():
    """Two query runs at far-apart global positions and KV segments in a permuted buffer order (context-parallel layout)."""
    from parallelkernelbench_b200.ops.attention import flash_attn_bwd, flash_attn_fwd
    from parallelkernelbench_b200.refs.attention import attention_bwd_positions_ref

    torch.manual_seed(4)
    C, hq, hkv, D = 128, 4, 2, 128
    q_segs = [(C, 1 * C), (C, 6 * C)]                                      # rank 1 of 4 in the zigzag layout
    kv_segs = [(0, 1 * C, C), (C, 6 * C, C), (2 * C, 0, C), (3 * C, 7 * C, C), (4 * C, 2 * C, C), (5 * C, 5 * C, C),
               (6 * C, 3 * C, C), (7 * C, 4 * C, C)]
    q = torch.randn(1, 2 * C, hq, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, 8 * C, hkv, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(1, 8 * C, hkv, D, device="cuda", dtype=torch.bfloat16)
    dout = torch.randn(1, 2 * C, hq, D, device="cuda", dtype=torch.bfloat16)
    out, lse = flash_attn_fwd(q, k, v, causal=True, q_segments=q_segs, kv_segments=kv_segs)
    dq, dk, dv = flash_attn_bwd(q, k, v, out, lse, dout, causal=True, q_segments=q_segs, kv_segments=kv_segs)
    q_pos = torch.cat([torch.arange(p, p + r, device="cuda") for r, p in q_segs])
    kv_pos = torch.cat([torch.arange(p, p + n, device="cuda") for _, p, n in kv_segs])
    rq, rk, rv = attention_bwd_positions_ref(q[0], k[0], v[0], out[0], lse[0], dout[0], q_pos, kv_pos, True, D ** -0.5)
    for name, got, ref in (("dq", dq[0], rq), ("dk", dk[0], rk), ("dv", dv[0], rv)):
        err = (got - ref).abs().max().item()
        assert err <= 2e-2 * max(ref.abs().max().item(), 1.0), f"{name}: {err}"


@pytest.mark.parametrize("variant", ["PKB_FA_V3=0", "PKB_FA_V4=1", "PKB_FA_V4=1,PKB_FA_POLY=0", "PKB_FA_OPT=3", "PKB_FA_OPT=5", "PKB_FA_OPT=9"])
def test_forward_variants_pass_the_same_checks(variant):
    """The forward kernel variants are selected by an environment variable that is read once per process, so the forward
    checks of this file are repeated in a child process with the variable set."""
    import os
    import subprocess
    import sys

    extra = dict(item.split("=") for item in variant.split(","))
    if all(os.environ.get(k) == v for k, v in extra.items()):
        pytest.skip("already running under the variant")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.abspath(__file__), "-x", "-q", "-k", "matches_reference or zigzag_rank"],
                       cwd=root, capture_output=True, text=True, timeout=900, env={**os.environ, **extra})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-1500:]
