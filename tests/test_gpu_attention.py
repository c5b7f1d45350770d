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
