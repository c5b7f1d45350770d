"""Runs the flash-attention forward on a fixed set of seeded problems and saves outputs and log-sum-exps to the file given as
argv[1]. Kernel variants are selected by environment variables read once per process, so a test runs this script once per
variant and compares the files."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from parallelkernelbench_b200 import _native as nv  # noqa: E402
from parallelkernelbench_b200.ops.attention import flash_attn_fwd  # noqa: E402


def main() -> int:
    out = {}
    g = torch.Generator(device="cuda").manual_seed(7)
    cases = [(1, 1024, 1024, 8, 2, 128, True), (2, 512, 512, 4, 4, 64, False), (1, 2048, 2048, 4, 1, 128, True),
             (1, 768, 1280, 4, 2, 128, False)]
    for i, (B, sq, skv, hq, hkv, D, causal) in enumerate(cases):
        q = torch.randn(B, sq, hq, D, device="cuda", generator=g).to(torch.bfloat16)
        k = torch.randn(B, skv, hkv, D, device="cuda", generator=g).to(torch.bfloat16)
        v = torch.randn(B, skv, hkv, D, device="cuda", generator=g).to(torch.bfloat16)
        # rows whose scores grow sharply late in the walk make the running offset move after the first tile
        k[:, skv // 2:] *= 3.0
        o, lse = flash_attn_fwd(q, k, v, causal=causal and sq == skv)
        out[f"o{i}"], out[f"lse{i}"] = o.cpu(), lse.cpu()
    # a zigzag rank: two query runs against four KV segments in ring order
    S, Wn, hq, hkv, D = 256, 2, 4, 2, 128
    q = torch.randn(1, 2 * S, hq, D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(1, 4 * S, hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(1, 4 * S, hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    o, lse = flash_attn_fwd(q, k, v, causal=True, q_segments=[(S, 1 * S), (S, 2 * S)],
                            kv_segments=[(0, 1 * S, S), (S, 2 * S, S), (2 * S, 0, S), (3 * S, 3 * S, S)])
    out["oz"], out["lsez"] = o.cpu(), lse.cpu()
    torch.cuda.synchronize()
    nv.raise_on_status(sync=True)
    torch.save(out, sys.argv[1])
    print("saved", len(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
