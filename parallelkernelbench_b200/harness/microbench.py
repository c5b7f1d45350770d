"""Single-GPU kernel timings against the library kernel for the same work.

    python -m parallelkernelbench_b200.harness.microbench <case> [<case> ...] [--iters N] [--warmup W] [--json FILE]

Every case times one of our kernels and, where a library kernel for the same arithmetic exists, that kernel too
(cuBLAS through ``torch.matmul``, the fused attention behind ``scaled_dot_product_attention``), with the same protocol:
``warmup`` untimed calls, then ``iters`` calls each bracketed by its own pair of CUDA events with a write of a buffer
larger than L2 between calls (so no call finds its inputs cached), mean and minimum reported. One JSON line per case:
``{"case", "ours_ms", "lib_ms", "ours_tflops", "lib_tflops", "ratio_vs_lib", ...}`` with the fraction of the measured bf16
peak where the case is a contraction.

Cases: ``gemm`` (8192^3 bf16), ``gemm_bwd`` (dX and dW of a 4096 x 4096 x 14336 linear layer), ``fa_fwd`` / ``fa_bwd`` (sequence 16384, causal, 32 query / 8 KV heads, head dim 128),
``fa_fwd_4k``, ``grouped_bf16`` / ``grouped_fp8`` (32 experts x 2048 rows, 7168 -> 4096 gate/up with SwiGLU: the expert GEMM of
the 256-expert MoE configuration per rank), ``rmsnorm``, ``fp8_quant``, ``kalman`` and ``sinkhorn`` (fp64 block Kalman step and
Sinkhorn-Knopp normalisation, each on a 256 MiB operand, against the library-op forms of the same formulas).
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch


class _Timer:
    def __init__(self, warmup: int, iters: int):
        self.warmup, self.iters = warmup, iters
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")       # 2x the 126 MB L2

    def __call__(self, fn) -> dict:
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        ms = []
        for _ in range(self.iters):
            self.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ms.append(e0.elapsed_time(e1))
        return {"mean_ms": sum(ms) / len(ms), "min_ms": min(ms)}


def _peaks() -> dict:
    from ..utils.env import measured_peaks

    return measured_peaks()


def _line(case: str, ours: dict, lib: dict | None, flops: float = 0.0, bytes_moved: float = 0.0, **extra) -> dict:
    out = {"case": case, "ours_ms": ours["mean_ms"], "ours_min_ms": ours["min_ms"]}
    if lib is not None:
        out.update({"lib_ms": lib["mean_ms"], "lib_min_ms": lib["min_ms"], "ratio_vs_lib": lib["mean_ms"] / ours["mean_ms"]})
    pk = _peaks()
    if flops:
        out["ours_tflops"] = flops / (ours["mean_ms"] * 1e-3) / 1e12
        if lib is not None:
            out["lib_tflops"] = flops / (lib["mean_ms"] * 1e-3) / 1e12
        if pk.get("bf16_tflops"):
            out["frac_of_measured_bf16_burst_peak"] = out["ours_tflops"] / float(pk["bf16_tflops"])
    if bytes_moved:
        out["ours_gbs"] = bytes_moved / (ours["mean_ms"] * 1e-3) / 1e9
        if pk.get("hbm_gbs"):
            out["frac_of_measured_copy_bandwidth"] = out["ours_gbs"] / float(pk["hbm_gbs"])
    out.update(extra)
    return out


def case_gemm(t: _Timer) -> dict:
    from ..ops import gemm_bf16

    n = 8192
    a = torch.randn(n, n, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, n, device="cuda", dtype=torch.bfloat16) * 0.02
    out = torch.empty(n, n, device="cuda", dtype=torch.bfloat16)
    ours = t(lambda: gemm_bf16(a, w, out=out))
    wt = w.t()
    lib = t(lambda: torch.matmul(a, wt, out=out))
    return _line("gemm", ours, lib, flops=2.0 * n ** 3, shape=[n, n, n])


def case_gemm_bwd(t: _Timer) -> dict:
    """The two backward layouts of a linear layer at Llama-8B MLP size: dX = dY @ W (B given [K, N]) and dW = dY^T @ X."""
    from ..ops import gemm_bf16_kn, gemm_bf16_tn

    tokens, n_in, n_out = 4096, 4096, 14336
    dy = torch.randn(tokens, n_out, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n_out, n_in, device="cuda", dtype=torch.bfloat16) * 0.02
    x = torch.randn(tokens, n_in, device="cuda", dtype=torch.bfloat16)
    dx = torch.empty(tokens, n_in, device="cuda", dtype=torch.bfloat16)
    dw = torch.empty(n_out, n_in, device="cuda", dtype=torch.float32)
    ours_dx = t(lambda: gemm_bf16_kn(dy, w, out=dx))
    lib_dx = t(lambda: torch.matmul(dy, w, out=dx))
    ours_dw = t(lambda: gemm_bf16_tn(dy, x, out=dw))
    dwb = torch.empty(n_out, n_in, device="cuda", dtype=torch.bfloat16)
    lib_dw = t(lambda: torch.matmul(dy.t(), x, out=dwb))
    fl = 2.0 * tokens * n_in * n_out
    out = _line("gemm_bwd_dx", ours_dx, lib_dx, flops=fl, shape=[tokens, n_in, n_out])
    out["dw"] = _line("gemm_bwd_dw", ours_dw, lib_dw, flops=fl, note="ours writes fp32, the library call bf16")
    return out


def _attn_inputs(S, hq=32, hkv=8, d=128):
    g = torch.Generator(device="cuda").manual_seed(1)
    mk = lambda h: torch.randn(1, S, h, d, device="cuda", dtype=torch.bfloat16, generator=g)  # noqa: E731
    return mk(hq), mk(hkv), mk(hkv), mk(hq)


def _fa_fwd(t: _Timer, S: int, name: str) -> dict:
    import torch.nn.functional as F

    from ..ops.attention import flash_attn_fwd

    q, k, v, _ = _attn_inputs(S)
    ours = t(lambda: flash_attn_fwd(q, k, v, causal=True))
    qt, kt, vt = (x.transpose(1, 2) for x in (q, k, v))            # [B, H, S, D] views: the layout the library call takes
    lib = t(lambda: F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=True))
    o_ours = flash_attn_fwd(q, k, v, causal=True)[0]
    o_lib = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=True).transpose(1, 2)
    err = float((o_ours.float() - o_lib.float()).abs().max())
    flops = 4.0 * S * S * 32 * 128 / 2                               # causal: half of the score matrix
    return _line(name, ours, lib, flops=flops, seq=S, heads="32/8", head_dim=128, max_abs_diff_vs_lib=err)


def case_fa_fwd(t):
    return _fa_fwd(t, 16384, "fa_fwd")


def case_fa_fwd_4k(t):
    return _fa_fwd(t, 4096, "fa_fwd_4k")


def case_umma_rate(t: _Timer) -> dict:
    """SM cycles per ``tcgen05.mma`` (M = 128, K = 16, bf16) by operand form, one issuing thread, 512 products in a row; with
    one CTA alone on the GPU and with one CTA on every SM. Nominal: 64 cycles at N = 128, 32 at N = 64, 128 at N = 256."""
    import ctypes

    from .. import _native as nv

    forms = {0: "ss_n128", 1: "ss_n64", 2: "ss_n256", 3: "ts_bmn_n128", 4: "ss_bmn_n128", 5: "ts_n128", 6: "ts_bmn_n64",
             7: "ss_n128_two_accumulators"}
    out: dict = {"case": "umma_rate", "mmas": 512}
    for ctas in (1, 148):
        res = {}
        for form, name in forms.items():
            buf = torch.zeros(ctas, dtype=torch.int64, device="cuda")
            for _ in range(2):
                nv.check(nv.cuda_lib().pkb_umma_rate(form, 512, ctas, nv.ptr(buf), nv.current_stream()), "pkb_umma_rate")
            torch.cuda.synchronize()
            nv.raise_on_status(sync=True)
            res[name] = round(float(buf.double().median()) / 512, 1)
        out[f"cycles_per_mma_{ctas}cta"] = res
    return out


def case_fa_trace(t: _Timer) -> dict:
    """Device-side timeline of the attention forward's longest CTA: the roles stamp ``clock64`` at every hand-over, and the
    medians of the intervals between consecutive stamps (over the unmasked KV tiles) say which hand-over the chain waits on.
    Roles: 0 MMA issuer, 1 / 2 softmax of Q tile 0 / 1 (first warp), 3 correction. Cycles of the SM clock."""
    from ..ops.attention import flash_attn_fwd

    q, k, v, _ = _attn_inputs(16384)
    flash_attn_fwd(q, k, v, causal=True)
    tiles_cap = 160                                                     # kFaTraceTiles of the kernel
    trace = torch.zeros(4 + 4 * tiles_cap * 8, dtype=torch.int64, device="cuda")
    flash_attn_fwd(q, k, v, causal=True, trace=trace)
    torch.cuda.synchronize()
    slots = trace[4:].view(4, tiles_cap, 8).cpu().tolist()
    by_role: dict[int, dict[int, dict[int, int]]] = {}
    flagged: dict = {}                                                  # stamps whose flag bit is set, tiles 8..99
    n = 0
    for role in range(4):
        for tile in range(tiles_cap):
            for ev in range(8):
                if slots[role][tile][ev]:
                    by_role.setdefault(role, {}).setdefault(tile, {})[ev] = slots[role][tile][ev] & ((1 << 62) - 1)
                    if slots[role][tile][ev] >> 62 and 8 <= tile < 100:
                        flagged[(role, ev)] = flagged.get((role, ev), 0) + 1
                    n += 1
    out: dict = {"case": "fa_trace", "records": n, "flagged_of_92": {f"role{r}_e{e}": c for (r, e), c in sorted(flagged.items())}}
    for role, tiles in sorted(by_role.items()):
        idx = sorted(tiles)
        steady = [i for i in idx if 8 <= i < 100 and i + 1 in tiles]
        evs = sorted({e for i in steady for e in tiles[i]})
        if steady:                                                     # order the events by their time inside a step
            ref = steady[len(steady) // 2]
            evs = sorted((e for e in evs if e in tiles[ref]), key=lambda e: tiles[ref][e])
        med = lambda xs: sorted(xs)[len(xs) // 2] if xs else None  # noqa: E731
        row = {"period": med([tiles[i + 1][evs[0]] - tiles[i][evs[0]] for i in steady if evs and evs[0] in tiles[i] and evs[0] in tiles[i + 1]])}
        for a, b in zip(evs, evs[1:]):
            row[f"e{a}->e{b}"] = med([tiles[i][b] - tiles[i][a] for i in steady if a in tiles[i] and b in tiles[i]])
        if evs:
            row[f"e{evs[-1]}->next e{evs[0]}"] = med([tiles[i + 1][evs[0]] - tiles[i][evs[-1]] for i in steady if evs[-1] in tiles[i] and evs[0] in tiles[i + 1]])
        out[f"role{role}"] = row
    # offset between the two softmax roles at the same tile index (are the Q tiles half a period apart?)
    if 1 in by_role and 2 in by_role:
        offs = [by_role[2][i][0] - by_role[1][i][0] for i in by_role[1] if 8 <= i < 100 and i in by_role[2] and 0 in by_role[1][i] and 0 in by_role[2][i]]
        out["softmax1_minus_softmax0_at_s_ready"] = sorted(offs)[len(offs) // 2] if offs else None
    # hand-overs between roles: P written -> P V issued (the issuer handles tile j's P V in its iteration j + 1), and
    # S issued -> S seen complete by the softmax warp
    def cross(ra, ea, rb, eb, shift):
        xs = [by_role[rb][i + shift][eb] - by_role[ra][i][ea] for i in by_role.get(ra, {})
              if 8 <= i < 100 and ea in by_role[ra][i] and (i + shift) in by_role.get(rb, {}) and eb in by_role[rb][i + shift]]
        return sorted(xs)[len(xs) // 2] if xs else None
    last = max(by_role.get(1, {}).get(10, {0: 0}))                   # the last softmax event: all of P is published
    out["handover"] = {"p0_written->pv0_issued": cross(1, last, 0, 2, 1), "s0_issued->s0_seen": cross(0, 3, 1, 0, 0),
                       "p1_written->pv1_issued": cross(2, last, 0, 4, 1), "s1_issued->s1_seen": cross(0, 5, 2, 0, 0)}
    return out


def case_fa_bwd_trace(t: _Timer) -> dict:
    """Device-side timeline of the attention backward's heaviest CTA (the first KV tile, which every query tile sees): medians
    of the intervals between consecutive stamps of each role over the steady steps, in SM cycles. Roles: 0 issuing warp
    (0 step start, 1 Q/dO landed, 2 dQ drained, 3 S and dP issued, 4 P and dS in shared memory, 5 dV and dK issued, 6 dQ issued),
    1 P / dS warps (0 start, 1 S and dP complete, 2 previous P/dS consumed, 3 computed, 4 published), 2 dQ drain warps
    (0 start, 1 dQ complete, 2 drained)."""
    from .. import _native as nv
    from ..ops.attention import flash_attn_bwd, flash_attn_fwd

    q, k, v, do = _attn_inputs(16384)
    out, lse = flash_attn_fwd(q, k, v, causal=True)
    flash_attn_bwd(q, k, v, out, lse, do, causal=True)
    steps_cap = 160
    trace = torch.zeros(3 * steps_cap * 8, dtype=torch.int64, device="cuda")
    nv.check(nv.cuda_lib().pkb_flash_attn_bwd_set_trace(nv.ptr(trace)), "pkb_flash_attn_bwd_set_trace")
    try:
        flash_attn_bwd(q, k, v, out, lse, do, causal=True)
        torch.cuda.synchronize()
    finally:
        nv.check(nv.cuda_lib().pkb_flash_attn_bwd_set_trace(None), "pkb_flash_attn_bwd_set_trace")
    slots = trace.view(3, steps_cap, 8).cpu().tolist()
    res: dict = {"case": "fa_bwd_trace"}
    med = lambda xs: sorted(xs)[len(xs) // 2] if xs else None  # noqa: E731
    for role in range(3):
        steps = {i: {e: c for e, c in enumerate(slots[role][i]) if c} for i in range(steps_cap)}
        steady = [i for i in range(8, 100) if steps[i] and steps.get(i + 1)]
        if not steady:
            continue
        ref = steady[len(steady) // 2]
        evs = sorted(steps[ref], key=lambda e: steps[ref][e])
        row = {"period": med([steps[i + 1][evs[0]] - steps[i][evs[0]] for i in steady if evs[0] in steps[i] and evs[0] in steps[i + 1]])}
        for a, b in zip(evs, evs[1:]):
            row[f"e{a}->e{b}"] = med([steps[i][b] - steps[i][a] for i in steady if a in steps[i] and b in steps[i]])
        row[f"e{evs[-1]}->next e{evs[0]}"] = med([steps[i + 1][evs[0]] - steps[i][evs[-1]] for i in steady if evs[-1] in steps[i] and evs[0] in steps[i + 1]])
        res[f"role{role}"] = row
    return res


def case_fa_bwd(t: _Timer) -> dict:
    import torch.nn.functional as F

    from ..ops.attention import flash_attn_bwd, flash_attn_fwd

    S = 16384
    q, k, v, do = _attn_inputs(S)
    out, lse = flash_attn_fwd(q, k, v, causal=True)
    ours = t(lambda: flash_attn_bwd(q, k, v, out, lse, do, causal=True))
    qt, kt, vt = (x.transpose(1, 2).detach().requires_grad_(True) for x in (q, k, v))
    dot = do.transpose(1, 2)

    def lib_step():
        with torch.enable_grad():
            o = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=True)
        return o

    o = lib_step()

    def lib_bwd():
        torch.autograd.grad(o, (qt, kt, vt), dot, retain_graph=True)

    lib = t(lib_bwd)
    flops = 10.0 * S * S * 32 * 128 / 2
    return _line("fa_bwd", ours, lib, flops=flops, seq=S, heads="32/8", head_dim=128)


def _grouped_shapes():
    G, rows, H, I2 = 32, 2048, 7168, 4096
    offs = (torch.arange(G + 1, dtype=torch.int32) * rows).cuda()
    return G, rows, H, I2, offs


def case_grouped_bf16(t: _Timer) -> dict:
    from ..ops.moe import grouped_gemm

    G, rows, H, I2, offs = _grouped_shapes()
    a = torch.randn(G * rows, H, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(G, I2, H, device="cuda", dtype=torch.bfloat16) * 0.02
    out = torch.empty(G * rows, I2 // 2, device="cuda", dtype=torch.bfloat16)
    ours = t(lambda: grouped_gemm(a, w, offs, epilogue="swiglu", out=out))
    return _line("grouped_bf16", ours, None, flops=2.0 * G * rows * H * I2, groups=G, rows_per_group=rows, k=H, n=I2)


def case_grouped_fp8(t: _Timer) -> dict:
    from ..ops.gemm_fp8 import gemm_fp8_blockscaled
    from ..refs.gemm_fp8 import quantize_rows_1x128, quantize_weight_128x128

    G, rows, H, I2, offs = _grouped_shapes()
    a8, sa = quantize_rows_1x128(torch.randn(G * rows, H, device="cuda"))
    w8, sb = quantize_weight_128x128(torch.randn(G, I2, H, device="cuda") * 0.02)
    out = torch.empty(G * rows, I2 // 2, device="cuda", dtype=torch.uint8)
    osc = torch.empty(G * rows, I2 // 256, device="cuda", dtype=torch.float32)
    ours = t(lambda: gemm_fp8_blockscaled(a8, sa, w8, sb, offsets=offs, epilogue="swiglu_quant", out=out, out_scales=osc))
    return _line("grouped_fp8", ours, None, flops=2.0 * G * rows * H * I2, groups=G, rows_per_group=rows, k=H, n=I2,
                 note="e4m3 operands, fp32 1x128 / 128x128 scales, SwiGLU + 1x128 re-quantise epilogue")


def case_rmsnorm(t: _Timer) -> dict:
    from ..ops import rmsnorm

    x = torch.randn(16384, 8192, device="cuda", dtype=torch.bfloat16)
    g = torch.ones(8192, device="cuda", dtype=torch.bfloat16)
    ours = t(lambda: rmsnorm(x, g))
    lib = t(lambda: torch.nn.functional.rms_norm(x, (8192,), g, 1e-6))
    return _line("rmsnorm", ours, lib, bytes_moved=2.0 * x.numel() * 2)


def case_fp8_quant(t: _Timer) -> dict:
    from ..ops import fp8_quantize_1x128

    x = torch.randn(16384, 8192, device="cuda", dtype=torch.bfloat16)
    ours = t(lambda: fp8_quantize_1x128(x))
    return _line("fp8_quant", ours, None, bytes_moved=x.numel() * (2 + 1 + 4 / 128))


def case_kalman(t: _Timer) -> dict:
    """Block Kalman-filter step in fp64, 32 blocks of 1024 x 1024 (a 256 MiB covariance, twice the L2): our three launches
    (P read twice, written once) against the same formulas as library products (reference/63_deepmd_kalman_filter_optimizer.py)."""
    from ..ops.wild import kalman_block_step

    nb, n, lam = 32, 1024, 0.98
    H = torch.randn(nb, n, 1, dtype=torch.float64, device="cuda") * 0.01
    w = torch.randn(nb, n, 1, dtype=torch.float64, device="cuda")
    P = torch.eye(n, dtype=torch.float64, device="cuda").repeat(nb, 1, 1) + 0.01 * torch.randn(nb, n, n, dtype=torch.float64, device="cuda")
    err = torch.randn(1, dtype=torch.float64, device="cuda")

    def lib_step():
        K = torch.bmm(P, H)
        A = 1.0 / (lam + torch.bmm(H.transpose(1, 2), K)).sum().reshape(1)
        return w + A * err * K, (1.0 / lam) * (P - A * torch.bmm(K, K.transpose(1, 2)))

    ours = t(lambda: kalman_block_step(H, err, w, P, lam))
    lib = t(lib_step)
    return _line("kalman", ours, lib, bytes_moved=3.0 * P.numel() * 8)


def case_sinkhorn(t: _Timer) -> dict:
    """Sinkhorn-Knopp, 4096 samples x 16384 prototypes fp32 (256 MiB), three iterations: our scale-vector form (nine passes
    over the logits: one for the mass, two per iteration, one read and one write for the result) against the matrix-rewriting
    form of reference/80_dinov2_distributed_sinkhorn_knopp.py."""
    from ..ops.wild import sinkhorn_knopp

    B, Pn, temp, iters = 4096, 16384, 0.07, 3
    x = torch.randn(B, Pn, device="cuda") * 0.01

    def lib_form():
        q = torch.exp(x / temp).T.contiguous()
        q /= q.sum()
        for _ in range(iters):
            q /= q.sum(dim=1, keepdim=True)
            q /= Pn
            q /= q.sum(dim=0, keepdim=True)
            q /= B
        q *= B
        return q.T.contiguous()

    ours = t(lambda: sinkhorn_knopp(x, temp, iters))
    lib = t(lib_form)
    return _line("sinkhorn", ours, lib, bytes_moved=(3.0 + 2 * iters) * x.numel() * 4)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("cases", nargs="+")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--json", default=None, help="append the result lines to this file as well")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("microbench needs a GPU", file=sys.stderr)
        return 2
    from .. import _native as nv

    t = _Timer(max(3, a.warmup), a.iters)
    rc = 0
    for name in a.cases:
        fn = globals().get("case_" + name)
        if fn is None:
            print(f"unknown case {name}", file=sys.stderr)
            rc = 2
            continue
        res = fn(t)
        nv.raise_on_status(sync=True)
        res = {k: (round(v, 5) if isinstance(v, float) and math.isfinite(v) else v) for k, v in res.items()}
        line = json.dumps(res)
        print(line, flush=True)
        if a.json:
            with open(a.json, "a") as fh:
                fh.write(line + "\n")
    return rc


if __name__ == "__main__":
    sys.exit(main())
