"""Tensor-parallel / sequence-parallel building blocks and the flagship TP-MLP block.

"ours" uses the tcgen05 GEMM, the fused gather/scatter GEMM kernels and the symmetric-heap
collectives on GPUs; on a CPU-only machine the same composition runs with PyTorch math over the
shared-memory transport, so the data flow is testable without a GPU.
Reference workloads covered: reference/9_layernorm_backward.py ... reference/18_tp_rms_norm.py,
reference/45_reducescatter_fused_rmsnorm.py, reference/46_gemv_decode.py, reference/48_fsdp_and_tp.py.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..harness.roofline import Cost
from .registry import OpSpec, RunCtx, register


def _mm(rc: RunCtx, a: torch.Tensor, b_kn: torch.Tensor, epilogue: str = "none", out_dtype=None) -> torch.Tensor:
    """``a[M,K] @ b_kn[K,N]`` on the tcgen05 GEMM (weights re-laid out K-major once and cached)."""
    if not rc.dist.is_cuda or a.dtype != torch.bfloat16:
        y = a.float() @ b_kn.float()
        if epilogue == "silu":
            y = F.silu(y)
        return y.to(out_dtype or a.dtype)
    from ..ops import gemm_bf16

    key = ("w_kmajor", b_kn.data_ptr(), tuple(b_kn.shape))
    w = rc.cache.get(key)
    if w is None:
        w = b_kn.t().contiguous()
        rc.cache[key] = w
    k = a.shape[1]
    if k % 8 != 0:      # TMA rows must be 16-byte multiples: pad K with zeros
        pad = 8 - k % 8
        a = F.pad(a, (0, pad))
        w = F.pad(w, (0, pad))
    return gemm_bf16(a.contiguous(), w, epilogue=epilogue, out_dtype=out_dtype or torch.bfloat16)


def _rms(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()).to(x.dtype)


# ---- 9: LayerNorm backward parameter gradients -------------------------------------------------
def _ln_inputs(rc, cfg):
    xh = rc.randn(cfg["m"], cfg["n"])
    xh = (xh.float() / (xh.float().norm(dim=-1, keepdim=True) + 1e-5)).to(rc.dtype)
    return (xh, rc.randn(cfg["m"], cfg["n"], salt=1))


def _ln_ref(rc, xh, dy):
    dbeta = dy.float().sum(0)
    dgamma = (dy.float() * xh.float()).sum(0)
    if rc.world > 1:
        dist.all_reduce(dbeta)
        dist.all_reduce(dgamma)
    return dgamma, dbeta


def _ln_ours(rc, xh, dy):
    if rc.dist.is_cuda:
        from ..ops import ln_bwd_colreduce

        dg, db = ln_bwd_colreduce(xh, dy)
    else:
        dg, db = (dy.float() * xh.float()).sum(0), dy.float().sum(0)
    packed = rc.comm.all_reduce(torch.stack([dg, db]))      # one packed exchange instead of two
    return packed[0], packed[1]


register(OpSpec(name="layernorm_backward", problem_ids=(9,), group="tp", configs={"default": {"m": 1024, "n": 1024}, "small": {"m": 64, "n": 96}},
                make_inputs=_ln_inputs, reference=_ln_ref, ours=_ln_ours, atol=2e-2, rtol=2e-2,
                cost=lambda cfg, W: Cost(hbm_bytes=2 * cfg["m"] * cfg["n"] * 2, nvlink_bytes=8 * cfg["n"] * (W - 1))))


# ---- 10: vocab-sharded embedding lookup --------------------------------------------------------
def _emb_inputs(rc, cfg):
    shard = rc.randn(cfg["m"], cfg["n"])
    idx = rc.randint(0, rc.world * cfg["m"], (cfg["m"],), salt=1)
    return (idx, shard)


def _emb_ref(rc, idx, shard):
    W, S = rc.world, shard.shape[0]
    if W == 1:
        return shard[idx]
    owner = idx // S
    order = torch.argsort(owner, stable=True)
    counts = torch.bincount(owner, minlength=W)
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts)
    send_ids = (idx[order] % S).contiguous()
    got_ids = torch.empty(int(recv_counts.sum()), dtype=idx.dtype, device=idx.device)
    dist.all_to_all_single(got_ids, send_ids, output_split_sizes=recv_counts.tolist(), input_split_sizes=counts.tolist())
    rows = shard[got_ids]
    back = torch.empty((idx.numel(), shard.shape[1]), dtype=shard.dtype, device=shard.device)
    dist.all_to_all_single(back, rows, output_split_sizes=counts.tolist(), input_split_sizes=recv_counts.tolist())
    out = torch.empty_like(back)
    out[order] = back
    return out


def _emb_ours(rc, idx, shard):
    # remote gather: every rank can read every shard, so the lookup needs no request/reply exchange
    W, S = rc.world, shard.shape[0]
    if W == 1:
        return shard[idx]
    if rc.dist.is_cuda:
        from ..ops.collectives import row_gather

        return row_gather(shard, idx, rc.comm.group())
    table = rc.comm.all_gather(shard).reshape(W * S, -1)
    return table[idx]


register(OpSpec(name="embedding_lookup", problem_ids=(10,), group="tp", configs={"default": {"m": 1024, "n": 1024}, "small": {"m": 32, "n": 16}},
                make_inputs=_emb_inputs, reference=_emb_ref, ours=_emb_ours,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (W - 1) / max(W, 1))))


# ---- 11 / 12: all-gather (along K) then GEMM ---------------------------------------------------
def _agk_inputs(rc, cfg):
    kl = cfg["k"] // rc.world
    return (rc.randn(cfg["m"], kl), rc.randn(kl * rc.world, cfg["n"], shared=True, salt=1))


def _agk_ref(rc, a_local, b):
    if rc.world > 1:
        parts = [torch.empty_like(a_local) for _ in range(rc.world)]
        dist.all_gather(parts, a_local.contiguous())
        a = torch.cat(parts, dim=1)
    else:
        a = a_local
    return a @ b


def _agk_ours(rc, a_local, b):
    a = rc.comm.all_gather_cat(a_local.contiguous(), dim=1) if rc.world > 1 else a_local
    return _mm(rc, a, b)


_GEMM_CFG = {"default": {"m": 1024, "n": 1024, "k": 512}, "small": {"m": 128, "n": 64, "k": 64}}
register(OpSpec(name="allgather_gemm", problem_ids=(11, 12), group="tp", configs=_GEMM_CFG, make_inputs=_agk_inputs,
                reference=_agk_ref, ours=_agk_ours, atol=0.5, rtol=2e-2,
                cost=lambda cfg, W: Cost(flops=2.0 * cfg["m"] * cfg["n"] * cfg["k"], nvlink_bytes=cfg["m"] * cfg["k"] * 2 * (W - 1) / max(W, 1))))


# ---- 13: row-parallel GEMM then all-reduce -----------------------------------------------------
def _gar_inputs(rc, cfg):
    return (rc.randn(cfg["m"], cfg["k"]), rc.randn(cfg["k"], cfg["n"], salt=1))


def _gar_ref(rc, a, b):
    c = a @ b
    if rc.world > 1:
        dist.all_reduce(c)
    return c


def _gar_ours(rc, a, b):
    """Two launches (tcgen05 GEMM, symmetric-heap all-reduce), or the single fused kernel when PKB_FUSED_GEMM_AR=1 and
    the shapes fit it (rows a multiple of 256 per rank, K and N multiples of 8)."""
    import os

    W, (M, K), N = rc.world, a.shape, b.shape[1]
    if (os.environ.get("PKB_FUSED_GEMM_AR") == "1" and rc.dist.is_cuda and a.dtype == torch.bfloat16 and M % (256 * W) == 0
            and K % 8 == 0 and N % 8 == 0):
        from ..ops.tp import GemmAllReduce

        key = ("gemm_ar", M, N)                   # one set of symmetric buffers per shape; the K-major weight per weight tensor
        if key not in rc.cache:
            rc.cache[key] = GemmAllReduce(rc.comm.group(), M // W, N)
        wkey = ("gemm_ar_w", b.data_ptr(), b._version)
        if wkey not in rc.cache:
            rc.cache[wkey] = b.t().contiguous()
        return rc.cache[key](a.contiguous(), rc.cache[wkey]).clone()
    return rc.comm.all_reduce(_mm(rc, a, b))


register(OpSpec(name="gemm_allreduce", problem_ids=(13,), group="tp", configs={**_GEMM_CFG, "large": {"m": 4096, "n": 8192, "k": 1024}},
                make_inputs=_gar_inputs, reference=_gar_ref, ours=_gar_ours, atol=1.0, rtol=3e-2,
                cost=lambda cfg, W: Cost(flops=2.0 * cfg["m"] * cfg["n"] * cfg["k"], nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (W - 1) / max(W, 1))))


# ---- 14: column-parallel GEMM then all-gather along N ------------------------------------------
def _gag_inputs(rc, cfg):
    return (rc.randn(cfg["m"], cfg["k"], shared=True), rc.randn(cfg["k"], cfg["n"] // rc.world, salt=1))


def _gag_ref(rc, a, b):
    c = a @ b
    if rc.world == 1:
        return c
    parts = [torch.empty_like(c) for _ in range(rc.world)]
    dist.all_gather(parts, c.contiguous())
    return torch.cat(parts, dim=1)


def _gag_ours(rc, a, b):
    """The single fused kernel (the GEMM's TMA-store epilogue writes every tile into the gathered result of every rank) when the
    shapes fit it (local N a multiple of 64, K a multiple of 8); PKB_FUSED_GEMM_AG=0 selects the two-launch form (tcgen05 GEMM,
    then the symmetric-heap all-gather). Measured on 2 GPUs at 4096 x 8192 x 1024: 0.112 ms fused, 0.146 ms two launches,
    0.193 ms cuBLAS + NCCL."""
    import os

    (M, K), nl = a.shape, b.shape[1]
    if os.environ.get("PKB_FUSED_GEMM_AG", "1") != "0" and rc.dist.is_cuda and a.dtype == torch.bfloat16 and nl % 64 == 0 and K % 8 == 0:
        from ..ops.tp import GemmAllGather

        key = ("gemm_ag", M, nl)
        if key not in rc.cache:
            rc.cache[key] = GemmAllGather(rc.comm.group(), M, nl)
        wkey = ("gemm_ag_w", b.data_ptr(), b._version)
        if wkey not in rc.cache:
            rc.cache[wkey] = b.t().contiguous()
        return rc.cache[key](a.contiguous(), rc.cache[wkey]).clone()
    return rc.comm.all_gather_cat(_mm(rc, a, b), dim=1) if rc.world > 1 else _mm(rc, a, b)


register(OpSpec(name="gemm_allgather", problem_ids=(14,), group="tp", configs={**_GEMM_CFG, "large": {"m": 4096, "n": 8192, "k": 1024}},
                make_inputs=_gag_inputs, reference=_gag_ref, ours=_gag_ours,
                atol=0.5, rtol=2e-2,
                cost=lambda cfg, W: Cost(flops=2.0 * cfg["m"] * cfg["n"] * cfg["k"] / W, nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (W - 1) / max(W, 1))))


# ---- 15: gather -> GEMM+SiLU -> GEMM on own rows -> reduce-scatter ------------------------------
def _comb_inputs(rc, cfg):
    W = rc.world
    m = (cfg["m"] + W - 1) // W * W
    h = (cfg["h"] + W - 1) // W * W
    return (rc.randn(m, h // W), rc.randn(h, cfg["f"], shared=True, salt=1, std=0.1), rc.randn(cfg["f"], h, shared=True, salt=2, std=0.1))


def _comb_ref(rc, x_local, w1, w2):
    W, r = rc.world, rc.rank
    m = x_local.shape[0]
    ml = m // W
    if W > 1:
        parts = [torch.empty_like(x_local) for _ in range(W)]
        dist.all_gather(parts, x_local.contiguous())
        x = torch.cat(parts, dim=1)
    else:
        x = x_local
    a = F.silu(x @ w1)
    blk = a[r * ml:(r + 1) * ml] @ w2
    if W == 1:
        return blk
    buf = blk.new_zeros((m, blk.shape[1]))
    buf[r * ml:(r + 1) * ml] = blk
    out = blk.new_empty((ml, blk.shape[1]))
    dist.reduce_scatter_tensor(out, buf)
    return out


def _comb_ours(rc, x_local, w1, w2):
    # every rank contributes zeros except for its own row block, so the reduce-scatter moves no
    # information: after the gather each rank computes exactly its own output rows.
    W, r = rc.world, rc.rank
    ml = x_local.shape[0] // W
    x_rows = rc.comm.all_gather_cat(x_local[r * ml:(r + 1) * ml].contiguous(), dim=1) if W > 1 else x_local
    if W > 1:
        # the row block this rank needs is spread over all ranks' column shards: gather those columns
        cols = rc.comm.all_gather(x_local.contiguous())           # [W, m, h/W]
        x_rows = torch.cat([cols[p, r * ml:(r + 1) * ml] for p in range(W)], dim=1)
    a = _mm(rc, x_rows, w1, epilogue="silu")
    return _mm(rc, a, w2)


register(OpSpec(name="combined_sharded_gemms", problem_ids=(15,), group="tp",
                configs={"default": {"m": 1024, "h": 256, "f": 512}, "small": {"m": 64, "h": 32, "f": 64}},
                make_inputs=_comb_inputs, reference=_comb_ref, ours=_comb_ours, atol=5e-2, rtol=3e-2,
                cost=lambda cfg, W: Cost(flops=4.0 * cfg["m"] / W * cfg["h"] * cfg["f"], nvlink_bytes=cfg["m"] * cfg["h"] * 2 * (W - 1) / max(W, 1))))


# ---- 16: K-sharded GEMM then reduce-scatter over rows ------------------------------------------
def _grs_inputs(rc, cfg):
    kl = cfg["k"] // rc.world
    return (rc.randn(cfg["m"], kl), rc.randn(kl, cfg["n"], salt=1))


def _grs_ref(rc, a, b):
    c = (a @ b).contiguous()
    if rc.world == 1:
        return c
    out = c.new_empty((c.shape[0] // rc.world, c.shape[1]))
    dist.reduce_scatter_tensor(out, c)
    return out


register(OpSpec(name="gemm_reducescatter", problem_ids=(16,), group="tp", configs=_GEMM_CFG, make_inputs=_grs_inputs,
                reference=_grs_ref, ours=lambda rc, a, b: rc.comm.reduce_scatter(_mm(rc, a, b)) if rc.world > 1 else _mm(rc, a, b),
                atol=0.5, rtol=3e-2,
                cost=lambda cfg, W: Cost(flops=2.0 * cfg["m"] * cfg["n"] * cfg["k"] / W, nvlink_bytes=cfg["m"] * cfg["n"] * 2 * (W - 1) / max(W, 1))))


# ---- 17: RoPE then all-gather along the sequence -----------------------------------------------
def _rope_inputs(rc, cfg):
    b, t, h, d = cfg["b"], max(1, cfg["t"] // rc.world), cfg["heads"], cfg["d"]
    return (rc.randn(b, t, h, d), rc.randn(b, t, h, d, salt=1), rc.randn(b, t, d, salt=2), rc.randn(b, t, d, salt=3))


def _rot(x, cos, sin):
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos.unsqueeze(-2) + rot * sin.unsqueeze(-2)


def _rope_ref(rc, q, k, cos, sin):
    qr, kr = _rot(q, cos, sin), _rot(k, cos, sin)
    if rc.world == 1:
        return qr, kr
    qs = [torch.empty_like(qr) for _ in range(rc.world)]
    ks = [torch.empty_like(kr) for _ in range(rc.world)]
    dist.all_gather(qs, qr.contiguous())
    dist.all_gather(ks, kr.contiguous())
    return torch.cat(qs, dim=1), torch.cat(ks, dim=1)


def _rope_ours(rc, q, k, cos, sin):
    import os

    if (rc.dist.is_cuda and rc.world > 1 and q.dtype == torch.bfloat16 and q.shape[-1] % 16 == 0
            and os.environ.get("PKB_UNFUSED_PUSH") != "1"):
        # rotate and gather in one launch: every rotated 16-byte piece is stored into the gathered q / k of all ranks
        from ..ops.fused_push import RopeAllGather

        b, t, hq, d = q.shape
        key = ("rope_ag", tuple(q.shape), tuple(k.shape))
        if key not in rc.cache:
            rc.cache[key] = RopeAllGather(rc.comm.group(), b, t, hq, k.shape[2], d)
        qg, kg = rc.cache[key](q, k, cos, sin)
        return qg.clone(), kg.clone()
    if rc.dist.is_cuda:
        from ..ops import rope

        qk = torch.stack([rope(q, cos, sin), rope(k, cos, sin)])
    else:
        qk = torch.stack([_rot(q, cos, sin), _rot(k, cos, sin)])
    if rc.world == 1:
        return qk[0], qk[1]
    g = rc.comm.all_gather(qk)                        # one gather for q and k: [W, 2, b, t, h, d]
    return torch.cat(list(g[:, 0].unbind(0)), dim=1), torch.cat(list(g[:, 1].unbind(0)), dim=1)


register(OpSpec(name="rope_allgather", problem_ids=(17,), group="tp",
                configs={"default": {"b": 16, "t": 16, "heads": 8, "d": 64}, "long": {"b": 1, "t": 32768, "heads": 32, "d": 128}},
                make_inputs=_rope_inputs, reference=_rope_ref, ours=_rope_ours, atol=3e-2, rtol=2e-2,
                # q and k of this rank's t / W positions go to every peer; every rank reads its shard and writes the gathered q, k
                cost=lambda cfg, W: Cost(nvlink_bytes=2.0 * cfg["b"] * max(1, cfg["t"] // W) * cfg["heads"] * cfg["d"] * 2 * (W - 1),
                                         hbm_bytes=2.0 * cfg["b"] * max(1, cfg["t"] // W) * cfg["heads"] * cfg["d"] * 2 * (1 + W))))


# ---- 18: RMSNorm over a TP-sharded hidden dimension ---------------------------------------------
def _tprms_ref(rc, x, w, eps):
    ss = x.float().pow(2).sum(-1, keepdim=True)
    if rc.world > 1:
        dist.all_reduce(ss)
    var = ss / (x.shape[-1] * rc.world)
    return (w.float() * (x.float() * torch.rsqrt(var + eps))).to(x.dtype)


def _tprms_ours(rc, x, w, eps):
    if rc.dist.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        from ..ops import tp_rmsnorm

        return tp_rmsnorm(x, w, eps, rc.comm.group())
    ss = rc.comm.all_reduce(x.float().pow(2).sum(-1, keepdim=True).contiguous())
    return (w.float() * (x.float() * torch.rsqrt(ss / (x.shape[-1] * rc.world) + eps))).to(x.dtype)


register(OpSpec(name="tp_rmsnorm", problem_ids=(18,), group="tp", configs={"default": {"m": 1024, "n": 1024}, "small": {"m": 16, "n": 64}},
                make_inputs=lambda rc, cfg: (rc.randn(cfg["m"], cfg["n"]), rc.randn(cfg["n"], salt=1), 1e-5),
                reference=_tprms_ref, ours=_tprms_ours, atol=3e-2, rtol=2e-2,
                cost=lambda cfg, W: Cost(hbm_bytes=2 * cfg["m"] * cfg["n"] * 2, nvlink_bytes=cfg["m"] * 4 * (W - 1))))


# ---- 45: reduce-scatter fused with RMSNorm -----------------------------------------------------
def _rsrms_inputs(rc, cfg):
    return (rc.randn(rc.world * cfg["rows"] * cfg["cols"]), rc.randn(cfg["cols"], shared=True, salt=1), 1e-6)


def _rsrms_ref(rc, flat, gamma, eps):
    W = rc.world
    out = flat.new_empty(flat.numel() // W)
    if W > 1:
        dist.reduce_scatter_tensor(out, flat.contiguous())
    else:
        out.copy_(flat)
    y = (out.float() / W).view(-1, gamma.numel())
    return _rms(y, gamma, eps).to(flat.dtype)


def _rsrms_ours(rc, flat, gamma, eps):
    W = rc.world
    cols = gamma.numel()
    if rc.dist.is_cuda and flat.dtype == torch.bfloat16 and cols % 8 == 0:
        from ..ops import sum_rmsnorm

        # every rank needs its chunk from all peers: all-to-all of chunks, then sum + RMSNorm in one kernel
        parts = rc.comm.all_to_all(flat.view(W, -1, cols).contiguous()) if W > 1 else flat.view(1, -1, cols)
        return sum_rmsnorm(parts.contiguous(), gamma, eps, scale=1.0 / W).view(-1, cols)
    y = rc.comm.reduce_scatter(flat.float().contiguous(), scale=1.0 / W) if W > 1 else flat.float()
    return _rms(y.view(-1, cols), gamma, eps).to(flat.dtype)


register(OpSpec(name="reducescatter_rmsnorm", problem_ids=(45,), group="tp",
                configs={"default": {"rows": 128, "cols": 128}, "large": {"rows": 2048, "cols": 8192}},
                make_inputs=_rsrms_inputs, reference=_rsrms_ref, ours=_rsrms_ours, atol=3e-2, rtol=2e-2,
                cost=lambda cfg, W: Cost(nvlink_bytes=cfg["rows"] * cfg["cols"] * 2 * (W - 1))))


# ---- 46: vocab-sharded LM-head GEMV (decode) then all-gather ------------------------------------
def _gemv_inputs(rc, cfg):
    return (rc.randn(1, cfg["hidden"], shared=True), rc.randn(cfg["vocab_local"], cfg["hidden"], salt=1, std=0.05), rc.randn(cfg["vocab_local"], salt=2))


def _gemv_ref(rc, h, w, b):
    y = (h @ w.t() + b).contiguous()
    if rc.world == 1:
        return y
    parts = [torch.empty_like(y) for _ in range(rc.world)]
    dist.all_gather(parts, y)
    return torch.cat(parts, dim=1)


def _gemv_ours(rc, h, w, b):
    import os

    if (os.environ.get("PKB_FUSED_GEMV_AG") == "1" and rc.dist.is_cuda and h.dtype == torch.bfloat16 and h.shape[0] in (1, 2, 4)
            and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0):
        from ..ops.tp import GemvAllGather

        key = ("gemv_ag", h.shape[0], w.shape[0])
        if key not in rc.cache:
            rc.cache[key] = GemvAllGather(rc.comm.group(), h.shape[0], w.shape[0])
        return rc.cache[key](h.contiguous(), w.contiguous(), b.contiguous()).clone()
    if rc.dist.is_cuda and h.dtype == torch.bfloat16:
        from ..ops import gemm_bf16

        y = gemm_bf16(h.contiguous(), w, bias=b.contiguous(), mode="single", block_n=128)
    else:
        y = (h.float() @ w.float().t() + b.float()).to(h.dtype)
    return rc.comm.all_gather_cat(y.contiguous(), dim=1) if rc.world > 1 else y


register(OpSpec(name="gemv_decode", problem_ids=(46,), group="tp",
                configs={"default": {"hidden": 1024, "vocab_local": 1024}, "llama": {"hidden": 4096, "vocab_local": 16032}},
                make_inputs=_gemv_inputs, reference=_gemv_ref, ours=_gemv_ours, atol=5e-2, rtol=2e-2,
                cost=lambda cfg, W: Cost(hbm_bytes=cfg["hidden"] * cfg["vocab_local"] * 2, flops=2.0 * cfg["hidden"] * cfg["vocab_local"])))


# ---- 48: 2-D mesh (TP x FSDP) SwiGLU MLP forward -------------------------------------------------
def _mesh48(rc):
    from ..parallel.mesh import Mesh2D, factor_two_level

    key = "mesh48"
    if key not in rc.cache:
        n_fsdp, n_tp = factor_two_level(rc.world, 2)
        rc.cache[key] = Mesh2D.build(rc.world, n_tp, rc.rank, inner_name="tp", outer_name="fsdp")
    return rc.cache[key]


def _fsdp_tp_inputs(rc, cfg):
    m = _mesh48(rc)
    n_tp, n_fsdp = m.inner, m.outer
    d, dff = cfg["d"], cfg["dff"]
    # full weights are identical everywhere (shared seed); each rank keeps its (fsdp, tp) shard
    w1 = rc.randn(dff, d, shared=True, salt=1, std=0.05)
    w2 = rc.randn(dff, d, shared=True, salt=2, std=0.05)
    w3 = rc.randn(d, dff, shared=True, salt=3, std=0.05)
    f_tp = dff // n_tp
    tp, fs = m.inner_rank, m.outer_rank
    rows = f_tp // n_fsdp
    w1s = w1[tp * f_tp + fs * rows: tp * f_tp + (fs + 1) * rows].contiguous()
    w2s = w2[tp * f_tp + fs * rows: tp * f_tp + (fs + 1) * rows].contiguous()
    w3s = w3[:, tp * f_tp + fs * rows: tp * f_tp + (fs + 1) * rows].contiguous()
    x = rc.randn(cfg["batch"], d, salt=10 + fs)      # the TP peers of one FSDP row see the same batch
    g = torch.Generator(device=rc.device).manual_seed(991 + fs + 1000 * rc.trial)
    x = torch.randn(cfg["batch"], d, device=rc.device, generator=g).to(rc.dtype)
    return (x, w1s, w2s, w3s, n_tp, n_fsdp)


def _fsdp_tp_ref(rc, x, w1s, w2s, w3s, n_tp, n_fsdp):
    m = _mesh48(rc)

    def ag(t, dim):
        if n_fsdp == 1:
            return t
        parts = [torch.empty_like(t) for _ in range(n_fsdp)]
        dist.all_gather(parts, t.contiguous(), group=m.outer_group)
        return torch.cat(parts, dim=dim)
    w1, w2, w3 = ag(w1s, 0), ag(w2s, 0), ag(w3s, 1)
    y = (F.silu(x @ w1.t()) * (x @ w2.t())) @ w3.t()
    if n_tp > 1:
        dist.all_reduce(y, group=m.inner_group)
    return y


def _fsdp_tp_ours(rc, x, w1s, w2s, w3s, n_tp, n_fsdp):
    m = _mesh48(rc)
    fs_g = rc.comm.group(m.outer_ranks)
    tp_g = rc.comm.group(m.inner_ranks)
    if n_fsdp > 1:
        w12 = rc.comm.all_gather(torch.stack([w1s, w2s]), fs_g)        # [F, 2, rows, d] in one exchange
        w1 = w12[:, 0].reshape(-1, w1s.shape[1])
        w2 = w12[:, 1].reshape(-1, w2s.shape[1])
        w3 = rc.comm.all_gather_cat(w3s.contiguous(), dim=1, group=fs_g)
    else:
        w1, w2, w3 = w1s, w2s, w3s
    if rc.dist.is_cuda and x.dtype == torch.bfloat16:
        from ..ops import gemm_bf16

        gate = gemm_bf16(x.contiguous(), w1.contiguous(), epilogue="silu")
        up = gemm_bf16(x.contiguous(), w2.contiguous())
        y = gemm_bf16((gate * up), w3.contiguous())
    else:
        y = ((F.silu(x.float() @ w1.float().t()) * (x.float() @ w2.float().t())) @ w3.float().t()).to(x.dtype)
    return rc.comm.all_reduce(y, group=tp_g) if n_tp > 1 else y


register(OpSpec(name="fsdp_tp_swiglu", problem_ids=(48,), group="tp", configs={"default": {"d": 256, "dff": 1024, "batch": 512}},
                make_inputs=_fsdp_tp_inputs, reference=_fsdp_tp_ref, ours=_fsdp_tp_ours, atol=5e-2, rtol=3e-2))


# ---- flagship: TP MLP block (all-gather -> GEMM -> SiLU -> GEMM -> reduce-scatter -> RMSNorm) ----
def _tpmlp_inputs(rc, cfg):
    W = rc.world
    f = cfg["ffn"] // W
    x = rc.randn(cfg["rows"], cfg["hidden"])
    w1 = rc.randn(f, cfg["hidden"], std=0.02, salt=1)        # K-major shard of W1 (columns of the full weight)
    w2 = rc.randn(cfg["hidden"], f, std=0.02, salt=2)        # K-major shard of W2 (rows of the full weight)
    gamma = torch.ones(cfg["hidden"], device=rc.device, dtype=rc.dtype)
    return (x, w1, w2, gamma, 1e-6)


def _tpmlp_ref(rc, x, w1, w2, gamma, eps):
    from ..refs.tp_mlp import TPMLPReference

    key = ("tpmlp_ref", x.shape, w1.data_ptr())
    if key not in rc.cache:
        rc.cache[key] = TPMLPReference(rc.world, x.shape[0], x.shape[1], w1, w2, gamma, eps)
    return rc.cache[key](x).clone()


def _tpmlp_ours(rc, x, w1, w2, gamma, eps):
    if not rc.dist.is_cuda:
        W = rc.world
        xf = rc.comm.all_gather_cat(x.contiguous(), dim=0) if W > 1 else x
        h = F.silu(xf.float() @ w1.float().t()).to(x.dtype)
        p = (h.float() @ w2.float().t()).to(x.dtype)
        y = rc.comm.reduce_scatter(p.float().contiguous()) if W > 1 else p.float()
        return _rms(y, gamma, eps).to(x.dtype)
    from ..models import TPMLPBlock, TPMLPConfig

    key = ("tpmlp_block", x.shape, w1.data_ptr())
    if key not in rc.cache:
        cfg = TPMLPConfig(rows_per_rank=x.shape[0], hidden=x.shape[1], ffn=w1.shape[0] * rc.world, eps=eps)
        rc.cache[key] = TPMLPBlock(rc.comm.group(), cfg, w1, w2, gamma)
    return rc.cache[key](x).clone()


def _tpmlp_cost(cfg, W):
    m = cfg["rows"] * W
    return Cost(flops=4.0 * m * cfg["hidden"] * cfg["ffn"] / W, nvlink_bytes=2.0 * (W - 1) * cfg["rows"] * cfg["hidden"] * 2,
                hbm_bytes=2.0 * (cfg["hidden"] * cfg["ffn"] / W * 2) + 3.0 * m * cfg["hidden"] * 2)


register(OpSpec(name="tp_mlp", problem_ids=(12, 15, 16, 45), group="tp",
                configs={"default": {"rows": 2048, "hidden": 8192, "ffn": 28672}, "small": {"rows": 256, "hidden": 512, "ffn": 2048}},
                make_inputs=_tpmlp_inputs, reference=_tpmlp_ref, ours=_tpmlp_ours, atol=6e-2, rtol=3e-2, cost=_tpmlp_cost,
                doc="sequence-sharded activations, column/row sharded weights; two fused launches per forward"))
