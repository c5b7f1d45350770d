"""Roofline estimator.

``roofline_ms = max(FLOPs / peak_flops, NVLink bytes per GPU per direction / link bandwidth)``; an
HBM term is reported alongside for information and ``limiter`` names the largest of the three. The
compute and HBM denominators are the values measured on this pool (``MEASURED_PEAKS.json`` - a
cuBLAS bf16 GEMM and a device copy), the link bandwidth is the measured peer-copy rate. The
reference points at a roofline tool but does not ship one (reference: README.md:27).
"""
from __future__ import annotations

from dataclasses import dataclass

from ..utils import env


@dataclass
class Cost:
    """Algorithmic cost of one call on one GPU."""
    flops: float = 0.0
    nvlink_bytes: float = 0.0   # bytes that must leave (or enter) this GPU over NVLink, per direction
    hbm_bytes: float = 0.0      # compulsory HBM traffic
    dtype: str = "bf16"         # selects the compute peak (bf16 / fp8 / fp32)


def peaks() -> dict:
    p = env.measured_peaks()
    bf16 = float(p.get("bf16_tflops_sustained") or p.get("bf16_tflops") or 1400.0)
    return {"bf16_tflops": bf16, "bf16_tflops_burst": float(p.get("bf16_tflops") or bf16),
            "fp8_tflops": 2.0 * bf16, "fp32_tflops": bf16 / 16.0,
            "hbm_gbs": float(p.get("hbm_gbs") or 6650.0), "nvlink_gbs": env.NVLINK_GBS_PER_DIR,
            "source": p.get("source", "fallback")}


def estimate(cost: Cost, measured_ms: float | None = None) -> dict:
    pk = peaks()
    tf = {"bf16": pk["bf16_tflops"], "fp16": pk["bf16_tflops"], "fp8": pk["fp8_tflops"], "fp32": pk["fp32_tflops"],
          "fp64": pk["fp32_tflops"] / 2}.get(cost.dtype, pk["bf16_tflops"])
    t_compute = cost.flops / (tf * 1e12) * 1e3
    t_link = cost.nvlink_bytes / (pk["nvlink_gbs"] * 1e9) * 1e3
    t_hbm = cost.hbm_bytes / (pk["hbm_gbs"] * 1e9) * 1e3
    roof = max(t_compute, t_link)
    limiter = max((("compute", t_compute), ("nvlink", t_link), ("hbm", t_hbm)), key=lambda kv: kv[1])[0]
    out = {"roofline_ms": roof, "compute_ms": t_compute, "nvlink_ms": t_link, "hbm_ms": t_hbm, "limiter": limiter,
           "peaks_source": pk["source"]}
    if measured_ms:
        out["pct_of_roofline"] = 100.0 * max(roof, 1e-9) / measured_ms
        out["achieved_tflops"] = cost.flops / (measured_ms * 1e-3) / 1e12
        out["achieved_nvlink_gbs"] = cost.nvlink_bytes / (measured_ms * 1e-3) / 1e9
        out["achieved_hbm_gbs"] = cost.hbm_bytes / (measured_ms * 1e-3) / 1e9
    return out
