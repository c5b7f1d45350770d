"""Python entry points of the small project-derived compute kernels (csrc/kernels/wild.cu)."""
from __future__ import annotations

import torch

from .. import _native as nv


def disco_contract(x: torch.Tensor, row_ptr: torch.Tensor, col: torch.Tensor, val: torch.Tensor, rows: int, nlon_out: int) -> torch.Tensor:
    """``x`` [BC, nlat_in, nlon_in] fp32; CSR (``row_ptr`` int32 [rows+1], ``col`` int32 = lat * nlon_in + lon, ``val`` fp32).
    Returns ``y`` [BC, rows, nlon_out] with ``y[b,r,p] = sum_e val[e] * x[b, lat_e, (lon_e + p*(nlon_in/nlon_out)) % nlon_in]``."""
    bc, nlat_in, nlon_in = x.shape
    xc = x.contiguous()
    y = torch.empty((bc, rows, nlon_out), dtype=torch.float32, device=x.device)
    nv.check(nv.cuda_lib().pkb_disco_contract(nv.ptr(xc), nv.ptr(row_ptr), nv.ptr(col), nv.ptr(val), nv.ptr(y), nv.c_ll(bc), rows,
                                              nlat_in, nlon_in, nlon_out, nv.current_stream()), "pkb_disco_contract")
    nv.count_launch()
    return y
