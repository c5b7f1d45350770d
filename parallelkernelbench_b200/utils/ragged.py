"""Results whose length is only known on the device.

A variable exchange (all-to-all with device-side counts, a gather of uneven shards) ends with ``n`` valid rows in a buffer of
a fixed capacity, ``n`` being a device scalar. Trimming the buffer to ``n`` rows needs the value on the host, which stalls
the stream. An implementation therefore returns ``Ragged(buffer, n)`` and never reads ``n`` itself; the harness trims when it
stores the output for comparison, outside the timed region (``harness.compare.normalize_output``). The PyTorch + NCCL
references pay that host round trip inside every call (reference: reference/27_moe_all2all_primitive.py:22, the output size is read back with ``.item()``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class Ragged:
    """``data.narrow(dim, 0, count)`` is the result; ``count`` is a one-element integer tensor on ``data``'s device."""
    data: torch.Tensor
    count: torch.Tensor
    dim: int = 0

    def trimmed(self) -> torch.Tensor:
        """The valid part (reads ``count`` on the host: call it outside hot paths only)."""
        n = int(self.count.reshape(-1)[0])
        return self.data.narrow(self.dim, 0, min(n, self.data.shape[self.dim])).contiguous()


def compact_padded(segments: torch.Tensor, counts: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``segments`` is ``[S, cap, ...]`` with ``counts[s]`` valid leading rows in segment ``s``. Returns ``(rows, total)``:
    ``rows`` is ``[S * cap, ...]`` whose first ``total`` rows are the valid rows of segment 0, then of segment 1, ...
    Everything is a gather through computed indices: no mask selection, hence no size comes back to the host."""
    S, cap = segments.shape[0], segments.shape[1]
    counts = counts.reshape(-1).to(torch.int64)
    ends = torch.cumsum(counts, 0)
    j = torch.arange(S * cap, device=segments.device)
    seg = torch.searchsorted(ends, j, right=True).clamp(max=S - 1)
    within = (j - (ends - counts)[seg]).clamp(min=0, max=cap - 1)
    flat = segments.reshape(S * cap, *segments.shape[2:])
    return flat[seg * cap + within], ends[-1:].clone()


def permute_segments_padded(data: torch.Tensor, seg_len: torch.Tensor, order: torch.Tensor, valid: torch.Tensor | None = None) -> Ragged:
    """Concatenate the segments of the 1-D ``data`` (lengths ``seg_len``) in the order ``order``. ``data`` may be longer than
    the sum of the lengths (a capacity buffer); the result has ``data``'s length with the valid part in front."""
    seg_len = seg_len.to(torch.int64)
    starts = torch.cumsum(seg_len, 0) - seg_len
    new_len = seg_len[order]
    new_ends = torch.cumsum(new_len, 0)
    j = torch.arange(data.shape[0], device=data.device)
    seg = torch.searchsorted(new_ends, j, right=True).clamp(max=order.numel() - 1)
    src = starts[order][seg] + (j - (new_ends - new_len)[seg])
    return Ragged(data[src.clamp(min=0, max=data.shape[0] - 1)], new_ends[-1:].clone() if valid is None else valid)


__all__ = ["Ragged", "compact_padded", "permute_segments_padded"]
