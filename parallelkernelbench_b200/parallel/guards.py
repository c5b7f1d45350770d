"""Guard bands around symmetric-heap allocations (debug aid, ``PKB_HEAP_GUARD=1``).

With the switch on, every allocation of the GPU heap and of its CPU twin is bracketed by two bands of ``GUARD_BYTES`` filled
with a known byte; the trailing band starts at the first byte after the requested size, so an overrun by a single byte is
seen. ``check()`` reports the allocations whose bands were written - by this rank's kernels or by a peer storing through
NVLink into this rank's heap. Nothing traps and nothing is checked on the device: the bands are compared on demand (the
launcher's worker does it after the run and after the timing loop). The reference has no counterpart; it relies on
``compute-sanitizer``-style tools being available, which they are not here.
"""
from __future__ import annotations

import os
from typing import Callable

GUARD_BYTES = 4096
PATTERN = 0xA5


def enabled() -> bool:
    return os.environ.get("PKB_HEAP_GUARD") == "1"


class GuardBook:
    """Bookkeeping of the bands of one heap. ``fill(offset, nbytes)`` writes the pattern into this rank's heap and
    ``first_bad(offset, nbytes)`` returns the index of the first byte that no longer holds it (or -1)."""

    def __init__(self, fill: Callable[[int, int], None], first_bad: Callable[[int, int], int], align: int):
        self._fill, self._first_bad, self.align = fill, first_bad, align
        self.bands: list[dict] = []

    def allocate(self, raw_alloc: Callable[[int], int], nbytes: int) -> int:
        """Allocate ``nbytes`` through ``raw_alloc`` with a band on either side; returns the offset of the user region."""
        lead = (GUARD_BYTES + self.align - 1) // self.align * self.align      # keeps the user region aligned like a plain allocation
        tail = (nbytes + self.align - 1) // self.align * self.align - nbytes + GUARD_BYTES
        off = raw_alloc(lead + nbytes + tail)
        self._fill(off, lead)
        self._fill(off + lead + nbytes, tail)
        self.bands.append({"offset": off + lead, "nbytes": nbytes, "lead": (off, lead), "tail": (off + lead + nbytes, tail)})
        return off + lead

    def check(self) -> list[dict]:
        """Allocations with a damaged band: ``{"offset", "nbytes", "side", "distance"}`` where ``distance`` is how far from
        the user region the first damaged byte lies (1 = the byte right before / after it)."""
        bad = []
        for b in self.bands:
            o, n = b["lead"]
            i = self._first_bad(o, n)
            if i >= 0:
                # report the damaged byte closest to the user region for an underrun
                j = n - 1
                while j > i and self._first_bad(o + j, 1) < 0:
                    j -= 1
                bad.append({"offset": b["offset"], "nbytes": b["nbytes"], "side": "before", "distance": n - j})
            o, n = b["tail"]
            i = self._first_bad(o, n)
            if i >= 0:
                bad.append({"offset": b["offset"], "nbytes": b["nbytes"], "side": "after", "distance": i + 1})
        return bad

    def refill(self) -> None:
        for b in self.bands:
            self._fill(*b["lead"])
            self._fill(*b["tail"])


class GuardViolation(RuntimeError):
    def __init__(self, violations: list[dict]):
        self.violations = violations
        first = violations[0]
        super().__init__(f"{len(violations)} symmetric-heap allocation(s) were written outside their bounds; first: allocation at "
                         f"offset {first['offset']} ({first['nbytes']} bytes), {first['distance']} byte(s) {first['side']} it")
