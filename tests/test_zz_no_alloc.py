"""The allocation-free cross-entropy entry point, called through its exported C symbol.

Some callers of the library cannot allocate device memory when they call it (a frozen memory pool,
a host runtime that owns the GPU's memory, a serving loop that must not touch the allocator). For
them ``pkb_ce_loss_noalloc`` keeps its per-row scratch in a fixed array inside the library instead
of a buffer from ``cudaMalloc``. This test checks it against the ordinary two-kernel entry points
(``pkb_ce_stats`` + ``pkb_ce_finalize``, which use a caller-allocated statistics buffer) on two calls
in a row - the second call reuses the same scratch with different data and a different row count.
The file sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _noalloc(lib, logits, target):
    loss = torch.full((logits.shape[0],), float("nan"), device="cuda", dtype=torch.float32)
    fn = lib.pkb_ce_loss_noalloc                       # the exported C symbol itself
    fn.restype = ctypes.c_int
    rc = fn(ctypes.c_void_p(logits.data_ptr()), ctypes.c_void_p(target.data_ptr()), ctypes.c_void_p(loss.data_ptr()),
            ctypes.c_int(logits.shape[0]), ctypes.c_int(logits.shape[1]), ctypes.c_int(0 if logits.dtype == torch.bfloat16 else 1),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.pkb_last_error()
    return loss


def _existing(logits, target):
    from parallelkernelbench_b200.ops import ce_finalize, ce_local_stats

    return ce_finalize(ce_local_stats(logits, target, 0).unsqueeze(0))


def test_noalloc_cross_entropy_matches_existing_entry_point_twice():
    from parallelkernelbench_b200 import _native as nv

    lib = nv.cuda_lib()
    g = torch.Generator(device="cuda").manual_seed(2024)
    # 5000 x 257: more rows than the kernel's grid has blocks (its row loop strides) and an odd vocabulary;
    # 65536 x 8: exactly the capacity of the scratch array
    for rows, vocab, dtype in ((777, 4096, torch.bfloat16), (33, 1000, torch.float32), (5000, 257, torch.float32),
                               (65536, 8, torch.bfloat16)):
        logits = (torch.randn(rows, vocab, device="cuda", generator=g) * 3).to(dtype)
        target = torch.randint(0, vocab, (rows,), device="cuda", generator=g)
        got = _noalloc(lib, logits, target)
        want = _existing(logits, target)
        torch.cuda.synchronize()
        torch.testing.assert_close(got, want, atol=2e-3, rtol=2e-3)
        ref = torch.nn.functional.cross_entropy(logits.float(), target, reduction="none")
        torch.testing.assert_close(got, ref, atol=2e-3, rtol=2e-3)


def test_noalloc_rejects_sizes_beyond_its_scratch():
    from parallelkernelbench_b200 import _native as nv

    lib = nv.cuda_lib()
    lib.pkb_last_error.restype = ctypes.c_char_p
    dummy = torch.zeros(8, device="cuda")
    rc = lib.pkb_ce_loss_noalloc(ctypes.c_void_p(dummy.data_ptr()), ctypes.c_void_p(dummy.data_ptr()),
                                 ctypes.c_void_p(dummy.data_ptr()), ctypes.c_int(65537), ctypes.c_int(8), ctypes.c_int(1),
                                 ctypes.c_void_p(0))
    assert rc != 0 and b"exceed" in lib.pkb_last_error()
