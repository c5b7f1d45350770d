"""Argument checks of the op wrappers run before any native call, so they can be exercised without a GPU."""
import pytest
import torch


def _fp8_operands(M=128, N=256, K=256, G=0):
    from parallelkernelbench_b200.refs.gemm_fp8 import quantize_rows_1x128, quantize_weight_128x128

    a8, sa = quantize_rows_1x128(torch.randn(M, K))
    w8, sb = quantize_weight_128x128(torch.randn((G, N, K) if G else (N, K)) * 0.1)
    return a8, sa, w8, sb


def test_gemm_fp8_rejects_malformed_operands():
    from parallelkernelbench_b200.ops.gemm_fp8 import gemm_fp8_blockscaled

    a8, sa, w8, sb = _fp8_operands()
    with pytest.raises(TypeError):
        gemm_fp8_blockscaled(a8.float(), sa, w8, sb)
    with pytest.raises(TypeError):
        gemm_fp8_blockscaled(a8, sa.double(), w8, sb)
    with pytest.raises(ValueError, match="offsets"):
        gemm_fp8_blockscaled(a8, sa, w8, sb, offsets=torch.zeros(2, dtype=torch.int32))      # dense weights with offsets
    with pytest.raises(ValueError, match="sb must hold"):
        gemm_fp8_blockscaled(a8, sa, w8, sb[:1])
    with pytest.raises(ValueError, match="sa must be"):
        gemm_fp8_blockscaled(a8, sa[:, :1], w8, sb)
    with pytest.raises(ValueError, match="multiples of 128"):
        gemm_fp8_blockscaled(a8[:, :192].contiguous(), sa, w8[:, :192].contiguous(), sb)
    g8, gs, gw8, gsb = _fp8_operands(G=2)
    with pytest.raises(ValueError, match="offsets must be int32"):
        gemm_fp8_blockscaled(g8, gs, gw8, gsb, offsets=torch.zeros(3, dtype=torch.int64))
    with pytest.raises(ValueError, match="row_meta"):
        gemm_fp8_blockscaled(g8, gs, gw8, gsb, offsets=torch.zeros(3, dtype=torch.int32), epilogue="row_scatter")
    with pytest.raises(ValueError, match="destination"):
        gemm_fp8_blockscaled(g8, gs, gw8, gsb, offsets=torch.zeros(3, dtype=torch.int32), epilogue="row_scatter",
                             row_meta=torch.zeros(128, 2, dtype=torch.int32), dest_ptrs=[], dest_pitch=256)
    with pytest.raises(ValueError, match="wrong shape or dtype"):
        gemm_fp8_blockscaled(a8, sa, w8, sb, out=torch.empty(128, 256, dtype=torch.float32))
    with pytest.raises(KeyError):
        gemm_fp8_blockscaled(a8, sa, w8, sb, epilogue="gelu")


def test_router_and_scatter_wrappers_reject_malformed_operands():
    from parallelkernelbench_b200.ops.moe import grouped_gemm_scatter, route_topk

    with pytest.raises(TypeError):
        route_topk(torch.randn(4, 8).to(torch.bfloat16), None, 2)
    with pytest.raises(ValueError):
        route_topk(torch.randn(4, 300), None, 2)
    with pytest.raises(ValueError):
        route_topk(torch.randn(4, 8), None, 9)
    with pytest.raises(TypeError):
        route_topk(torch.randn(4, 8), torch.randn(8).to(torch.bfloat16), 2)
    a, w = torch.randn(64, 32).to(torch.bfloat16), torch.randn(2, 16, 32).to(torch.bfloat16)
    off = torch.tensor([0, 32, 64], dtype=torch.int32)
    meta = torch.zeros(64, 2, dtype=torch.int32)
    with pytest.raises(TypeError):
        grouped_gemm_scatter(a.float(), w, off, meta, [4096], 16)
    with pytest.raises(ValueError, match="row_meta"):
        grouped_gemm_scatter(a, w, off, meta[:10], [4096], 16)
    with pytest.raises(ValueError, match="destination"):
        grouped_gemm_scatter(a, w, off, meta, [4096] * 9, 16)
    with pytest.raises(ValueError, match="destination"):
        grouped_gemm_scatter(a, w, off, meta, [4096], 12)


def test_fused_tp_objects_validate_shapes_before_touching_the_heap():
    from parallelkernelbench_b200.ops.tp import GemmAllGather, GemmAllReduce, GemvAllGather

    with pytest.raises(ValueError, match="256"):
        GemmAllReduce(None, 100, 64)
    with pytest.raises(ValueError, match="multiple of 8"):
        GemmAllReduce(None, 256, 30)
    with pytest.raises(ValueError, match="64"):
        GemmAllGather(None, 128, 100)
    with pytest.raises(ValueError, match="1, 2 or 4"):
        GemvAllGather(None, 3, 64)
    with pytest.raises(ValueError, match="multiple of 8"):
        GemvAllGather(None, 1, 12)


def test_small_kernel_entry_points_reject_bad_arguments_before_any_launch():
    """The argument checks of the native entry points return an error code (and a message) before anything is launched,
    so they run on a machine without a GPU; host memory stands in for the tensors."""
    import ctypes

    from parallelkernelbench_b200 import _native as nv

    lib = nv.cuda_lib()
    buf = torch.zeros(64, dtype=torch.float64)
    p, dbl, ll = nv.ptr(buf), ctypes.c_double, nv.c_ll
    calls = {
        "kalman_gain: no blocks": lambda: lib.pkb_kalman_gain(p, p, p, p, ll(0), 4, dbl(0.98), None),
        "kalman_gain: null tensor": lambda: lib.pkb_kalman_gain(None, p, p, p, ll(1), 4, dbl(0.98), None),
        "kalman_update: lambda zero": lambda: lib.pkb_kalman_update(p, p, p, p, p, p, p, ll(1), 4, dbl(0.0), None),
        "sinkhorn_rowdot: temperature": lambda: lib.pkb_sinkhorn_rowdot(p, p, p, 4, 4, dbl(0.0), None),
        "sinkhorn_coldot: more splits than rows": lambda: lib.pkb_sinkhorn_coldot(p, p, p, 4, 4, 5, dbl(0.07), None),
        "sinkhorn_coldot: an empty split": lambda: lib.pkb_sinkhorn_coldot(p, p, p, 10, 4, 8, dbl(0.07), None),
        "sinkhorn_scale: null tensor": lambda: lib.pkb_sinkhorn_scale(None, p, p, p, 4, 4, dbl(0.07), None),
        "knn_topk: dense without labels": lambda: lib.pkb_knn_topk(p, None, ll(1), ll(8), ll(0), 1, 8, 1, 2, 0, p, None, None, None),
        "knn_topk: too many candidates": lambda: lib.pkb_knn_topk(p, p, ll(1), ll(8192), ll(0), 1, 8192, 1, 2, 0, p, None, None, None),
        "knn_topk: k beyond the candidates": lambda: lib.pkb_knn_topk(p, p, ll(1), ll(8), ll(0), 1, 8, 1, 9, 0, p, None, None, None),
        "knn_topk: no output": lambda: lib.pkb_knn_topk(p, p, ll(1), ll(8), ll(0), 1, 8, 1, 2, 0, None, None, None, None),
        "knn_topk: votes without classes": lambda: lib.pkb_knn_topk(p, p, ll(1), ll(8), ll(0), 1, 8, 1, 2, 0, None, p, p, None),
        "mask_iou: pixels not a multiple of 32": lambda: lib.pkb_mask_iou_suppress(p, p, p, p, p, 2, 33, dbl(0.7), 0, None),
        "siglip: matching pairs outside the matrix": lambda: lib.pkb_siglip_loss_partials(p, p, 4, 4, 1, dbl(10.0), dbl(-10.0), 4, None),
        "siglip: more blocks than rows": lambda: lib.pkb_siglip_loss_partials(p, p, 4, 8, 0, dbl(10.0), dbl(-10.0), 5, None),
    }
    for what, call in calls.items():
        rc = call()
        msg = lib.pkb_last_error()
        assert rc != 0 and b"bad argument" in msg, (what, rc, msg)


def test_small_kernel_wrappers_reject_malformed_tensors():
    from parallelkernelbench_b200.ops import wild

    with pytest.raises(TypeError):
        wild.kalman_block_step(torch.zeros(1, 4, 1), torch.zeros(1), torch.zeros(1, 4, 1), torch.zeros(1, 4, 4), 0.98)     # fp32, CPU
    with pytest.raises(TypeError):
        wild.sinkhorn_knopp(torch.zeros(4, 4), 0.07, 3)
    with pytest.raises(ValueError):
        wild.knn_topk_local(torch.zeros(2, 8), torch.zeros(7, dtype=torch.int64), 2)
    with pytest.raises(ValueError):
        wild.knn_topk_local(torch.zeros(2, 5000), torch.zeros(5000, dtype=torch.int64), 2)
    with pytest.raises(ValueError):
        wild.knn_merge_votes(torch.zeros(4, 2, 2000, 2), 5, 10)
    with pytest.raises(ValueError):
        wild.mask_iou_suppress(torch.zeros(2, 3, 11), torch.zeros(2, dtype=torch.int64), 0.7)
    with pytest.raises(TypeError):
        wild.siglip_loss_from_products(torch.zeros(4, 4), 10.0, -10.0, 0)
    assert wild._sk_splits(1024) == (32, 32) and wild._sk_splits(10) == (10, 1) and wild._sk_splits(40) == (20, 2) and wild._sk_splits(1) == (1, 1)


def test_default_number_of_push_ctas_follows_the_rank_count():
    """A bulk-push CTA sustains a fixed rate while the GEMM consumes one remote shard per 1/W of its run time, so the default
    grows with the group; it stays a multiple of the 8 sub-blocks of a shard from 8 ranks on."""
    from parallelkernelbench_b200 import _native as nv

    f = nv.cuda_lib().pkb_tp_default_comm_ctas
    assert [f(w, 1) for w in (1, 2, 4, 6, 8)] == [2, 8, 8, 12, 16]
    assert [f(w, 0) for w in (1, 2, 4, 8)] == [2, 8, 8, 16]
    assert all(f(w, b) % 2 == 0 for w in range(1, 9) for b in (0, 1))          # whole CTA pairs
