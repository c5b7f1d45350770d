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
