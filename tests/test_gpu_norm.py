import pytest
import torch

pytestmark = pytest.mark.gpu


def _rms_ref(x, gamma, eps):
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()


@pytest.mark.parametrize("rows,cols", [(1, 8), (7, 1024), (2048, 8192), (33, 4104)])
def test_rmsnorm(rows, cols):
    from parallelkernelbench_b200.ops import rmsnorm

    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(cols, device="cuda")).to(torch.bfloat16)
    y = rmsnorm(x, gamma, 1e-6)
    torch.testing.assert_close(y.float(), _rms_ref(x, gamma, 1e-6), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_sum_rmsnorm(dtype):
    from parallelkernelbench_b200.ops import sum_rmsnorm

    parts = torch.randn(4, 257, 2048, device="cuda", dtype=dtype)
    gamma = torch.ones(2048, device="cuda", dtype=torch.bfloat16)
    y = sum_rmsnorm(parts, gamma, 1e-6, scale=0.25)
    ref = _rms_ref(parts.float().sum(0) * 0.25, gamma, 1e-6)
    torch.testing.assert_close(y.float(), ref, atol=2e-2, rtol=2e-2)
