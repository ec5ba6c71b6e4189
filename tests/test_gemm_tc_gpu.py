"""The tcgen05/TMA matrix product alone against a float32 reference, at sizes that are no
multiple of its tiles, with and without a split of K over a cluster."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from acorninfer_b200.kernels import ops as o
    return o


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 256, 128), (16, 96, 72), (5, 331, 120), (33, 200, 4096),
                                   (64, 1000, 264), (100, 384, 512), (300, 130, 96)])
@pytest.mark.parametrize("splits", [1, 2, 4])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tc_matches_float32(M, N, K, splits, out_dtype):
    torch.manual_seed(M * 1000 + N)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = torch.randn(N, K, device=DEV).to(torch.bfloat16)
    out = ops().gemm_tc(x, w, out_dtype, splits=splits)
    assert ops().gemm_tc_error() == 0
    want = x.double() @ w.double().T
    if out_dtype == torch.float32:
        assert torch.allclose(out.double(), want, atol=1e-3 * K ** 0.5, rtol=1e-4)
    else:
        assert torch.allclose(out.double(), want, atol=0.03 * K ** 0.5, rtol=1e-2)
    assert torch.equal(out, ops().gemm_tc(x, w, out_dtype, splits=splits))      # deterministic


def test_gemm_tc_strided_operands_and_refusals():
    from acorninfer_b200.kernels.ops import KernelError
    big = torch.randn(40, 512, device=DEV).to(torch.bfloat16)
    x = big[:, 128:384]                                       # row stride 512, K = 256
    w = torch.randn(77, 256, device=DEV).to(torch.bfloat16)
    out = ops().gemm_tc(x, w, torch.float32)
    assert torch.allclose(out.double(), x.double() @ w.double().T, atol=2e-2, rtol=1e-4)
    with pytest.raises(KernelError):
        ops().gemm_tc(torch.zeros(4, 36, device=DEV, dtype=torch.bfloat16), torch.zeros(8, 36, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(KernelError):
        ops().gemm_tc(torch.zeros(4, 64, device=DEV), torch.zeros(8, 64, device=DEV))
