"""Each kernel alone against a plain PyTorch float32 reference of the same operation, at
sizes other than the engine tests use (widths that are no power of two, head sizes in steps
of 16, odd head counts).  float32 inputs catch indexing faults (tolerance 1e-5); bfloat16
inputs are compared at bfloat16's resolution."""

import math

import pytest
import torch

from tests.plain import model as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from acorninfer_b200.kernels import ops as o
    return o


def tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    table = torch.randn(331, 120, device=DEV).to(dtype)
    ids = torch.randint(0, 331, (77,), device=DEV, dtype=torch.int32)
    out = ops().embed(ids, table)
    assert out.dtype == torch.float32 and torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [48, 120, 1000, 4100])
def test_add_rmsnorm(dtype, H):
    rows, eps = 13, 3e-6
    resid = torch.randn(rows, H, device=DEV)
    delta = torch.randn(rows, H, device=DEV).to(dtype)
    w = 1 + 0.1 * torch.randn(H, device=DEV)
    want_resid = resid + delta.float()
    want = plain.rms_norm(want_resid.double(), w.double(), eps)
    r = resid.clone()
    out = ops().add_rmsnorm(r, delta, w, eps, dtype)
    assert torch.allclose(r, want_resid, atol=1e-6)
    assert torch.allclose(out.double(), want, **tol(dtype))
    # norm only (no delta): the residual is untouched
    r2 = resid.clone()
    out2 = ops().add_rmsnorm(r2, None, w, eps, dtype)
    assert torch.equal(r2, resid)
    assert torch.allclose(out2.double(), plain.rms_norm(resid.double(), w.double(), eps), **tol(dtype))
    # selected rows (one listed twice): normed into rows 0.., residual not written
    idx = torch.tensor([5, 0, 5, 12], device=DEV, dtype=torch.int32)
    r3 = resid.clone()
    out3 = ops().add_rmsnorm(r3, delta, w, eps, dtype, row_idx=idx)
    assert torch.equal(r3, resid)
    assert torch.allclose(out3.double(), want[idx.long()], **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,H", [(1024, 4096), (1500, 1000), (2500, 132), (1100, 8200)])
def test_add_rmsnorm_many_rows(dtype, rows, H):
    """Thousands of rows (a prompt portion): more blocks than fit on the device at once, widths that do
    not fill the last vector step and one beyond what the vector kernel keeps in registers, with and
    without the residual sum."""
    eps = 1e-5
    resid = torch.randn(rows, H, device=DEV)
    delta = torch.randn(rows, H, device=DEV).to(dtype)
    w = 1 + 0.1 * torch.randn(H, device=DEV)
    r = resid.clone()
    out = ops().add_rmsnorm(r, delta, w, eps, dtype)
    want_resid = resid + delta.float()
    assert torch.allclose(r, want_resid, atol=1e-6)
    assert torch.allclose(out.double(), plain.rms_norm(want_resid.double(), w.double(), eps), **tol(dtype))
    r2 = resid.clone()
    out2 = ops().add_rmsnorm(r2, None, w, eps, dtype)
    assert torch.equal(r2, resid)
    assert torch.allclose(out2.double(), plain.rms_norm(resid.double(), w.double(), eps), **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_and_cast(dtype):
    gu = torch.randn(9, 2 * 200, device=DEV).to(dtype)
    out = ops().swiglu(gu)
    g, u = gu.double()[:, :200], gu.double()[:, 200:]
    assert torch.allclose(out.double(), g * torch.sigmoid(g) * u, **tol(dtype))
    # gate and up in interleaved blocks of 64 outputs, rows wider than one pass of a thread block
    T, I, b = 5, 9 * 1024 + 64, 64
    gu = torch.randn(T, 2 * I, device=DEV).to(dtype)
    out = ops().swiglu(gu, block=b)
    blocks = gu.double().view(T, I // b, 2, b)
    g, u = blocks[:, :, 0].reshape(T, I), blocks[:, :, 1].reshape(T, I)
    assert torch.allclose(out.double(), g * torch.sigmoid(g) * u, **tol(dtype))
    x = torch.randn(1000, device=DEV)
    assert torch.equal(ops().cast(x, torch.bfloat16), x.to(torch.bfloat16))
    assert torch.equal(ops().cast(x.to(torch.bfloat16), torch.float32), x.to(torch.bfloat16).float())


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (7, 331, 120), (130, 65, 33), (64, 64, 16), (3, 1000, 257),
                                   (16, 100, 324), (17, 40, 1028), (65, 300, 200), (300, 130, 516)])
def test_gemm_f32_is_true_float32(M, N, K):
    """K a multiple of 4 takes the streaming kernel (up to 64 rows) or the 128 x 128 tile kernel, other K
    the plain one; (17, 40, 1028) runs more k-steps than the streaming kernel's ring has stages."""
    a = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV)
    out = ops().gemm_f32(a, w)
    want = a.double() @ w.double().T
    assert torch.allclose(out.double(), want, atol=1e-5 * math.sqrt(K), rtol=1e-5)
    # a row's result does not depend on the other rows
    assert torch.equal(ops().gemm_f32(a[:1].contiguous(), w)[0], out[0])


def test_gemm_f32_gives_the_same_bits_from_each_of_its_kernels():
    """A row's result is one chain of fused multiply-adds in the order of K in every kernel: the
    streaming kernel (8 rows), the tile kernel (200 rows) and the plain kernel (operands whose rows
    are not 16-byte aligned) agree bit for bit, also where tiles end inside the matrix."""
    M, N, K = 200, 333, 712
    a = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV)
    tile = ops().gemm_f32(a, w)
    rows = ops().gemm_f32(a[:8].contiguous(), w)
    assert torch.equal(rows, tile[:8])
    mid = ops().gemm_f32(a[100:140].contiguous(), w)            # 40 rows: three row blocks of the streaming kernel
    assert torch.equal(mid, tile[100:140])
    a_odd = torch.zeros(M, K + 1, device=DEV)[:, :K]            # row stride K + 1: the plain kernel
    a_odd.copy_(a)
    assert a_odd.stride(0) % 4 != 0
    assert torch.equal(ops().gemm_f32(a_odd, w), tile)
    assert torch.allclose(tile.double(), a.double() @ w.double().T, atol=1e-5 * math.sqrt(K), rtol=1e-5)


def test_gemm_f32_shows_what_a_reduced_precision_mode_would_hide():
    # 1 + 2^-12 is lost by a product that rounds its inputs to 10 mantissa bits (TF32) or to bfloat16
    a = torch.full((4, 8), 1 + 2 ** -12, device=DEV)
    w = torch.eye(8, device=DEV)
    assert torch.equal(ops().gemm_f32(a, w), a)
