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


@pytest.mark.parametrize("M,N,K,splits", [(3, 500, 512, 2), (16, 128, 4096, 8), (29, 333, 1000, 3), (32, 40, 256, 1)])
def test_gemm_tc_three_ctas_to_an_sm(M, N, K, splits):
    """The form with short rings (three CTAs fit on an SM) gives the same product."""
    torch.manual_seed(M + N)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = torch.randn(N, K, device=DEV).to(torch.bfloat16)
    out = ops().gemm_tc(x, w, torch.float32, splits=splits, per_sm=3)
    assert ops().gemm_tc_error() == 0
    assert torch.allclose(out.double(), x.double() @ w.double().T, atol=1e-3 * K ** 0.5, rtol=1e-4)
    assert torch.equal(out, ops().gemm_tc(x, w, torch.float32, splits=splits, per_sm=2))     # same order of sums
    # the plan takes that form for a matrix with more tiles than SMs and fewer than 1.5 to an SM
    assert ops().gemm_tc_plan(8, 24576, 4096) == (2, 3) and ops().gemm_tc_plan(8, 4096, 4096)[1] == 2


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


@pytest.mark.parametrize("M,N,K,splits", [(1, 256, 128, 1), (8, 4096, 512, 8), (13, 200, 264, 2), (32, 384, 1024, 4)])
def test_gemm_tc_add_norm_epilogue_and_normed_rows(M, N, K, splits):
    """product -> residual += ; h = residual * w_norm (no RMS factor yet) + partial sums of squares;
    the next product applies rsqrt(mean + eps) to its rows: together they equal add + RMSNorm + product."""
    from acorninfer_b200.kernels.ops import AddNormEpilogue, NormedRows
    torch.manual_seed(N + M)
    eps = 1e-5
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w1 = (torch.randn(N, K, device=DEV) / K ** 0.5).to(torch.bfloat16)
    resid = torch.randn(M, N, device=DEV)
    nw = 1 + 0.1 * torch.randn(N, device=DEV)
    N2 = 136
    w2 = (torch.randn(N2, N, device=DEV) / N ** 0.5).to(torch.bfloat16)
    want_resid = resid.double() + x.double() @ w1.double().T
    want_h = want_resid * torch.rsqrt(want_resid.pow(2).mean(-1, keepdim=True) + eps) * nw.double()
    want_out = want_h @ w2.double().T
    r = resid.clone()
    rows = ops().gemm_tc(x, w1, torch.bfloat16, splits=splits, epilogue=AddNormEpilogue(r, nw, eps))
    assert isinstance(rows, NormedRows) and rows.ss.shape == (-(-N // 128), M)
    assert torch.allclose(r.double(), want_resid, atol=2e-3, rtol=1e-4)
    assert torch.allclose(rows.ss.sum(0).double(), want_resid.pow(2).sum(-1), rtol=1e-3)
    if N % 8 == 0:
        out = ops().gemm_tc(rows, w2, torch.float32, splits=1)
        assert torch.allclose(out.double(), want_out, atol=3e-2, rtol=3e-2)
        out2 = ops().gemm_tc(rows, w2, torch.float32, splits=2)
        assert torch.allclose(out2.double(), want_out, atol=3e-2, rtol=3e-2)
    assert ops().gemm_tc_error() == 0


@pytest.mark.parametrize("M,I,K,splits", [(1, 64, 64, 1), (8, 640, 512, 1), (20, 192, 1024, 4)])
def test_gemm_tc_swiglu_epilogue(M, I, K, splits):
    torch.manual_seed(I)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    g = (torch.randn(I, K, device=DEV) / K ** 0.5).to(torch.bfloat16)
    u = (torch.randn(I, K, device=DEV) / K ** 0.5).to(torch.bfloat16)
    w = torch.stack([g.view(I // 64, 64, K), u.view(I // 64, 64, K)], dim=1).reshape(2 * I, K).contiguous()
    out = ops().gemm_tc(x, w, torch.bfloat16, splits=splits, swiglu=True)
    gg, uu = x.double() @ g.double().T, x.double() @ u.double().T
    assert out.shape == (M, I)
    assert torch.allclose(out.double(), gg * torch.sigmoid(gg) * uu, atol=2e-2, rtol=2e-2)
    # the stand-alone kernel reads the same block layout
    gu = ops().gemm_tc(x, w, torch.bfloat16, splits=1)
    assert torch.allclose(ops().swiglu(gu, block=64).float(), out.float(), atol=2e-2, rtol=2e-2)
    assert ops().gemm_tc_error() == 0


@pytest.mark.parametrize("nq,nkv,K,qlens,norm,write", [(4, 2, 256, [7, 1, 5], True, True), (6, 1, 520, [1, 1, 1, 1], True, True),
                                                       (2, 2, 128, [30], False, True), (8, 4, 1024, [3, 20], True, False)])
def test_gemm_tc_qkv_rope_epilogue(nq, nkv, K, qlens, norm, write):
    """The q/k/v product with norm, rotation and cache write as its epilogue, against the plain
    product followed by the stand-alone kernel (which rounds to bfloat16 in between)."""
    from acorninfer_b200.kernels.ops import RopeKvEpilogue
    from tests.paged import rows_layout
    torch.manual_seed(nq * 10 + nkv)
    d, P, NP, eps, theta = 128, 16, 300, 3e-6, 1e4
    befores = [0, 37, 4000, 15][:len(qlens)]
    lay = rows_layout(befores, qlens, P, NP, seed=2)
    T = lay["num_tokens"]
    x = torch.randn(T, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn((nq + 2 * nkv) * d, K, device=DEV) / K ** 0.5).to(torch.bfloat16)
    qw = (1 + 0.2 * torch.randn(d, device=DEV)) if norm else None
    kw = (1 + 0.2 * torch.randn(d, device=DEV)) if norm else None
    inv = (1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV)
    # reference: the two kernels one after the other
    ref = ops().gemm_tc(x, w, torch.bfloat16)
    k_ref = torch.zeros(NP, nkv, P, d, device=DEV, dtype=torch.bfloat16)
    v_ref = torch.zeros_like(k_ref)
    ops().qk_rope_kv(ref, qw, kw, inv, lay["positions"], lay["token_row"], lay["block_table"], lay["page_base"],
                     k_ref, v_ref, nq, nkv, d, d, False, eps)
    k_pages, v_pages = torch.zeros_like(k_ref), torch.zeros_like(k_ref)
    out = ops().gemm_tc_qkv_rope(x, w, RopeKvEpilogue(
        lay["positions"], lay["token_row"], lay["block_table"], lay["page_base"], k_pages if write else None,
        v_pages if write else None, qw, kw, inv, nq, nkv, eps))
    assert ops().gemm_tc_error() == 0
    tol = dict(atol=4e-2, rtol=2e-2)
    assert torch.allclose(out[:, :nq * d].float(), ref[:, :nq * d].float(), **tol)
    if write:
        assert torch.allclose(k_pages.float(), k_ref.float(), **tol)
        assert torch.allclose(v_pages.float(), v_ref.float(), **tol)
        assert float(k_pages.float().abs().sum()) > 0
    else:
        assert float(k_pages.float().abs().sum()) == 0 and float(v_pages.float().abs().sum()) == 0
    # against float64 arithmetic for the query heads: norm and rotation of the exact product
    q = (x.double() @ w.double().T)[:, :nq * d].view(T, nq, d).cpu()
    if norm:
        q = q * torch.rsqrt((q * q).mean(-1, keepdim=True) + eps) * qw.double().cpu()
    ang = lay["positions"].cpu().double()[:, None] * inv.cpu().double()[None, :]
    c, s_ = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = q[..., :64], q[..., 64:]
    want = torch.cat([a * c - b * s_, b * c + a * s_], dim=-1).reshape(T, nq * d)
    assert torch.allclose(out[:, :nq * d].double().cpu(), want, atol=3e-2, rtol=2e-2)


# ---------------------------------------------------------------------------- the paired kernel


@pytest.mark.parametrize("M,N,K", [(1, 8, 8), (256, 256, 64), (300, 504, 200), (513, 1000, 4160), (40, 6144, 512),
                                   (700, 264, 1024)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tc_pair_matches_float64(M, N, K, out_dtype):
    """The pair-of-CTAs kernel alone: tiles that end inside the matrix in both directions, a K that is no
    multiple of the stage, more tiles than pairs of SMs (700 x 264 with two pairs), one row."""
    torch.manual_seed(M + N)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / K ** 0.5).to(torch.bfloat16)
    want = x.double() @ w.double().T
    for pairs in (None, 2):
        out = ops().gemm_tc_pair(x, w, out_dtype, pairs=pairs)
        assert ops().gemm_tc_pair_error() == 0
        tol = dict(atol=2e-2, rtol=2e-2) if out_dtype == torch.bfloat16 else dict(atol=1e-4, rtol=1e-4)
        assert torch.allclose(out.double(), want, **tol)
    assert torch.equal(ops().gemm_tc_pair(x, w, out_dtype), out)             # the same sums whatever the number of pairs


@pytest.mark.parametrize("M,H,I", [(64, 256, 192), (300, 1024, 1536), (700, 200, 320)])
def test_gemm_tc_pair_epilogues(M, H, I):
    """SwiGLU and add + norm sums with rows that arrive un-normalised, against float64; widths that are
    no multiple of the 256-column tile (200: the second half of the only tile is empty)."""
    from acorninfer_b200.kernels.ops import AddNormEpilogue, NormedRows
    torch.manual_seed(M)
    x = (torch.randn(M, H, device=DEV) * 0.5).to(torch.bfloat16)
    wgu = (torch.randn(2 * I, H, device=DEV) / H ** 0.5).to(torch.bfloat16)
    ss = (torch.rand(5, M, device=DEV) + 0.5) * H
    inv = torch.rsqrt(ss.double().sum(0) / H + 1e-6)
    got = ops().gemm_tc_pair(NormedRows(x, ss, 1e-6, H), wgu, swiglu=True)
    gu = ((x.double() @ wgu.double().T) * inv[:, None]).view(M, I // 64, 2, 64)
    g, u = gu[:, :, 0].reshape(M, I), gu[:, :, 1].reshape(M, I)
    assert got.shape == (M, I)
    assert torch.allclose(got.double(), g * torch.sigmoid(g) * u, atol=2e-2, rtol=2e-2)
    h = (torch.randn(M, I, device=DEV) * 0.5).to(torch.bfloat16)
    wd = (torch.randn(H, I, device=DEV) / I ** 0.5).to(torch.bfloat16)
    resid = torch.randn(M, H, device=DEV)
    nw = torch.rand(H, device=DEV) + 0.5
    r = resid.clone()
    rows = ops().gemm_tc_pair(h, wd, epilogue=AddNormEpilogue(r, nw, 1e-6))
    want_r = resid.double() + h.double() @ wd.double().T
    assert torch.allclose(r.double(), want_r, atol=1e-4, rtol=1e-4)
    assert torch.allclose(rows.x.double(), want_r * nw.double(), atol=3e-2, rtol=2e-2)
    assert torch.allclose(rows.ss.double().sum(0), (want_r ** 2).sum(1), rtol=1e-4)
    assert rows.width == H and ops().gemm_tc_pair_error() == 0
    # the rows it hands on are what the one-CTA kernel hands on for the rows that kernel takes
    if M <= 64:
        r1 = resid.clone()
        one = ops().gemm_tc(h, wd, epilogue=AddNormEpilogue(r1, nw, 1e-6))
        assert torch.allclose(r1, r, atol=1e-5, rtol=1e-5) and torch.allclose(one.x.float(), rows.x.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("nq,nkv,K,qlens,norm,write,table", [(4, 2, 256, [70, 1, 50], True, True, True),
                                                             (5, 1, 520, [33, 40], True, True, False),
                                                             (2, 2, 128, [300], False, True, True),
                                                             (8, 4, 1024, [3, 200, 90], True, False, True)])
def test_gemm_tc_pair_qkv_rope_epilogue(monkeypatch, nq, nkv, K, qlens, norm, write, table):
    """The paired kernel's q/k/v epilogue (more than 32 rows go to it): against the plain product
    followed by the stand-alone kernel, with the cos/sin table and with angles computed in the epilogue;
    seven heads (5 + 1 + 1) leave the second half of the last tile without a head."""
    from acorninfer_b200.kernels.ops import RopeKvEpilogue
    from tests.paged import rows_layout
    torch.manual_seed(nq * 10 + nkv)
    d, P, NP, eps, theta = 128, 16, 400, 3e-6, 1e4
    befores = [0, 37, 4000][:len(qlens)]
    lay = rows_layout(befores, qlens, P, NP, seed=2)
    T = lay["num_tokens"]
    assert T > 32
    x = torch.randn(T, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn((nq + 2 * nkv) * d, K, device=DEV) / K ** 0.5).to(torch.bfloat16)
    qw = (1 + 0.2 * torch.randn(d, device=DEV)) if norm else None
    kw = (1 + 0.2 * torch.randn(d, device=DEV)) if norm else None
    inv = (1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV)
    ref = torch.mm(x, w.t())
    k_ref = torch.zeros(NP, nkv, P, d, device=DEV, dtype=torch.bfloat16)
    v_ref = torch.zeros_like(k_ref)
    ops().qk_rope_kv(ref, qw, kw, inv, lay["positions"], lay["token_row"], lay["block_table"], lay["page_base"],
                     k_ref, v_ref, nq, nkv, d, d, False, eps)
    k_pages, v_pages = torch.zeros_like(k_ref), torch.zeros_like(k_ref)
    cos_sin = ops().rope_table(lay["positions"], inv) if table else None
    if table:
        ang = (lay["positions"].float()[:, None] * inv[None, :]).double()       # the angle itself is a float32 product
        assert torch.allclose(cos_sin.double(), torch.cat([ang.cos(), ang.sin()], dim=1), atol=1e-6)
    out = ops().gemm_tc_qkv_rope(x, w, RopeKvEpilogue(
        lay["positions"], lay["token_row"], lay["block_table"], lay["page_base"], k_pages if write else None,
        v_pages if write else None, qw, kw, inv, nq, nkv, eps, cos_sin=cos_sin))
    assert ops().gemm_tc_pair_error() == 0
    tol = dict(atol=4e-2, rtol=2e-2)
    assert torch.allclose(out[:, :nq * d].float(), ref[:, :nq * d].float(), **tol)
    if write:
        assert torch.allclose(k_pages.float(), k_ref.float(), **tol)
        assert torch.allclose(v_pages.float(), v_ref.float(), **tol)
        assert float(k_pages.float().abs().sum()) > 0
    else:
        assert float(k_pages.float().abs().sum()) == 0 and float(v_pages.float().abs().sum()) == 0


def test_gemm_tc_pair_random_shapes():
    """Thirty random shapes (rows 1 .. 3,000, widths that are no multiple of the tile, K in steps of 8)
    against the library product of the same bfloat16 operands, with every number of pairs from few to all."""
    import random
    rng = random.Random(7)
    for _ in range(30):
        M, N, K = rng.randint(1, 3000), 8 * rng.randint(1, 600), 8 * rng.randint(1, 300)
        x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
        w = (torch.randn(N, K, device=DEV) / K ** 0.5).to(torch.bfloat16)
        out = ops().gemm_tc_pair(x, w, torch.float32, pairs=rng.choice([None, 1, 3, 37]))
        want = torch.mm(x, w.t(), out_dtype=torch.float32)
        assert torch.allclose(out, want, atol=2e-3, rtol=2e-3), (M, N, K)
    assert ops().gemm_tc_pair_error() == 0
