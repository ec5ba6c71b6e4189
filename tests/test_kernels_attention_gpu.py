"""The attention-side kernels alone: q/k norm + rotary + page write, and paged attention,
against the plain formulas; inputs are made so that a far key, a window's edge or a page's
edge decides the result."""

import pytest
import torch

from tests.paged import rows_layout, scatter_to_pages
from tests.plain import model as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from acorninfer_b200.kernels import ops as o
    return o


def rope_reference(x, positions, rot, theta, interleaved):
    """x [T, heads, d] float64; rotates the first ``rot`` dims (plain formulas)."""
    inv = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    ang = (positions.to(torch.float32)[:, None] * inv[None]).double()
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:rot:2], x[..., 1:rot:2]
        out[..., 0:rot:2], out[..., 1:rot:2] = a * c - b * s, b * c + a * s
    else:
        a, b = x[..., :rot // 2], x[..., rot // 2:rot]
        out[..., :rot // 2], out[..., rot // 2:rot] = a * c - b * s, b * c + a * s
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,rot,inter,norm,P", [
    (4, 2, 16, 16, False, True, 4), (10, 2, 48, 48, False, True, 16), (3, 3, 80, 32, True, True, 8),
    (6, 1, 112, 112, False, False, 32), (2, 1, 272, 64, False, True, 16), (32, 8, 128, 128, False, True, 16),
    (5, 5, 64, 64, False, False, 8), (8, 1, 32, 32, False, True, 4), (2, 2, 256, 256, False, True, 16)])
@pytest.mark.parametrize("qlens", [[21, 1, 2, 17], [290, 1, 2, 17]])      # few tokens / many: two shapes of the kernel
def test_qk_rope_kv(dtype, nq, nkv, d, rot, inter, norm, P, qlens):
    theta, eps, NP = 5e5, 2e-6, 1400
    befores = [0, 37, 4095, 15]
    lay = rows_layout(befores, qlens, P, NP, seed=1)
    T = lay["num_tokens"]
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device=DEV).to(dtype)
    qw = (1 + 0.2 * torch.randn(d, device=DEV)) if norm else None
    kw = (1 + 0.2 * torch.randn(d, device=DEV)) if norm else None
    inv = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(DEV)
    k_pages = torch.zeros(NP, nkv, P, d, device=DEV, dtype=dtype)
    v_pages = torch.zeros_like(k_pages)
    src = qkv.double().cpu().view(T, nq + 2 * nkv, d)
    ops().qk_rope_kv(qkv, qw, kw, inv, lay["positions"], lay["token_row"], lay["block_table"], lay["page_base"],
                     k_pages, v_pages, nq, nkv, d, rot, inter, eps)
    q, k, v = src[:, :nq], src[:, nq:nq + nkv], src[:, nq + nkv:]
    if norm:
        q = plain.rms_norm(q, qw.double().cpu(), eps)
        k = plain.rms_norm(k, kw.double().cpu(), eps)
    pos = lay["positions"].cpu()
    q, k = rope_reference(q, pos, rot, theta, inter), rope_reference(k, pos, rot, theta, inter)
    tol = dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    got_q = qkv.double().cpu().view(T, nq + 2 * nkv, d)[:, :nq]
    assert torch.allclose(got_q, q, **tol)
    at = 0
    for r, (before, n) in enumerate(zip(befores, qlens)):
        for i in range(n):
            p = before + i
            page, slot = lay["tables"][r][p // P], p % P
            assert torch.allclose(k_pages[page, :, slot].double().cpu(), k[at + i], **tol)
            assert torch.equal(v_pages[page, :, slot].cpu(), qkv.cpu().view(T, -1, d)[at + i, nq + nkv:])
        at += n
    # pages of other rows and untouched slots stay zero
    used = {(lay["tables"][r][(b + i) // P], (b + i) % P) for r, (b, n) in enumerate(zip(befores, qlens)) for i in range(n)}
    mask = torch.ones(NP, P, dtype=torch.bool)
    for pg, sl in used:
        mask[pg, sl] = False
    assert float(k_pages.cpu().float().abs().sum(dim=(1, 3))[mask].sum()) == 0


def dense_attention(q, k, v, scale, window, q_start):
    """q [n, nq, d] at positions q_start..; k, v [L, nkv, d]: plain formulas on the tail."""
    L = k.shape[0]
    full_q = torch.zeros(L, q.shape[1], q.shape[2], dtype=q.dtype)
    full_q[q_start:] = q
    out = plain.causal_attention(full_q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1), scale, window)
    return out.transpose(0, 1)[q_start:]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,P,window", [(4, 2, 16, 4, None), (10, 2, 48, 16, None), (8, 1, 128, 16, None),
                                               (6, 3, 80, 8, 13), (5, 5, 32, 32, 40), (20, 2, 18, 16, None),
                                               (3, 1, 200, 8, None), (24, 2, 36, 16, 700)])
def test_attention_plain(dtype, nq, nkv, d, P, window):
    """Among the cases: more query heads to a kv head than one block takes (10, 12), head sizes whose rows
    are not 16-byte aligned (18; 36 in bfloat16) or wider than the 128 lanes (200), a row of 1,100 keys
    (three chunks of 512) and a window that starts inside the second chunk."""
    before, qlens = [0, 300, 129, 16, 0, 1100], [150, 1, 2, 1, 1, 3]
    num_pages = sum(-(-(b + n) // P) for b, n in zip(before, qlens)) + 7
    lay = rows_layout(before, qlens, P, num_pages, seed=2)
    scale = d ** -0.5
    k_pages = torch.zeros(num_pages, nkv, P, d, device=DEV, dtype=dtype)
    v_pages = torch.zeros_like(k_pages)
    qs, wants = [], []
    for r, (b, n) in enumerate(zip(before, qlens)):
        L = b + n
        k = torch.randn(L, nkv, d).to(dtype)
        v = torch.randn(L, nkv, d).to(dtype)
        q = torch.randn(n, nq, d).to(dtype)
        if r == 1:
            # one far key stands out: key 7 matches the query, all others score low
            k[7] = (q[0, :nkv] * 8).to(dtype)
        scatter_to_pages(k_pages, lay["tables"][r], k.to(DEV), P)
        scatter_to_pages(v_pages, lay["tables"][r], v.to(DEV), P)
        qs.append(q)
        wants.append(dense_attention(q.double(), k.double(), v.double(), scale, window, b))
    q_all = torch.cat(qs).reshape(-1, nq * d).to(DEV)
    wide = torch.cat([q_all, torch.randn(q_all.shape[0], 2 * nkv * d, device=DEV).to(dtype)], dim=1).contiguous()
    out = ops().attention_plain(wide, wide.stride(0), k_pages, v_pages, lay["block_table"], lay["page_base"],
                                lay["token_row"], lay["positions"], lay["num_tokens"], nq, nkv, d, scale, window)
    want = torch.cat(wants).reshape(-1, nq * d)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    assert torch.allclose(out.double().cpu(), want, **tol)


def build_case(before, qlens, nq, nkv, d, P, window, num_pages, seed, standout_row=None):
    """Random paged K/V and queries for rows with ``before`` cached tokens and ``qlens`` new ones;
    returns the device inputs and the plain float64 result [tokens, nq * d]."""
    dtype = torch.bfloat16
    num_pages = max(num_pages, sum(-(-(b + n) // P) for b, n in zip(before, qlens)) + 7)
    lay = rows_layout(before, qlens, P, num_pages, seed=seed)
    torch.manual_seed(seed)
    k_pages = torch.zeros(num_pages, nkv, P, d, device=DEV, dtype=dtype)
    v_pages = torch.zeros_like(k_pages)
    qs, wants = [], []
    for r, (b, n) in enumerate(zip(before, qlens)):
        L = b + n
        k, v, q = torch.randn(L, nkv, d).to(dtype), torch.randn(L, nkv, d).to(dtype), torch.randn(n, nq, d).to(dtype)
        if r == standout_row and L > 70:
            # a far key decides: key 3 is aligned with the last query of the row, its value is large
            k[3] = (q[-1].view(nkv, nq // nkv, d)[:, 0] * 6).to(dtype)
            v[3] = 5.0
        scatter_to_pages(k_pages, lay["tables"][r], k.to(DEV), P)
        scatter_to_pages(v_pages, lay["tables"][r], v.to(DEV), P)
        qs.append(q)
        wants.append(dense_attention(q.double(), k.double(), v.double(), d ** -0.5, window, b))
    q_all = torch.cat(qs).reshape(-1, nq * d).to(DEV)
    wide = torch.cat([q_all, torch.randn(q_all.shape[0], 2 * nkv * d, device=DEV).to(dtype)], dim=1).contiguous()
    row_start = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=DEV)
    row_pos = torch.tensor(before, dtype=torch.int32, device=DEV)
    tiles = torch.tensor([(r, q0) for r, n in enumerate(qlens) for q0 in range(0, n, 64)], dtype=torch.int32,
                         device=DEV).view(-1, 2)
    return lay, wide, k_pages, v_pages, row_start, row_pos, tiles, torch.cat(wants).reshape(-1, nq * d)


BF16_TOL = dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("nq,nkv,d,P,window", [(32, 8, 128, 16, None), (4, 2, 16, 4, None), (8, 1, 32, 8, None),
                                               (10, 2, 48, 16, None), (6, 3, 80, 8, 50), (16, 1, 64, 32, None),
                                               (5, 5, 112, 16, 129), (4, 2, 256, 16, None), (6, 2, 128, 8, 300),
                                               (8, 8, 128, 128, None), (4, 1, 128, 4, None)])
@pytest.mark.parametrize("splits", [1, 3, 8, 16, 32])
def test_attention_decode_kernel(nq, nkv, d, P, window, splits):
    before = [0, 1, 63, 64, 65, 700, 127, 2000]           # one key; page and chunk edges; long rows
    qlens = [1] * len(before)
    lay, wide, k_pages, v_pages, _, _, _, want = build_case(before, qlens, nq, nkv, d, P, window, 400, 3, standout_row=5)
    out = ops().attention_decode(wide, wide.stride(0), k_pages, v_pages, lay["block_table"], lay["page_base"],
                                 lay["token_row"], lay["positions"], len(before), nq, nkv, d, d ** -0.5, window, splits)
    assert torch.allclose(out.double().cpu(), want, **BF16_TOL)
    if d == 128:       # head size 128 took the TMA variant above: the cp.async variant must agree
        other = ops().attention_decode(wide, wide.stride(0), k_pages, v_pages, lay["block_table"], lay["page_base"],
                                       lay["token_row"], lay["positions"], len(before), nq, nkv, d, d ** -0.5, window,
                                       splits, use_tma=False)
        assert torch.allclose(other.double().cpu(), want, **BF16_TOL)
    if d == 128 and P >= 8:
        # up to sixteen splits the TMA variant merged them inside the kernel (a cluster); with scratch given
        # it takes the separate merge pass, which must agree
        n = len(before)
        scratch = (torch.empty((n, nq, splits, d), dtype=torch.float32, device=DEV),
                   torch.empty((n, nq, splits), dtype=torch.float32, device=DEV))
        counts = dict(ops().COUNTS)
        passes = ops().attention_decode(wide, wide.stride(0), k_pages, v_pages, lay["block_table"], lay["page_base"],
                                        lay["token_row"], lay["positions"], n, nq, nkv, d, d ** -0.5, window, splits,
                                        scratch=scratch)
        assert torch.allclose(passes.double().cpu(), want, **BF16_TOL)
        assert ops().COUNTS.get("attention_decode_merge", 0) - counts.get("attention_decode_merge", 0) == (splits > 1)
        assert ops().attention_decode_tma_error() == 0
    # a second run gives the same bits
    again = ops().attention_decode(wide, wide.stride(0), k_pages, v_pages, lay["block_table"], lay["page_base"],
                                   lay["token_row"], lay["positions"], len(before), nq, nkv, d, d ** -0.5, window, splits)
    assert torch.equal(out, again)


def test_attention_decode_token_list_leaves_other_rows():
    nq, nkv, d, P = 8, 2, 64, 16
    before, qlens = [10, 300, 77, 5], [1, 1, 1, 1]
    lay, wide, k_pages, v_pages, _, _, _, want = build_case(before, qlens, nq, nkv, d, P, None, 100, 4)
    out = torch.full((4, nq * d), 7.0, device=DEV, dtype=torch.bfloat16)
    chosen = torch.tensor([3, 1], dtype=torch.int32, device=DEV)
    ops().attention_decode(wide, wide.stride(0), k_pages, v_pages, lay["block_table"], lay["page_base"],
                           lay["token_row"], lay["positions"], 4, nq, nkv, d, d ** -0.5, None, 4, token_list=chosen,
                           out=out)
    assert torch.allclose(out[[1, 3]].double().cpu(), want[[1, 3]], **BF16_TOL)
    assert bool((out[[0, 2]] == 7.0).all())


def test_attention_decode_refuses_what_it_cannot_compute():
    from acorninfer_b200.kernels.ops import KernelError
    assert not ops().attention_decode_supported(34, 2, 64)       # 17 query heads a group
    assert not ops().attention_decode_supported(8, 2, 72)        # head size not a multiple of 16
    with pytest.raises(KernelError):
        x = torch.zeros(1, 8 * 72 * 2, device=DEV, dtype=torch.bfloat16)
        pages = torch.zeros(2, 2, 16, 72, device=DEV, dtype=torch.bfloat16)
        i32 = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops().attention_decode(x, x.stride(0), pages, pages, i32.view(1, 1), i32, i32, i32, 1, 8, 2, 72, 1.0, None, 1)


@pytest.mark.parametrize("nq,nkv,d,P,window", [(32, 8, 128, 16, None), (4, 2, 16, 4, None), (8, 1, 32, 8, None),
                                               (10, 2, 48, 16, None), (6, 3, 80, 8, 50), (5, 5, 112, 32, 129)])
def test_attention_prefill_kernel(nq, nkv, d, P, window):
    # portions that start inside a request, tiles that end inside a page, single tokens beside them
    before = [0, 130, 64, 500, 0, 31]
    qlens = [150, 64, 1, 2, 1, 65]
    lay, wide, k_pages, v_pages, row_start, row_pos, tiles, want = build_case(before, qlens, nq, nkv, d, P, window, 400, 5,
                                                                             standout_row=3)
    out = ops().attention_prefill(wide, wide.stride(0), k_pages, v_pages, lay["block_table"], lay["page_base"],
                                  row_start, row_pos, tiles, sum(qlens), nq, nkv, d, d ** -0.5, window)
    assert torch.allclose(out.double().cpu(), want, **BF16_TOL)
    plain_out = ops().attention_plain(wide, wide.stride(0), k_pages, v_pages, lay["block_table"], lay["page_base"],
                                      lay["token_row"], lay["positions"], sum(qlens), nq, nkv, d, d ** -0.5, window)
    assert torch.allclose(out.float(), plain_out.float(), **BF16_TOL)


@pytest.mark.parametrize("nq,nkv,P,window", [(32, 8, 16, None), (4, 4, 8, None), (6, 2, 64, None), (8, 1, 16, 200),
                                             (2, 1, 128, None), (10, 2, 32, 300)])
def test_attention_prefill_tcgen05_kernel(nq, nkv, P, window):
    """The tcgen05/TMA prefill kernel (head size 128): portions that start inside a request and inside
    a page, tiles that end inside a page, rows shorter than a tile, a far key that decides."""
    d = 128
    before = [0, 130, 77, 500, 31, 1000]
    qlens = [300, 128, 129, 40, 65, 32]
    lay, wide, k_pages, v_pages, row_start, row_pos, _, want = build_case(before, qlens, nq, nkv, d, P, window, 200, 6,
                                                                         standout_row=3)
    tiles = torch.tensor([(r, q0) for r, n in enumerate(qlens) for q0 in range(0, n, 128)], dtype=torch.int32,
                         device=DEV).view(-1, 2)
    out = ops().attention_prefill_tc(wide, wide.stride(0), k_pages, v_pages, lay["block_table"], lay["page_base"],
                                     row_start, row_pos, tiles, sum(qlens), nq, nkv, d, d ** -0.5, window)
    assert ops().attention_tc_error() == 0
    assert torch.allclose(out.double().cpu(), want, **BF16_TOL)
    again = ops().attention_prefill_tc(wide, wide.stride(0), k_pages, v_pages, lay["block_table"], lay["page_base"],
                                       row_start, row_pos, tiles, sum(qlens), nq, nkv, d, d ** -0.5, window)
    assert torch.equal(out, again)
