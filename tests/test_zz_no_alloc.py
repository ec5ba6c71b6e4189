"""The entry point for callers that cannot allocate device memory (decode attention whose
split-K scratch is a fixed array inside the library): called through its exported C symbol,
twice in a row with different sizes, and compared with the ordinary entry point, which gets
its scratch from the caller.  Such callers exist (a process under a fixed memory budget, code
running where cudaMalloc is not allowed); for them the test also checks that a request beyond
the fixed array is refused with a readable message instead of computing anything.

Its result is also compared with a float64 computation of the same attention written here, so the
file stands on its own.  The file's name makes pytest collect it last: a run that stops at the first
failure has then already run every other test.
"""

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

from tests.paged import gather_from_pages, rows_layout

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def library():
    from acorninfer_b200.kernels.build import ensure_built
    lib = ctypes.CDLL(str(ensure_built()))
    lib.acorn_attention_decode_noalloc.argtypes = [
        c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
    lib.acorn_attention_decode_noalloc.restype = c_int
    lib.acorn_attention_decode_noalloc_needs.argtypes = [c_int, c_int, c_int, c_int]
    lib.acorn_attention_decode_noalloc_needs.restype = c_int64
    lib.acorn_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def case(before, nq, nkv, d, P, seed):
    torch.manual_seed(seed)
    n = len(before)
    lay = rows_layout(before, [1] * n, P, sum(-(-(b + 1) // P) for b in before) + 5, seed=seed)
    pages = max(max(t) for t in lay["tables"]) + 1
    k_pages = torch.randn(pages, nkv, P, d, device=DEV).to(torch.bfloat16)
    v_pages = torch.randn(pages, nkv, P, d, device=DEV).to(torch.bfloat16)
    qkv = torch.randn(n, (nq + 2 * nkv) * d, device=DEV).to(torch.bfloat16)
    return lay, qkv, k_pages, v_pages


def dense_float64(lay, qkv, k_pages, v_pages, before, nq, nkv, d, P):
    """Softmax attention of each row's single query over all its keys, in float64 on the host."""
    out = torch.empty(len(before), nq * d, dtype=torch.float64)
    for r, b in enumerate(before):
        k = gather_from_pages(k_pages.cpu(), lay["tables"][r], b + 1, P).double()     # [S, nkv, d]
        v = gather_from_pages(v_pages.cpu(), lay["tables"][r], b + 1, P).double()
        q = qkv[r, :nq * d].cpu().double().view(nq, d)
        for h in range(nq):
            g = h // (nq // nkv)
            p = torch.softmax((k[:, g] @ q[h]) * d ** -0.5, dim=0)
            out[r, h * d:(h + 1) * d] = p @ v[:, g]
    return out


def run_both(lib, lay, qkv, k_pages, v_pages, nq, nkv, d, splits):
    from acorninfer_b200.kernels import ops
    n = qkv.shape[0]
    # the ordinary entry point of the same kernel (scratch from the caller; head size 128 would
    # otherwise take the TMA variant, which merges its splits differently)
    want = ops.attention_decode(qkv, qkv.stride(0), k_pages, v_pages, lay["block_table"], lay["page_base"],
                                lay["token_row"], lay["positions"], n, nq, nkv, d, d ** -0.5, None, splits,
                                use_tma=False)
    got = torch.zeros_like(want)
    rc = lib.acorn_attention_decode_noalloc(
        qkv.data_ptr(), qkv.stride(0), got.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
        lay["block_table"].data_ptr(), lay["page_base"].data_ptr(), lay["block_table"].stride(0),
        lay["token_row"].data_ptr(), lay["positions"].data_ptr(), None, n, nq, nkv, d, k_pages.shape[2],
        d ** -0.5, 0, splits, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, got, want


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    lib = library()
    # first call: long rows, many splits (fills much of the scratch)
    before = [900, 64, 2047, 1, 500, 333]
    a = case(before, 32, 8, 128, 16, seed=1)
    rc, got, want = run_both(lib, *a, 32, 8, 128, 8)
    assert rc == 0, lib.acorn_noalloc_last_error()
    assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2) and torch.equal(got, want)
    assert torch.allclose(got.double().cpu(), dense_float64(*a, before, 32, 8, 128, 16), atol=2e-2, rtol=2e-2)
    # second call right after: other sizes, fewer splits, short rows whose later splits are empty;
    # what the first call left in the scratch must not matter
    b = case([10, 70, 3], 10, 2, 48, 8, seed=2)
    rc, got, want = run_both(lib, *b, 10, 2, 48, 5)
    assert rc == 0, lib.acorn_noalloc_last_error()
    assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2) and torch.equal(got, want)
    assert torch.allclose(got.double().cpu(), dense_float64(*b, [10, 70, 3], 10, 2, 48, 8), atol=2e-2, rtol=2e-2)
    # one split needs no scratch at all
    rc, got, want = run_both(lib, *b, 10, 2, 48, 1)
    assert rc == 0 and torch.equal(got, want)


def test_no_alloc_entry_point_refuses_what_exceeds_its_array():
    lib = library()
    assert lib.acorn_attention_decode_noalloc_needs(8, 32, 128, 4) == 8 * 32 * 4 * 129
    assert lib.acorn_attention_decode_noalloc_needs(8, 32, 128, 1) == 0
    lay, qkv, k_pages, v_pages = case([5] * 600, 32, 8, 128, 16, seed=3)       # 600 * 32 * 32 * 129 floats
    out = torch.full((600, 32 * 128), 3.0, device=DEV, dtype=torch.bfloat16)
    rc = lib.acorn_attention_decode_noalloc(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
        lay["block_table"].data_ptr(), lay["page_base"].data_ptr(), lay["block_table"].stride(0),
        lay["token_row"].data_ptr(), lay["positions"].data_ptr(), None, 600, 32, 8, 128, 16, 128 ** -0.5, 0, 32,
        torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 10002
    msg = lib.acorn_noalloc_last_error().decode()
    assert "floats of scratch wanted" in msg and "2097152" in msg
    assert bool((out == 3.0).all())                                            # nothing was computed
