"""Python faces of the CUDA kernels: argument checks, then one launch on the current stream.

The shared library is loaded with ctypes on first use (compiled first if stale).
Every wrapper checks dtype, device, contiguity and the sizes the kernel supports and
raises ``KernelError`` for what it cannot compute; there is no other implementation
to fall back to.  Tensors are passed as raw device pointers.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from .build import ensure_built


class KernelError(RuntimeError):
    pass


_lib = None
F32, BF16 = 0, 1


def lib():
    if _TIMER is not None and _lib is not None:
        return _TimedLib(_lib)
    return _load()


def _load():
    global _lib
    if _lib is None:
        if not torch.cuda.is_available():
            raise KernelError("acorninfer_b200 needs a CUDA device (sm_100a); none is visible and there is no CPU path")
        path = ensure_built()
        _lib = ctypes.CDLL(str(path))
        for name in dir(_Sigs):
            if name.startswith("acorn_"):
                fn = getattr(_lib, name, None)
                if fn is None:
                    raise KernelError(f"{path} lacks the symbol {name}: stale build?")
                fn.argtypes = getattr(_Sigs, name)
                fn.restype = c_int
        _lib.acorn_uniform.restype = c_float
        _init_error_word(_lib)
    return _lib


_error_word: ctypes.c_int | None = None       # pinned host memory that kernels write when a bounded wait gives up
_KERNEL_NAMES = {1: "gemm_tcgen05", 2: "attention_prefill_tc", 3: "attention_decode_tma", 4: "gemm_tcgen05_pair", 9: "error-word self-test"}


def _init_error_word(library) -> None:
    global _error_word
    host, dev = c_void_p(), c_void_p()
    code = library.acorn_error_word_alloc(ctypes.byref(host), ctypes.byref(dev))
    if code != 0 or not host.value:
        raise KernelError(f"could not allocate the kernels' error word: CUDA error {code}")
    for setter in ("acorn_gemm_tc_set_error_word", "acorn_attention_tc_set_error_word",
                   "acorn_attention_decode_tma_set_error_word", "acorn_selftest_set_error_word",
                   "acorn_gemm_tc_pair_set_error_word"):
        code = getattr(library, setter)(dev)
        if code != 0:
            raise KernelError(f"{setter}: CUDA error {code}")
    _error_word = ctypes.c_int.from_address(host.value)


def raise_on_kernel_error() -> None:
    """Raises if a kernel of a step that has completed gave up a bounded wait (its results are not
    valid).  Costs a read of host memory: callers look after every step whose results they read."""
    if _error_word is None or _error_word.value == 0:
        return
    word = _error_word.value
    _error_word.value = 0
    for getter in (gemm_tc_error, attention_tc_error, attention_decode_tma_error, gemm_tc_pair_error):   # clear the kernels' own flags
        getter()
    raise KernelError(f"kernel {_KERNEL_NAMES.get(word // 100, word // 100)} gave up a bounded wait at point "
                      f"{word % 100}: the results of the step are not valid")


def error_word_selftest(point: int) -> None:
    """Launches a kernel that does nothing but report ``point`` the way a failing kernel would."""
    _ok(lib().acorn_error_word_selftest(point, _stream()), "error_word_selftest")


class _Sigs:
    acorn_embed = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    acorn_patch_tokens = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
    acorn_add_rmsnorm = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]
    acorn_swiglu = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    acorn_cast = [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]
    acorn_qk_rope_kv = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                        c_int, c_void_p]
    acorn_attention_plain = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                             c_void_p]
    acorn_attention_decode = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                              c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                              c_int, c_void_p, c_void_p, c_void_p]
    acorn_attention_decode_supported = [c_int, c_int, c_int]
    acorn_attention_decode_tma_main = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                       c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                       c_float, c_int, c_int, c_void_p, c_void_p, c_void_p]
    acorn_attention_decode_tma_supported = [c_int, c_int, c_int, c_int]
    acorn_attention_decode_tma_merges = [c_int, c_int]
    acorn_attention_decode_tma_error = []
    acorn_attention_decode_merge = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    acorn_attention_prefill = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                               c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                               c_void_p]
    acorn_attention_prefill_supported = [c_int, c_int, c_int]
    acorn_gemm_tc = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                     c_void_p]
    acorn_attention_prefill_tc = [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                  c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_int, c_void_p]
    acorn_attention_prefill_tc_supported = [c_int, c_int, c_int, c_int]
    acorn_attention_tc_error = []
    acorn_gemm_tc_ex = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                        c_int, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]
    acorn_gemm_tc_qkv_rope = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                              c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
    acorn_gemm_tc_supported = [c_int64, c_int64, c_int64, c_int64, c_int64]
    acorn_gemm_tc_pair = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                          c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]
    acorn_gemm_tc_pair_qkv_rope = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int,
                                   c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                   c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                                   c_void_p]
    acorn_rope_table = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
    acorn_gemm_tc_pair_error = []
    acorn_gemm_tc_error = []
    acorn_gemm_f32 = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]
    acorn_sample = [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                    c_void_p, c_void_p, c_void_p]
    acorn_uniform = [ctypes.c_uint64, ctypes.c_uint64]
    acorn_random_fill = [c_void_p, c_int64, ctypes.c_uint64, ctypes.c_uint64, c_float, c_float, c_int, c_void_p]
    acorn_error_word_alloc = [c_void_p, c_void_p]
    acorn_error_word_selftest = [c_int, c_void_p]
    acorn_gemm_tc_set_error_word = [c_void_p]
    acorn_attention_tc_set_error_word = [c_void_p]
    acorn_attention_decode_tma_set_error_word = [c_void_p]
    acorn_selftest_set_error_word = [c_void_p]
    acorn_gemm_tc_pair_set_error_word = [c_void_p]


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = None


def _stream() -> int:
    """The current CUDA stream's handle (also the capture stream while a graph is captured)."""
    global _device_index
    if _raw_stream is not None:
        if _device_index is None:
            _device_index = torch.cuda.current_device()      # the engine works on one device
        return _raw_stream(_device_index)
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _check(t: torch.Tensor, name: str, dtype=None, dims: int | None = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got shape {tuple(t.shape)}")


LAUNCHES = 0      # kernels of this library launched so far (for reports)
COUNTS: dict[str, int] = {}    # the same by entry point: tests use it to see which kernel a path really took


class KernelTimer:
    """Per-launch device times of everything launched while it is active (``with kernel_timer() as t``):
    a CUDA event before and after every launch of this library, and around the library matrix products
    of ``linear``.  The events keep kernels from overlapping (no programmatic dependent launch across
    them) and nothing may be captured meanwhile, so the times are those of each kernel alone, in the
    order and with the data of a real step.  ``records()`` gives ``[(entry point, tag, microseconds)]``
    after a synchronize; the tag tells launches of one entry point apart (a product's M x N x K)."""

    def __init__(self):
        self._events: list = []
        self._open = None

    def begin(self) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._open = ev

    def end(self, what: str, tag: str = "") -> None:
        if self._open is None:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._events.append((what, tag, self._open, ev))
        self._open = None

    def records(self) -> list[tuple[str, str, float]]:
        torch.cuda.synchronize()
        return [(what, tag, a.elapsed_time(b) * 1e3) for what, tag, a, b in self._events]


_TIMER: KernelTimer | None = None


class kernel_timer:
    def __enter__(self) -> KernelTimer:
        global _TIMER
        if _TIMER is not None:
            raise KernelError("kernel_timer: already active")
        _load()
        _TIMER = KernelTimer()
        return _TIMER

    def __exit__(self, *exc) -> None:
        global _TIMER
        _TIMER = None


class _TimedLib:
    """The library while a timer is active: every entry point records the start event first (the end
    event is recorded where the wrapper reports the launch, ``_ok``)."""

    def __init__(self, library):
        self._library = library

    def __getattr__(self, name):
        fn = getattr(self._library, name)
        if not name.startswith("acorn_") or name.endswith(("_supported", "_error", "_merges")):
            return fn

        def timed(*args):
            if _TIMER is not None:
                _TIMER.begin()
            return fn(*args)
        return timed


def _ok(code: int, what: str, tag: str = "") -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        COUNTS[what] = COUNTS.get(what, 0) + 1
        if _TIMER is not None:
            _TIMER.end(what, tag)
        return
    if code == 10001:
        raise KernelError(f"{what}: sizes or dtypes not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {code}")


def _ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


# ------------------------------------------------------------------ elementwise / norm


def embed(ids: torch.Tensor, table: torch.Tensor, out32: torch.Tensor | None = None) -> torch.Tensor:
    """out32[t] = table[ids[t]] as float32.  ids int32 [T]; table [V, H]."""
    _check(ids, "ids", torch.int32, 1)
    _check(table, "table", None, 2)
    T, H = ids.numel(), table.shape[1]
    if out32 is None:
        out32 = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _check(out32, "out32", torch.float32, 2)
    _ok(lib().acorn_embed(ids.data_ptr(), table.data_ptr(), out32.data_ptr(), T, H, dtype_code(table.dtype),
                          _stream()), "embed")
    return out32


def patch_tokens(token_ids: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, src_tokens: torch.Tensor) -> None:
    """token_ids[dst[i]] = src_tokens[src[i]] (all int32, on the device)."""
    for t, n in ((token_ids, "token_ids"), (dst, "dst"), (src, "src"), (src_tokens, "src_tokens")):
        _check(t, n, torch.int32, 1)
    if dst.numel() != src.numel():
        raise KernelError("patch_tokens: dst and src differ in length")
    _ok(lib().acorn_patch_tokens(token_ids.data_ptr(), dst.data_ptr(), src.data_ptr(), src_tokens.data_ptr(),
                                 dst.numel(), _stream()), "patch_tokens")


def add_rmsnorm(resid32: torch.Tensor, delta: torch.Tensor | None, weight32: torch.Tensor, eps: float,
                out_dtype: torch.dtype, row_idx: torch.Tensor | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """resid32 += delta (in place, unless row_idx is given); returns rmsnorm(resid32) * weight.

    With ``row_idx`` (int32 [R]) only those rows are normed, into rows 0..R-1 of the result,
    and the residual is left as it is.
    """
    _check(resid32, "resid32", torch.float32, 2)
    _check(weight32, "weight", torch.float32, 1)
    H = resid32.shape[1]
    if weight32.numel() != H:
        raise KernelError(f"norm weight has {weight32.numel()} elements, width is {H}")
    if delta is not None:
        _check(delta, "delta", out_dtype, 2)
        if delta.shape != resid32.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match the residual {tuple(resid32.shape)}")
    rows = resid32.shape[0]
    if row_idx is not None:
        _check(row_idx, "row_idx", torch.int32, 1)
        rows = row_idx.numel()
    if out is None:
        out = torch.empty((rows, H), dtype=out_dtype, device=resid32.device)
    _check(out, "out", out_dtype, 2)
    _ok(lib().acorn_add_rmsnorm(resid32.data_ptr(), _ptr(delta), weight32.data_ptr(), out.data_ptr(),
                                _ptr(row_idx), rows, H, float(eps), dtype_code(out_dtype), _stream()),
        "add_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, block: int | None = None) -> torch.Tensor:
    """silu(gate) * up.  A row holds, per block of ``block`` outputs, the gate values then the up
    values; the default (block = I) is the plain layout ``[gate | up]``."""
    _check(gate_up, "gate_up", None, 2)
    T, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("gate_up must have an even width")
    block = block or two_i // 2
    if (two_i // 2) % block:
        raise KernelError(f"swiglu: block {block} does not divide the width {two_i // 2}")
    if out is None:
        out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(out, "out", gate_up.dtype, 2)
    _ok(lib().acorn_swiglu(gate_up.data_ptr(), out.data_ptr(), T, two_i // 2, block, dtype_code(gate_up.dtype),
                           _stream()), "swiglu")
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _check(x, "x")
    if x.dtype == dtype:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _ok(lib().acorn_cast(x.data_ptr(), out.data_ptr(), x.numel(), dtype_code(x.dtype), dtype_code(dtype),
                         _stream()), "cast")
    return out


# ------------------------------------------------------------------ attention pieces


def qk_rope_kv(qkv: torch.Tensor, q_weight32: torch.Tensor | None, k_weight32: torch.Tensor | None,
               inv_freq: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor,
               block_table: torch.Tensor, page_base: torch.Tensor, k_pages: torch.Tensor | None,
               v_pages: torch.Tensor | None, num_heads: int, num_kv_heads: int, head_dim: int,
               rotary_dim: int, interleaved: bool, eps: float, write_kv: bool = True) -> None:
    """Per-head q/k norm, rotary encoding, K/V page write; q is updated in place inside ``qkv``."""
    _check(qkv, "qkv", None, 2)
    T = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"qkv width {qkv.shape[1]} != (nq + 2 nkv) * d")
    if head_dim > 1024 or rotary_dim > head_dim or rotary_dim % 2:
        raise KernelError(f"head_dim {head_dim} / rotary_dim {rotary_dim} not supported (d <= 1024, even rotary_dim <= d)")
    _check(inv_freq, "inv_freq", torch.float32, 1)
    if inv_freq.numel() != rotary_dim // 2:
        raise KernelError("inv_freq must have rotary_dim / 2 entries")
    for t, n in ((positions, "positions"), (token_row, "token_row"), (page_base, "page_base")):
        _check(t, n, torch.int32, 1)
    _check(block_table, "block_table", torch.int32, 2)
    for w, n in ((q_weight32, "q_norm weight"), (k_weight32, "k_norm weight")):
        if w is not None:
            _check(w, n, torch.float32, 1)
            if w.numel() != head_dim:
                raise KernelError(f"{n} must have head_dim entries")
    P = 0
    if write_kv:
        _check(k_pages, "k_pages", qkv.dtype, 4)
        _check(v_pages, "v_pages", qkv.dtype, 4)
        if k_pages.shape[1] != num_kv_heads or k_pages.shape[3] != head_dim or v_pages.shape != k_pages.shape:
            raise KernelError(f"cache pages {tuple(k_pages.shape)} do not fit nkv={num_kv_heads}, d={head_dim}")
        P = k_pages.shape[2]
    _ok(lib().acorn_qk_rope_kv(qkv.data_ptr(), _ptr(q_weight32), _ptr(k_weight32), inv_freq.data_ptr(),
                               positions.data_ptr(), token_row.data_ptr(), block_table.data_ptr(),
                               page_base.data_ptr(), block_table.stride(0), _ptr(k_pages), _ptr(v_pages), T,
                               num_heads, num_kv_heads, head_dim, rotary_dim, 1 if interleaved else 0,
                               max(P, 1), float(eps), 1 if write_kv else 0, dtype_code(qkv.dtype), _stream()),
        "qk_rope_kv")


def attention_plain(q: torch.Tensor, q_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                    block_table: torch.Tensor, page_base: torch.Tensor, token_row: torch.Tensor,
                    positions: torch.Tensor, num_tokens: int, num_heads: int, num_kv_heads: int, head_dim: int,
                    scale: float, window: int | None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Paged causal attention for any mix of rows; ``q`` may be the head of a wider buffer
    (row stride ``q_stride`` elements).  Returns [tokens, nq * d]."""
    if head_dim > 512:
        raise KernelError(f"plain attention supports head_dim <= 512, got {head_dim}")
    if num_heads % num_kv_heads:
        raise KernelError("num_heads must be a multiple of num_kv_heads")
    _check(k_pages, "k_pages", q.dtype, 4)
    _check(v_pages, "v_pages", q.dtype, 4)
    _check(block_table, "block_table", torch.int32, 2)
    if out is None:
        out = torch.empty((num_tokens, num_heads * head_dim), dtype=q.dtype, device=q.device)
    _check(out, "out", q.dtype, 2)
    _ok(lib().acorn_attention_plain(q.data_ptr(), q_stride, out.data_ptr(), k_pages.data_ptr(),
                                    v_pages.data_ptr(), block_table.data_ptr(), page_base.data_ptr(),
                                    block_table.stride(0), token_row.data_ptr(), positions.data_ptr(),
                                    num_tokens, num_heads, num_kv_heads, head_dim, k_pages.shape[2],
                                    float(scale), int(window or 0), dtype_code(q.dtype), _stream()),
        "attention_plain")
    return out


def attention_decode_supported(num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return bool(lib().acorn_attention_decode_supported(num_heads, num_kv_heads, head_dim))


def attention_prefill_supported(num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return bool(lib().acorn_attention_prefill_supported(num_heads, num_kv_heads, head_dim))


def attention_decode(q: torch.Tensor, q_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     block_table: torch.Tensor, page_base: torch.Tensor, token_row: torch.Tensor,
                     positions: torch.Tensor, num_tokens: int, num_heads: int, num_kv_heads: int, head_dim: int,
                     scale: float, window: int | None, num_splits: int, token_list: torch.Tensor | None = None,
                     out: torch.Tensor | None = None, scratch: tuple | None = None,
                     use_tma: bool | None = None) -> torch.Tensor:
    """Split-K decode attention (bfloat16) for single-token rows: the tokens 0..num_tokens-1, or
    those listed in ``token_list``.  ``out`` is [all tokens of the step, nq * d]; rows of tokens
    not handled are left as they are.  ``scratch`` = (part_o float32 [n, nq, splits, d],
    part_lse float32 [n, nq, splits]) is made here when absent and the kernel needs it (the TMA
    kernel merges up to sixteen splits without; give ``scratch`` to force the separate merge pass)."""
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_decode takes bfloat16")
    if not attention_decode_supported(num_heads, num_kv_heads, head_dim):
        raise KernelError(f"attention_decode does not take nq={num_heads}, nkv={num_kv_heads}, d={head_dim}")
    _check(k_pages, "k_pages", q.dtype, 4)
    _check(v_pages, "v_pages", q.dtype, 4)
    _check(block_table, "block_table", torch.int32, 2)
    n = num_tokens if token_list is None else token_list.numel()
    if n > 65535 or not (1 <= num_splits <= 32):
        raise KernelError(f"attention_decode: {n} tokens / {num_splits} splits beyond the grid limits")
    if out is None:
        out = torch.empty((num_tokens, num_heads * head_dim), dtype=q.dtype, device=q.device)
    P = k_pages.shape[2]
    if use_tma is None:
        use_tma = bool(lib().acorn_attention_decode_tma_supported(num_heads, num_kv_heads, head_dim, P))
    # the TMA kernel merges up to sixteen splits itself (a cluster, through shared memory): no scratch
    limit = lib().acorn_attention_decode_tma_merges(num_heads, num_kv_heads) if use_tma and scratch is None else 1
    in_kernel_merge = num_splits > 1 and (num_splits <= min(limit, 8) or (num_splits == 16 and limit >= 16))
    part_o = part_lse = None
    if num_splits > 1 and not in_kernel_merge:
        if scratch is None:
            scratch = (torch.empty((n, num_heads, num_splits, head_dim), dtype=torch.float32, device=q.device),
                       torch.empty((n, num_heads, num_splits), dtype=torch.float32, device=q.device))
        part_o, part_lse = scratch
        if part_o.numel() < n * num_heads * num_splits * head_dim or part_lse.numel() < n * num_heads * num_splits:
            raise KernelError("attention_decode: scratch too small")
    if use_tma:
        # head size 128: K/V tiles by TMA (attention_decode_tma.cu); more than sixteen splits, or splits
        # with scratch given, end in the common merge pass
        _ok(lib().acorn_attention_decode_tma_main(
            q.data_ptr(), q_stride, out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
            block_table.data_ptr(), page_base.data_ptr(), block_table.stride(0), token_row.data_ptr(),
            positions.data_ptr(), _ptr(token_list), n, num_heads, num_kv_heads, head_dim, P, float(scale),
            int(window or 0), num_splits, _ptr(part_o), _ptr(part_lse), _stream()), "attention_decode_tma")
        if num_splits > 1 and not in_kernel_merge:
            _ok(lib().acorn_attention_decode_merge(part_o.data_ptr(), part_lse.data_ptr(), out.data_ptr(),
                                                   _ptr(token_list), n, num_heads, head_dim, num_splits, _stream()),
                "attention_decode_merge")
        return out
    _ok(lib().acorn_attention_decode(q.data_ptr(), q_stride, out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
                                     block_table.data_ptr(), page_base.data_ptr(), block_table.stride(0),
                                     token_row.data_ptr(), positions.data_ptr(), _ptr(token_list), n, num_heads,
                                     num_kv_heads, head_dim, P, float(scale), int(window or 0),
                                     num_splits, _ptr(part_o), _ptr(part_lse), _stream()), "attention_decode")
    return out


def attention_decode_tma_error() -> int:
    return int(lib().acorn_attention_decode_tma_error())


def attention_prefill(q: torch.Tensor, q_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_table: torch.Tensor, page_base: torch.Tensor, row_start: torch.Tensor,
                      row_pos: torch.Tensor, tiles: torch.Tensor, num_tokens: int, num_heads: int,
                      num_kv_heads: int, head_dim: int, scale: float, window: int | None,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """Tensor-core prefill attention (bfloat16) for the query tiles listed in ``tiles``
    (int32 [n, 2]: row, first token within the row; 64 tokens a tile at most)."""
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill takes bfloat16")
    if not attention_prefill_supported(num_heads, num_kv_heads, head_dim):
        raise KernelError(f"attention_prefill does not take nq={num_heads}, nkv={num_kv_heads}, d={head_dim}")
    _check(k_pages, "k_pages", q.dtype, 4)
    _check(v_pages, "v_pages", q.dtype, 4)
    _check(block_table, "block_table", torch.int32, 2)
    _check(tiles, "tiles", torch.int32, 2)
    if out is None:
        out = torch.empty((num_tokens, num_heads * head_dim), dtype=q.dtype, device=q.device)
    _ok(lib().acorn_attention_prefill(q.data_ptr(), q_stride, out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
                                      block_table.data_ptr(), page_base.data_ptr(), block_table.stride(0),
                                      row_start.data_ptr(), row_pos.data_ptr(), tiles.data_ptr(), tiles.shape[0],
                                      num_heads, num_kv_heads, head_dim, k_pages.shape[2], float(scale),
                                      int(window or 0), _stream()), "attention_prefill")
    return out


def attention_prefill_tc_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    return bool(lib().acorn_attention_prefill_tc_supported(num_heads, num_kv_heads, head_dim, page_size))


def attention_prefill_tc(q: torch.Tensor, q_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                         block_table: torch.Tensor, page_base: torch.Tensor, row_start: torch.Tensor,
                         row_pos: torch.Tensor, tiles: torch.Tensor, num_tokens: int, num_heads: int,
                         num_kv_heads: int, head_dim: int, scale: float, window: int | None,
                         out: torch.Tensor | None = None) -> torch.Tensor:
    """tcgen05/TMA prefill attention (bfloat16, head size 128) for the query tiles listed in
    ``tiles`` (int32 [n, 2]: row, first token within the row; 128 tokens a tile at most).  CTAs
    start in the order of the list: give the tiles that read the most keys first."""
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc takes bfloat16")
    _check(k_pages, "k_pages", q.dtype, 4)
    _check(v_pages, "v_pages", q.dtype, 4)
    if not attention_prefill_tc_supported(num_heads, num_kv_heads, head_dim, k_pages.shape[2]):
        raise KernelError(f"attention_prefill_tc does not take nq={num_heads}, nkv={num_kv_heads}, d={head_dim}, "
                          f"page={k_pages.shape[2]}")
    if q_stride % 8 or q.data_ptr() % 16:
        raise KernelError("attention_prefill_tc: q rows must be 16-byte aligned")
    _check(block_table, "block_table", torch.int32, 2)
    _check(tiles, "tiles", torch.int32, 2)
    if out is None:
        out = torch.empty((num_tokens, num_heads * head_dim), dtype=q.dtype, device=q.device)
    _ok(lib().acorn_attention_prefill_tc(q.data_ptr(), q_stride, num_tokens, out.data_ptr(), k_pages.data_ptr(),
                                         v_pages.data_ptr(), k_pages.shape[0], block_table.data_ptr(),
                                         page_base.data_ptr(), block_table.stride(0), row_start.data_ptr(),
                                         row_pos.data_ptr(), tiles.data_ptr(), tiles.shape[0], num_heads,
                                         num_kv_heads, head_dim, k_pages.shape[2], float(scale), int(window or 0),
                                         _stream()), "attention_prefill_tc")
    return out


def attention_tc_error() -> int:
    """0, or where a bounded wait inside the tcgen05 attention kernel gave up since the last call."""
    return int(lib().acorn_attention_tc_error())


# ------------------------------------------------------------------ matrix products


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """a [M, K] @ w [N, K]^T in true float32 (CUDA cores)."""
    _check(w, "w", torch.float32, 2)
    if a.dtype != torch.float32 or a.dim() != 2 or a.stride(1) != 1:
        raise KernelError("a must be float32 [M, K] with contiguous K")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"inner sizes differ: a has K={K}, w has K={w.shape[1]}")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _check(out, "out", torch.float32, 2)
    _ok(lib().acorn_gemm_f32(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                             out.stride(0), M, N, K, _stream()), "gemm_f32", f"{M}x{N}x{K}")
    return out


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.stride(1) == 1 and w.stride(1) == 1 and x.shape[1] == w.shape[1]
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(lib().acorn_gemm_tc_supported(x.shape[0], w.shape[0], x.shape[1], x.stride(0), w.stride(0))))


_SMS: dict = {}


def device_sms(device) -> int:
    """Multiprocessors of ``device`` (asked of the driver once)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _SMS:
        _SMS[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _SMS[key]


def gemm_tc_plan(M: int, N: int, K: int, num_sms: int = 148) -> tuple[int, int]:
    """(splits of the K range, CTAs to an SM) for a product on the tcgen05 kernel.

    Splits: a cluster of that many CTAs per output tile, a power of two, at most 8, chosen so that a
    matrix with few 128-row tiles still puts one to two CTAs on every SM.  CTAs to an SM: two, with
    a deep ring, or three with a short one (up to 32 rows).  ``num_sms`` defaults to a B200's 148;
    launches pass the device's own count.  An SM takes in about 66 GB/s, so the SM
    with the most tiles sets the time: 192 tiles on 148 SMs leave 44 SMs with two tiles (2.0 tiles'
    worth), while 384 half tiles, three to an SM, leave none with more than three halves (1.5).  The
    second form is taken for unsplit matrices with 1 to 1.5 tiles to an SM; where K is split
    already it gained nothing."""
    rows = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
    tiles = -(-N // 128) * -(-M // rows)
    kblocks = -(-K // 64)
    splits = 1
    while splits < 8 and tiles * splits * 2 <= 2 * num_sms and kblocks // (splits * 2) >= 4:
        splits *= 2
    if rows <= 64 and splits == 1 and kblocks >= 8 and num_sms < tiles and tiles * 2 <= 3 * num_sms:
        return 2, 3                     # more tiles than SMs, fewer than 1.5 to an SM (measured: 36.0 -> 33.3 us)
    return splits, 2


def gemm_tc_splits(M: int, N: int, K: int) -> int:
    return gemm_tc_plan(M, N, K)[0]


# At or below this many rows the tcgen05 kernel (weights on the 128-row side of the MMA) streams the
# weight matrix at least as fast as the library product; above it the library's larger tiles win.
GEMM_TC_MAX_ROWS = 32
# The paired kernel (256 x 256 tiles, a pair of SMs to a tile at a time, fused epilogues) is used from
# this many rows on, where its tiles fill the device: see ``pair_rows_ok``.
GEMM_PAIR_MIN_ROWS = 256
GEMM_PAIR_MAX_ROWS = 3072
GEMM_PAIR_MIN_FILL = 0.8          # for every product of a layer, when the whole layer is fused
GEMM_PAIR_MIN_FILL_ALONE = 0.6    # for the widest product taken alone (gate/up with SwiGLU) ...
GEMM_PAIR_ALONE_MAX_ROWS = 8192
GEMM_PAIR_ALONE_MIN_K = 2048      # ... whose K must be long enough for a tile's k-steps to hide its epilogue


def pair_fill(num_rows: int, width: int, num_sms: int = 148) -> float:
    """How full the paired kernel's rounds are for a product of ``num_rows`` rows and ``width`` output
    columns: its tiles of 256 x 256 are taken in rounds of one tile to a pair of SMs; the product's
    elements over those the rounds could hold (128 full tiles on 74 pairs: two rounds, 0.86; 96 tiles:
    two rounds, 0.65; 257 rows: every second tile holds one row)."""
    pairs = max(num_sms // 2, 1)
    tiles = -(-num_rows // 256) * -(-width // 256)
    return num_rows * width / (-(-tiles // pairs) * pairs * 65536)


def pair_rows_ok(num_rows: int, width: int, num_sms: int = 148, min_fill: float | None = None,
                 max_rows: int | None = None) -> bool:
    """Whether a product of ``num_rows`` rows and ``width`` output columns suits the paired kernel: its
    rounds must be filled to ``min_fill`` (``GEMM_PAIR_MIN_FILL`` if not given); below that the library's
    choice of tile shapes is faster.  Steps of more than ``max_rows`` rows (``GEMM_PAIR_MAX_ROWS`` if not
    given) run so long under the power cap that the library's kernel, which moves half the bytes from L2
    (multicast loads), keeps the higher clock: with every product of the layers on the paired kernel a step
    of 4,096 rows took 53.3 ms against 51.8 ms with the gate/up product alone on it, one of 6,144 rows 84.2
    against 80.9 (54.7 and 84.3 on the library alone); the gate/up product alone stops paying at about
    12,000 rows."""
    if num_rows < GEMM_PAIR_MIN_ROWS or num_rows > (GEMM_PAIR_MAX_ROWS if max_rows is None else max_rows):
        return False
    return pair_fill(num_rows, width, num_sms) >= (GEMM_PAIR_MIN_FILL if min_fill is None else min_fill)


@dataclass
class NormedRows:
    """Activations whose rows still lack their RMS factor: ``x = residual * norm weight`` and, per
    row, partial sums of ``residual^2`` (``ss`` [parts, rows]).  The matrix product that consumes
    them multiplies each output row by ``rsqrt(sum(ss) / width + eps)``: the norm costs no kernel."""

    x: torch.Tensor
    ss: torch.Tensor
    eps: float
    width: int


@dataclass
class AddNormEpilogue:
    """What the last product of a part does with its result instead of writing it: add it to the
    float32 residual stream (in place) and hand on ``NormedRows`` for the norm with this weight."""

    resid32: torch.Tensor
    weight32: torch.Tensor
    eps: float


@dataclass
class RopeKvEpilogue:
    """What the q/k/v product of an attention layer with head size 128 does with its result instead of
    writing it: per-head RMSNorm of the query and key heads (weights or None), rotation of the whole
    head in half pairing by ``position * inv_freq``, query heads to the output, keys and values to the
    token's slot in its cache pages (``k_pages`` None: they are dropped).  The same arithmetic as
    ``qk_rope_kv`` after a plain product, without the bfloat16 rounding in between."""

    positions: torch.Tensor
    token_row: torch.Tensor
    block_table: torch.Tensor
    page_base: torch.Tensor
    k_pages: torch.Tensor | None
    v_pages: torch.Tensor | None
    q_weight32: torch.Tensor | None
    k_weight32: torch.Tensor | None
    inv_freq: torch.Tensor
    num_heads: int
    num_kv_heads: int
    eps: float
    cos_sin: torch.Tensor | None = None      # [M, 128] float32 from ``rope_table``: spares the epilogue its sincosf


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """[tokens, 2 * len(inv_freq)] float32: cos, then sin, of position * inv_freq for every token."""
    _check(positions, "positions", torch.int32, 1)
    _check(inv_freq, "inv_freq", torch.float32, 1)
    T, half = positions.numel(), inv_freq.numel()
    out = torch.empty((T, 2 * half), dtype=torch.float32, device=positions.device)
    _ok(lib().acorn_rope_table(positions.data_ptr(), inv_freq.data_ptr(), out.data_ptr(), T, half, _stream()), "rope_table")
    return out


def gemm_tc_qkv_rope(x, w: torch.Tensor, ep: RopeKvEpilogue, out: torch.Tensor | None = None) -> torch.Tensor:
    """The q/k/v product with ``RopeKvEpilogue``: returns [M, (nq + 2 nkv) * 128] bfloat16 whose first
    nq * 128 columns hold the finished query heads (the others are not written)."""
    rows = x if isinstance(x, NormedRows) else None
    xt = rows.x if rows is not None else x
    nq, nkv = ep.num_heads, ep.num_kv_heads
    M, K = xt.shape
    N = (nq + 2 * nkv) * 128
    if not gemm_tc_supported(xt, w) or w.shape[0] != N:
        raise KernelError(f"gemm_tc_qkv_rope does not take x {tuple(xt.shape)} {xt.dtype}, w {tuple(w.shape)} {w.dtype} "
                          f"for {nq}/{nkv} heads of 128")
    _check(ep.positions, "positions", torch.int32, 1)
    _check(ep.inv_freq, "inv_freq", torch.float32, 1)
    if ep.inv_freq.numel() != 64 or ep.positions.numel() < M:
        raise KernelError("gemm_tc_qkv_rope: inv_freq must have 64 entries and positions one per row")
    P = 1
    if ep.k_pages is not None:
        _check(ep.k_pages, "k_pages", torch.bfloat16, 4)
        _check(ep.v_pages, "v_pages", torch.bfloat16, 4)
        _check(ep.block_table, "block_table", torch.int32, 2)
        if tuple(ep.k_pages.shape[1:]) != (nkv, ep.k_pages.shape[2], 128) or ep.v_pages.shape != ep.k_pages.shape:
            raise KernelError("gemm_tc_qkv_rope: cache pages must be [pages, nkv, P, 128]")
        P = ep.k_pages.shape[2]
    for wt in (ep.q_weight32, ep.k_weight32):
        if wt is not None:
            _check(wt, "head norm weight", torch.float32, 1)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=xt.device)
    _check(out, "out", torch.bfloat16, 2)
    if M > GEMM_TC_MAX_ROWS:
        if ep.cos_sin is not None:
            _check(ep.cos_sin, "cos_sin", torch.float32, 2)
            if tuple(ep.cos_sin.shape) != (M, 128) or not ep.cos_sin.is_contiguous():
                raise KernelError("gemm_tc_qkv_rope: cos_sin must be contiguous [rows, 128]")
        pairs = device_sms(xt.device) // 2
        _ok(lib().acorn_gemm_tc_pair_qkv_rope(
            xt.data_ptr(), xt.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, K, pairs,
            rows.ss.data_ptr() if rows is not None else None, rows.ss.shape[0] if rows is not None else 0,
            rows.width if rows is not None else 0, float(rows.eps) if rows is not None else 0.0,
            ep.positions.data_ptr(), _ptr(ep.token_row), _ptr(ep.block_table), _ptr(ep.page_base),
            ep.block_table.stride(0) if ep.block_table is not None else 0, _ptr(ep.k_pages), _ptr(ep.v_pages),
            _ptr(ep.q_weight32), _ptr(ep.k_weight32), ep.inv_freq.data_ptr(), _ptr(ep.cos_sin), nq, nkv, P, float(ep.eps),
            _stream()), "gemm_tc_pair_qkv_rope", f"{M}x{N}x{K}")
        return out
    splits, per_sm = gemm_tc_plan(M, N, K, device_sms(xt.device))
    _ok(lib().acorn_gemm_tc_qkv_rope(
        xt.data_ptr(), xt.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, K, splits, per_sm,
        rows.ss.data_ptr() if rows is not None else None, rows.ss.shape[0] if rows is not None else 0,
        rows.width if rows is not None else 0, float(rows.eps) if rows is not None else 0.0,
        ep.positions.data_ptr(), _ptr(ep.token_row), _ptr(ep.block_table), _ptr(ep.page_base),
        ep.block_table.stride(0) if ep.block_table is not None else 0, _ptr(ep.k_pages), _ptr(ep.v_pages),
        _ptr(ep.q_weight32), _ptr(ep.k_weight32), ep.inv_freq.data_ptr(), nq, nkv, P, float(ep.eps), _stream()),
        "gemm_tc_qkv_rope", f"{M}x{N}x{K}")
    return out


def rope_kv_fusable(num_rows: int, dtype: torch.dtype, head_dim: int, rotary_dim: int, interleaved: bool) -> bool:
    """Whether the q/k/v product of such a layer can take ``RopeKvEpilogue`` (the row count is the
    caller's to check with ``fused_rows_ok``)."""
    return dtype == torch.bfloat16 and num_rows > 0 and head_dim == 128 and rotary_dim == 128 and not interleaved


def gemm_tc(x, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, splits: int | None = None,
            out: torch.Tensor | None = None, epilogue: AddNormEpilogue | None = None, swiglu: bool = False,
            per_sm: int = 2):
    """x [M, K] @ w [N, K]^T on tcgen05 tensor cores (bfloat16 in, float32 accumulate).

    ``x`` may be ``NormedRows`` (at most 64 rows): the rows' RMS factors are applied to the product.
    ``epilogue``: see ``AddNormEpilogue`` (returns ``NormedRows``).  ``swiglu``: ``w`` holds blocks
    of 64 gate rows and 64 up rows; returns ``silu(gate) * up`` [M, N / 2]."""
    rows = x if isinstance(x, NormedRows) else None
    xt = rows.x if rows is not None else x
    if not gemm_tc_supported(xt, w):
        raise KernelError(f"gemm_tc does not take x {tuple(xt.shape)} {xt.dtype} stride {xt.stride()}, "
                          f"w {tuple(w.shape)} {w.dtype}: bf16, K contiguous, K and strides multiples of 8")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tc writes bfloat16 or float32")
    M, K = xt.shape
    N = w.shape[0]
    if (rows is not None or epilogue is not None or swiglu) and M > 64:
        raise KernelError(f"gemm_tc: fused norm / SwiGLU epilogues take at most 64 rows, got {M}")
    if splits is None:
        splits, per_sm = gemm_tc_plan(M, N, K, device_sms(xt.device))
    mode, resid, ldr, norm_w, ss_out = 0, None, 0, None, None
    out_cols = N
    if epilogue is not None:
        if swiglu or out_dtype != torch.bfloat16:
            raise KernelError("gemm_tc: the add-norm epilogue writes bfloat16 and excludes SwiGLU")
        _check(epilogue.resid32, "resid32", torch.float32, 2)
        _check(epilogue.weight32, "norm weight", torch.float32, 1)
        if epilogue.resid32.shape != (M, N) or epilogue.weight32.numel() != N:
            raise KernelError("gemm_tc: residual / norm weight do not match the product's shape")
        mode, resid, ldr, norm_w = 1, epilogue.resid32, epilogue.resid32.stride(0), epilogue.weight32
        ss_out = torch.empty((-(-N // 128), M), dtype=torch.float32, device=xt.device)
    elif swiglu:
        if N % 128 or out_dtype != torch.bfloat16:
            raise KernelError("gemm_tc: SwiGLU epilogue needs N a multiple of 128 and bfloat16 output")
        mode, out_cols = 2, N // 2
    if out is None:
        out = torch.empty((M, out_cols), dtype=out_dtype, device=xt.device)
    _check(out, "out", out_dtype, 2)
    _ok(lib().acorn_gemm_tc_ex(
        xt.data_ptr(), xt.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, N, K,
        1 if out_dtype == torch.float32 else 0, int(splits), int(per_sm), mode,
        rows.ss.data_ptr() if rows is not None else None, rows.ss.shape[0] if rows is not None else 0,
        rows.width if rows is not None else 0, float(rows.eps) if rows is not None else 0.0,
        _ptr(resid), ldr, _ptr(norm_w), _ptr(ss_out), _stream()), "gemm_tc", f"{M}x{N}x{K}")
    if epilogue is not None:
        return NormedRows(out, ss_out, epilogue.eps, N)
    return out


def gemm_tc_pair(x, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, out: torch.Tensor | None = None,
                 epilogue: AddNormEpilogue | None = None, swiglu: bool = False, pairs: int | None = None):
    """x [M, K] @ w [N, K]^T in bfloat16 on pairs of CTAs (tcgen05 ``cta_group::2``), for many rows:
    tiles of 256 rows of ``x`` by 256 rows of ``w``, one pair of SMs to a tile at a time.  ``x`` as
    ``NormedRows``, ``epilogue`` and ``swiglu`` as in ``gemm_tc``."""
    rows = x if isinstance(x, NormedRows) else None
    xt = rows.x if rows is not None else x
    if not gemm_tc_supported(xt, w):
        raise KernelError(f"gemm_tc_pair does not take x {tuple(xt.shape)} {xt.dtype} stride {xt.stride()}, "
                          f"w {tuple(w.shape)} {w.dtype}: bf16, K contiguous, K and strides multiples of 8")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tc_pair writes bfloat16 or float32")
    M, K = xt.shape
    N = w.shape[0]
    mode, resid, ldr, norm_w, ss_out = 0, None, 0, None, None
    out_cols = N
    if epilogue is not None:
        if swiglu or out_dtype != torch.bfloat16:
            raise KernelError("gemm_tc_pair: the add-norm epilogue writes bfloat16 and excludes SwiGLU")
        _check(epilogue.resid32, "resid32", torch.float32, 2)
        _check(epilogue.weight32, "norm weight", torch.float32, 1)
        if epilogue.resid32.shape != (M, N) or epilogue.weight32.numel() != N:
            raise KernelError("gemm_tc_pair: residual / norm weight do not match the product's shape")
        mode, resid, ldr, norm_w = 1, epilogue.resid32, epilogue.resid32.stride(0), epilogue.weight32
        ss_out = torch.empty((2 * -(-N // 256), M), dtype=torch.float32, device=xt.device)
    elif swiglu:
        if N % 128 or out_dtype != torch.bfloat16:
            raise KernelError("gemm_tc_pair: SwiGLU epilogue needs N a multiple of 128 and bfloat16 output")
        mode, out_cols = 2, N // 2
    if out is None:
        out = torch.empty((M, out_cols), dtype=out_dtype, device=xt.device)
    _check(out, "out", out_dtype, 2)
    if pairs is None:
        pairs = device_sms(xt.device) // 2
    _ok(lib().acorn_gemm_tc_pair(
        xt.data_ptr(), xt.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, N, K,
        1 if out_dtype == torch.float32 else 0, int(pairs), mode,
        rows.ss.data_ptr() if rows is not None else None, rows.ss.shape[0] if rows is not None else 0,
        rows.width if rows is not None else 0, float(rows.eps) if rows is not None else 0.0,
        _ptr(resid), ldr, _ptr(norm_w), _ptr(ss_out), _stream()), "gemm_tc_pair", f"{M}x{N}x{K}")
    if epilogue is not None:
        return NormedRows(out, ss_out, epilogue.eps, N)
    return out


def gemm_tc_pair_error() -> int:
    """0, or where a bounded wait inside the paired tcgen05 GEMM gave up since the last call (clears it)."""
    return int(lib().acorn_gemm_tc_pair_error())


def gemm_tc_error() -> int:
    """0, or where a bounded wait inside the tcgen05 GEMM gave up since the last call (clears it)."""
    return int(lib().acorn_gemm_tc_error())


def fused_rows_ok(num_rows: int, dtype: torch.dtype, widths=None, num_sms: int = 148) -> bool:
    """Whether products of this many rows run on a tcgen05 kernel of this library with fused epilogues:
    the one-CTA kernel up to ``GEMM_TC_MAX_ROWS`` rows; for more rows the paired kernel, where every
    product of the part (``widths``: their output columns, one number or several) fills the device
    (``pair_rows_ok``)."""
    if dtype != torch.bfloat16 or num_rows <= 0:
        return False
    if num_rows <= GEMM_TC_MAX_ROWS:
        return True
    if widths is None:
        return False
    widths = (widths,) if isinstance(widths, int) else tuple(widths)
    return all(pair_rows_ok(num_rows, w, num_sms) for w in widths)


def linear(x, w: torch.Tensor, out_dtype: torch.dtype | None = None, epilogue: AddNormEpilogue | None = None,
           swiglu: bool = False, residual32: torch.Tensor | None = None):
    """x [T, K] times w [N, K] transposed.

    float32 operands: the CUDA-core kernel (no reduced-precision matrix mode).
    bfloat16 operands: up to GEMM_TC_MAX_ROWS rows the one-CTA tcgen05/TMA kernel of this library,
    above that the library matrix product (cuBLAS); float32 accumulation either way, and
    ``out_dtype=float32`` keeps the accumulator's precision (used for logits).
    A weight stored in float32 under a bfloat16 engine is multiplied in float32.
    ``x`` as ``NormedRows``, ``epilogue`` and ``swiglu`` exist on the tcgen05 kernels only: the one-CTA
    kernel up to GEMM_TC_MAX_ROWS rows, the paired kernel above (callers ask ``fused_rows_ok`` whether
    that pays for their sizes); asking for them with other operands is an error, not a silent detour.
    ``residual32`` ([T, N] float32) is an offer: where the product goes to the library it is
    added to ``residual32`` in place, in float32 (the library's C operand: the product is not
    rounded first), and None is returned; elsewhere the offer is ignored and the product returned.
    """
    fused = isinstance(x, NormedRows) or epilogue is not None or swiglu
    xt = x.x if isinstance(x, NormedRows) else x
    out_dtype = out_dtype or xt.dtype
    if fused:
        if not (xt.dtype == torch.bfloat16 and gemm_tc_supported(xt, w)):
            raise KernelError(f"linear: fused epilogues need a tcgen05 path (bf16, K a multiple of 8); got "
                              f"{tuple(xt.shape)} {xt.dtype} x {tuple(w.shape)} {w.dtype}")
        if xt.shape[0] > GEMM_TC_MAX_ROWS:
            return gemm_tc_pair(x, w, out_dtype, epilogue=epilogue, swiglu=swiglu)
        return gemm_tc(x, w, out_dtype, epilogue=epilogue, swiglu=swiglu)
    if w.dtype == torch.float32:
        y = gemm_f32(cast(x, torch.float32) if x.dtype != torch.float32 else x, w)
        return y if out_dtype == torch.float32 else cast(y, out_dtype)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported dtypes x={x.dtype}, w={w.dtype}")
    if x.shape[0] <= GEMM_TC_MAX_ROWS and gemm_tc_supported(x, w):
        return gemm_tc(x, w, out_dtype)
    if _TIMER is not None:
        _TIMER.begin()
    try:
        if residual32 is not None and residual32.dtype == torch.float32 and residual32.is_contiguous() \
                and tuple(residual32.shape) == (x.shape[0], w.shape[0]):
            torch.addmm(residual32, x, w.t(), out_dtype=torch.float32, out=residual32)
            return None
        if out_dtype == torch.float32:
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return torch.mm(x, w.t())
    finally:
        if _TIMER is not None:
            _TIMER.end("library_gemm", f"{x.shape[0]}x{w.shape[0]}x{x.shape[1]}")


# ------------------------------------------------------------------ sampling


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seed: torch.Tensor, counter: torch.Tensor, want_logprobs: bool = False):
    """One token per row of float32 logits.  Per-row parameters are device tensors:
    temperature/top_p float32, top_k int32, seed/counter int64 (used as unsigned)."""
    _check(logits, "logits", torch.float32, 2)
    R, V = logits.shape
    _check(temperature, "temperature", torch.float32, 1)
    _check(top_p, "top_p", torch.float32, 1)
    _check(top_k, "top_k", torch.int32, 1)
    _check(seed, "seed", torch.int64, 1)
    _check(counter, "counter", torch.int64, 1)
    for t in (temperature, top_k, top_p, seed, counter):
        if t.numel() != R:
            raise KernelError("per-row sampling parameters must have one entry per logits row")
    tokens = torch.empty(R, dtype=torch.int32, device=logits.device)
    logprobs = torch.empty(R, dtype=torch.float32, device=logits.device) if want_logprobs else None
    _ok(lib().acorn_sample(logits.data_ptr(), logits.stride(0), R, V, temperature.data_ptr(), top_k.data_ptr(),
                           top_p.data_ptr(), seed.data_ptr(), counter.data_ptr(), tokens.data_ptr(),
                           _ptr(logprobs), _stream()), "sample")
    return tokens, logprobs


def random_fill(out: torch.Tensor, key: int, first: int, scale: float, offset: float, kind: int) -> torch.Tensor:
    """Fills ``out`` (flat, contiguous) with elements ``first ..`` of the counter-based random tensor
    ``key``: ``offset + lane_sum * scale`` (kind 0 float32, 1 bfloat16) or 15-bit integers (kind 2)."""
    _check(out, "out", {0: torch.float32, 1: torch.bfloat16, 2: torch.int32}[kind])
    _ok(lib().acorn_random_fill(out.data_ptr(), out.numel(), ctypes.c_uint64(key), ctypes.c_uint64(first),
                                float(scale), float(offset), kind, _stream()), "random_fill")
    return out


def uniform(seed: int, counter: int) -> float:
    """The uniform number the sampling kernel draws for (seed, counter), computed on the host."""
    return float(lib_host().acorn_uniform(ctypes.c_uint64(seed & (2 ** 64 - 1)), ctypes.c_uint64(counter & (2 ** 64 - 1))))


def lib_host():
    """The library for its host-only helpers (no device needed)."""
    global _lib
    if _lib is not None:
        return _lib
    h = ctypes.CDLL(str(ensure_built()))
    h.acorn_uniform.argtypes = _Sigs.acorn_uniform
    h.acorn_uniform.restype = c_float
    return h
