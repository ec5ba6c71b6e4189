"""Grouped-query attention over the paged cache, as a mixer.

Per token: q/k/v projections (no bias), optional per-head RMSNorm of q and k (one weight
of head size shared by all heads), position encoding, K/V written to the request's
pages, causal attention of every query over the keys of its own request (all of them,
or a window), output projection.  Reference: ``Qwen3Attention`` in
``acorninfer/models/qwen3.py:106-152`` and its decode form ``:154-233``; scale
``head_dim ** -0.5`` (``acorninfer/ops/paged_attention.py:147``); query head h uses kv head
``h // (nq / nkv)`` (``acorninfer/models/qwen3.py:98-103``).

All sizes are parameters.  The q, k, v matrices are concatenated when bound so that one
matrix product yields ``[tokens, (nq + 2 nkv) * d]``.  A run that reads another run's
cache (``cache.write`` false) computes queries only.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels import attention as attn_kernels
from .base import MIXERS, BuildContext, CacheNeeds, KVNeeds, Mixer, TensorSpec


@MIXERS.register("attention")
class Attention(Mixer):
    graph_safe = True
    supports_epilogue = True
    adds_residual = True

    def __init__(self, ctx: BuildContext, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: str | None, scale: float, qk_norm_eps: float | None = None,
                 window: int | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be a multiple of num_kv_heads ({num_kv_heads})")
        if window is not None and window < 1:
            raise ValueError(f"window must be >= 1 or None, got {window}")
        self.ctx = ctx
        self.hidden_size = hidden_size
        self.nq, self.nkv, self.d = num_heads, num_kv_heads, head_dim
        self.scale = float(scale)
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.position = ctx.positions[position] if position is not None else None
        if self.position is not None and self.position.head_dim != head_dim:
            raise ValueError("position encoding was built for another head size")
        self.w_qkv = self.w_o = self.q_norm32 = self.k_norm32 = None

    def tensor_specs(self):
        specs = {
            "q_proj.weight": TensorSpec((self.nq * self.d, self.hidden_size)),
            "k_proj.weight": TensorSpec((self.nkv * self.d, self.hidden_size)),
            "v_proj.weight": TensorSpec((self.nkv * self.d, self.hidden_size)),
            "o_proj.weight": TensorSpec((self.hidden_size, self.nq * self.d)),
        }
        if self.qk_norm_eps is not None:
            specs["q_norm.weight"] = TensorSpec((self.d,), "norm")
            specs["k_norm.weight"] = TensorSpec((self.d,), "norm")
        return specs

    def bind(self, tensors):
        parts = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        dtype = parts[0].dtype if all(p.dtype == parts[0].dtype for p in parts) else torch.float32
        self.w_qkv = torch.cat([p.to(dtype) for p in parts], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()
        if self.qk_norm_eps is not None:
            self.q_norm32 = tensors["q_norm.weight"].to(torch.float32).contiguous()
            self.k_norm32 = tensors["k_norm.weight"].to(torch.float32).contiguous()

    def cache_needs(self):
        return CacheNeeds(kv=KVNeeds(self.nkv, self.d, self.window))

    def step_arrays(self):
        return attn_kernels.STEP_ARRAYS

    def fusable(self, num_rows):
        return (self._rows_fuse(num_rows) and self.w_qkv.dtype == torch.bfloat16
                and self.w_o.dtype == torch.bfloat16 and self.hidden_size % 8 == 0 and (self.nq * self.d) % 8 == 0)

    def _rows_fuse(self, num_rows):
        widths = ((self.nq + 2 * self.nkv) * self.d, self.hidden_size)         # of the q/k/v product and of the o product
        return ops.fused_rows_ok(num_rows, self.ctx.dtype, widths, ops.device_sms(self.ctx.device))

    def forward(self, x, inputs, cache, epilogue=None, residual32=None):
        g = inputs.groups[cache.group]
        pos = self.position
        rows = x.x.shape[0] if isinstance(x, ops.NormedRows) else x.shape[0]
        if (pos is not None and self.w_qkv.dtype == torch.bfloat16 and ops.gemm_tc_supported(
                x.x if isinstance(x, ops.NormedRows) else x, self.w_qkv)
                and self._rows_fuse(rows)
                and ops.rope_kv_fusable(rows, self.ctx.dtype, self.d, pos.rotary_dim, pos.interleaved)):
            # few rows or very many, head size 128: norm, rotation and the cache write are the epilogue of the product
            qkv = ops.gemm_tc_qkv_rope(x, self.w_qkv, ops.RopeKvEpilogue(
                inputs.positions, inputs.token_row, g.block_table, g.page_base,
                cache.k_pages if cache.write else None, cache.v_pages if cache.write else None,
                self.q_norm32, self.k_norm32, pos.inv_freq, self.nq, self.nkv,
                self.qk_norm_eps if self.qk_norm_eps is not None else 0.0,
                cos_sin=pos.table(inputs) if rows > ops.GEMM_TC_MAX_ROWS and hasattr(pos, "table") else None))
        else:
            qkv = ops.linear(x, self.w_qkv, out_dtype=self.ctx.dtype)
            ops.qk_rope_kv(qkv, self.q_norm32, self.k_norm32,
                           pos.inv_freq if pos is not None else _no_freq(self.ctx.device),
                           inputs.positions, inputs.token_row, g.block_table, g.page_base,
                           cache.k_pages, cache.v_pages, self.nq, self.nkv, self.d,
                           pos.rotary_dim if pos is not None else 0, pos.interleaved if pos is not None else False,
                           self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, write_kv=cache.write)
        out = attn_kernels.paged_attention(qkv, inputs, g, cache, self.nq, self.nkv, self.d, self.scale, self.window)
        return ops.linear(out, self.w_o, out_dtype=self.ctx.dtype, epilogue=epilogue,
                          residual32=residual32 if epilogue is None else None)


_NO_FREQ: dict = {}


def _no_freq(device):
    if device not in _NO_FREQ:
        _NO_FREQ[device] = torch.zeros(0, dtype=torch.float32, device=device)
    return _NO_FREQ[device]
