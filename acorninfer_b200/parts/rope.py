"""Rotary position encoding: the constants, and a stand-alone application.

``inv_freq[j] = 1 / theta^(2j / rotary_dim)`` in float32, angle = position * inv_freq[j];
pairing ``half`` rotates (x[j], x[j + rotary_dim/2]), ``interleaved`` rotates (x[2j], x[2j+1]);
dimensions beyond ``rotary_dim`` pass through.  Reference: ``RotaryEmbedding``, ``_rotate_half``,
``_apply_rope`` in ``acorninfer/models/qwen3.py:63-95`` (half pairing, full head rotated).
The mixers' kernels take these constants; nothing here knows about attention.
"""

from __future__ import annotations

import torch

from .base import POSITION_ENCODINGS, BuildContext, PositionEncoding


@POSITION_ENCODINGS.register("rope")
class Rope(PositionEncoding):
    def __init__(self, ctx: BuildContext, head_dim: int, theta: float, rotary_dim: int | None = None,
                 pairing: str = "half"):
        rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rope pairing must be 'half' or 'interleaved', got {pairing!r}")
        if rotary_dim % 2 or not (0 < rotary_dim <= head_dim):
            raise ValueError(f"rotary_dim must be even and in 2..head_dim, got {rotary_dim}")
        self.ctx = ctx
        self.head_dim = head_dim
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.interleaved = pairing == "interleaved"
        self._inv_freq_cpu = 1.0 / (self.theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
        self._inv_freq_dev: torch.Tensor | None = None

    @property
    def inv_freq(self) -> torch.Tensor:
        if self._inv_freq_dev is None:
            self._inv_freq_dev = self._inv_freq_cpu.to(self.ctx.device).contiguous()
        return self._inv_freq_dev

    def table(self, inputs) -> torch.Tensor:
        """cos and sin of every token's angles, [tokens, rotary_dim] float32 (cos, then sin): computed by
        the first layer of a step that asks and kept with the step's inputs for the others."""
        from ..kernels import ops
        key = ("rope.table", self.theta, self.rotary_dim)
        if key not in inputs.extra:
            inputs.extra[key] = ops.rope_table(inputs.positions, self.inv_freq)
        return inputs.extra[key]


@POSITION_ENCODINGS.register("none")
class NoPosition(PositionEncoding):
    """No position encoding: a rope of zero rotated dimensions."""

    def __init__(self, ctx: BuildContext, head_dim: int):
        self.ctx = ctx
        self.head_dim = head_dim
        self.rotary_dim = 0
        self.interleaved = False
        self._inv = None

    @property
    def inv_freq(self) -> torch.Tensor:
        if self._inv is None:
            self._inv = torch.zeros(0, dtype=torch.float32, device=self.ctx.device)
        return self._inv
