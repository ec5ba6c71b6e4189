"""Engine options, validated when constructed.

Names and meanings follow the reference where it has them
(``acorninfer/config.py:69-122``, ``acorninfer/engine/engine.py:31-45``):
``num_blocks`` pages in the pool of every cache group, ``page_size`` tokens a page,
``max_running`` requests in a step at most, ``watermark_blocks`` pages that admission
leaves free, ``chunked_budget`` the most tokens one step may carry (``None``: whole
prompts).  The reference's back-end switches have no counterpart: there is one back end.
"""

from __future__ import annotations

from dataclasses import dataclass

DTYPE_NAMES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


@dataclass(frozen=True)
class EngineConfig:
    model_dir: str | None = None
    device: str = "cuda:0"
    dtype: str = "bfloat16"
    num_blocks: int = 1024
    page_size: int = 16
    max_running: int = 8
    watermark_blocks: int = 8
    chunked_budget: int | None = None
    max_step_tokens: int = 8192      # capacity of the step workspace (tokens in one step)
    decode_graph: bool = True        # replay captured CUDA graphs for all-decode steps

    def __post_init__(self) -> None:
        if self.dtype not in DTYPE_NAMES:
            raise ValueError(f"dtype must be one of {sorted(DTYPE_NAMES)}, got {self.dtype!r}")
        object.__setattr__(self, "dtype", DTYPE_NAMES[self.dtype])
        if self.num_blocks < 1:
            raise ValueError(f"num_blocks must be >= 1, got {self.num_blocks}")
        if self.page_size < 1 or self.page_size > 256 or self.page_size & (self.page_size - 1):
            raise ValueError(f"page_size must be a power of two in 1..256, got {self.page_size}")
        if self.max_running < 1:
            raise ValueError(f"max_running must be >= 1, got {self.max_running}")
        if self.watermark_blocks < 0:
            raise ValueError(f"watermark_blocks must be >= 0, got {self.watermark_blocks}")
        if self.watermark_blocks >= self.num_blocks:
            raise ValueError(
                f"watermark_blocks ({self.watermark_blocks}) must be < num_blocks ({self.num_blocks})")
        if self.chunked_budget is not None and self.chunked_budget < 1:
            raise ValueError(f"chunked_budget must be >= 1, got {self.chunked_budget}")
        if self.max_step_tokens < 1:
            raise ValueError(f"max_step_tokens must be >= 1, got {self.max_step_tokens}")
