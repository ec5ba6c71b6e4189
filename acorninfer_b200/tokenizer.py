"""Thin wrapper over a ``tokenizer.json`` (the ``tokenizers`` package): text <-> ids.

As the reference's wrapper (``acorninfer/tokenizer.py:11-21``): encoding adds no special
tokens, decoding skips them.  Only the command line needs it, and only for ``--prompt``.
"""

from __future__ import annotations

from pathlib import Path


class Tokenizer:
    def __init__(self, path: str | Path):
        try:
            from tokenizers import Tokenizer as _Tok
        except ImportError as exc:  # pragma: no cover
            raise RuntimeError("the 'tokenizers' package is needed for text prompts; use --prompt-ids") from exc
        if not Path(path).is_file():
            raise FileNotFoundError(f"{path}: no tokenizer.json in the model folder; use --prompt-ids")
        self._tok = _Tok.from_file(str(path))

    def encode(self, text: str) -> list[int]:
        return self._tok.encode(text, add_special_tokens=False).ids

    def decode(self, ids: list[int]) -> str:
        return self._tok.decode(ids, skip_special_tokens=True)
