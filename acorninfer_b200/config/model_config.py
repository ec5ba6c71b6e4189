"""Typed model configurations, read from an architecture's own ``config.json`` keys.

Every size and constant of a model comes from here; nothing downstream carries a
default for a size.  A configuration class knows two things: how to read itself
from the raw ``config.json`` dictionary (``from_dict``) and how to write itself
back (``to_dict``), so that the random-weights mode can produce a model folder.

Reference behaviour: ``acorninfer/config.py:16-48`` reads twelve required keys with
``raw[...]`` and ignores every other key.  Here a missing key is an error that names
the key, and keys that would change the computation but are not implemented
(``attention_bias``, ``rope_scaling``, an active sliding window) are refused instead
of being ignored.
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field, fields
from pathlib import Path
from typing import ClassVar


class ConfigError(ValueError):
    """A ``config.json`` that cannot be turned into a model: names the key at fault."""


_MISSING = object()


def _take(raw: dict, key: str, kind, default=_MISSING):
    """Read ``raw[key]`` as ``kind``; a missing key without default is a ConfigError."""
    if key not in raw or raw[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    value = raw[key]
    if kind is bool:
        if not isinstance(value, bool):
            raise ConfigError(f"config.json: key '{key}' must be true/false, got {value!r}")
        return value
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise ConfigError(f"config.json: key '{key}' must be an integer, got {value!r}")
        return value
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config.json: key '{key}' must be a number, got {value!r}")
        return float(value)
    return value


@dataclass(frozen=True)
class ModelConfig:
    """Base of all architecture configurations.

    ``architecture`` is the name under which the model is registered
    (``config.json``'s ``architectures[0]``).
    """

    architecture: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":  # pragma: no cover - abstract
        raise NotImplementedError

    def to_dict(self) -> dict:
        out = {"architectures": [self.architecture]}
        out.update(asdict(self))
        return out


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    """Qwen3 dense decoder: GQA attention with per-head q/k RMSNorm, half-rotate
    RoPE, SwiGLU feed-forward, pre-norm residual blocks, optionally tied output head.

    Keys as in ``acorninfer/config.py:33-48``.  ``head_dim`` may be absent (then
    ``hidden_size / num_attention_heads``), ``tie_word_embeddings`` defaults to
    false, ``bos_token_id``/``eos_token_id`` are optional and only stored.
    """

    architecture: ClassVar[str] = "Qwen3ForCausalLM"

    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    vocab_size: int
    tie_word_embeddings: bool = False
    bos_token_id: int | None = None
    eos_token_id: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        for f in ("num_hidden_layers", "hidden_size", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size"):
            if getattr(self, f) < 1:
                raise ConfigError(f"config.json: '{f}' must be >= 1, got {getattr(self, f)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                "config.json: 'num_attention_heads' "
                f"({self.num_attention_heads}) must be a multiple of 'num_key_value_heads' "
                f"({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: 'head_dim' must be even for rotary pairs, got {self.head_dim}")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"config.json: 'rms_norm_eps' must be > 0, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise ConfigError(f"config.json: 'rope_theta' must be > 0, got {self.rope_theta}")

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        n_heads = _take(raw, "num_attention_heads", int)
        hidden = _take(raw, "hidden_size", int)
        if "head_dim" in raw and raw["head_dim"] is not None:
            head_dim = _take(raw, "head_dim", int)
        else:
            if hidden % n_heads != 0:
                raise ConfigError(
                    "config.json: 'head_dim' is absent and 'hidden_size' is not a multiple of "
                    "'num_attention_heads'")
            head_dim = hidden // n_heads
        # Keys that change the computation and are not implemented are refused.
        if _take(raw, "attention_bias", bool, False):
            raise ConfigError("config.json: 'attention_bias' = true is not supported by Qwen3ForCausalLM here")
        if raw.get("rope_scaling") is not None:
            raise ConfigError("config.json: 'rope_scaling' is not supported (only plain RoPE)")
        if _take(raw, "use_sliding_window", bool, False):
            raise ConfigError("config.json: 'use_sliding_window' = true is not supported for Qwen3ForCausalLM")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: 'hidden_act' must be 'silu', got {act!r}")
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        bos = raw.get("bos_token_id")
        return cls(
            num_hidden_layers=_take(raw, "num_hidden_layers", int),
            hidden_size=hidden,
            num_attention_heads=n_heads,
            num_key_value_heads=_take(raw, "num_key_value_heads", int),
            head_dim=head_dim,
            intermediate_size=_take(raw, "intermediate_size", int),
            rms_norm_eps=_take(raw, "rms_norm_eps", float),
            rope_theta=_take(raw, "rope_theta", float),
            vocab_size=_take(raw, "vocab_size", int),
            tie_word_embeddings=_take(raw, "tie_word_embeddings", bool, False),
            bos_token_id=None if bos is None else int(bos),
            eos_token_id=eos_ids,
        )

    def to_dict(self) -> dict:
        out = super().to_dict()
        out["eos_token_id"] = list(self.eos_token_id)
        out["hidden_act"] = "silu"
        out["attention_bias"] = False
        out["model_type"] = "qwen3"
        return out


def read_config_json(model_dir: str | Path) -> dict:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return raw


def architecture_name(raw: dict) -> str:
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return archs[0]


def config_field_names(cls) -> list[str]:
    return [f.name for f in fields(cls)]


def dump_config(cfg: ModelConfig, model_dir: str | Path) -> None:
    Path(model_dir).mkdir(parents=True, exist_ok=True)
    (Path(model_dir) / "config.json").write_text(json.dumps(cfg.to_dict(), indent=1) + "\n")
