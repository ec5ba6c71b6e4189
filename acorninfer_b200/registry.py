"""One registry from an architecture's name to its configuration class and its model.

``config.json``'s ``architectures[0]`` picks the entry.  An entry is a
configuration class (``from_dict``/``to_dict``) and a function that turns such a
configuration into a :class:`~acorninfer_b200.parts.base.ModelSpec`, the data
that the generic decoder is built from.  The reference has no registry
(``acorninfer/models/__init__.py:1-3`` re-exports its one model); this one exists so
that another architecture is added by one ``register_architecture`` call.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from .config.model_config import ConfigError, ModelConfig, architecture_name, read_config_json
from .parts.base import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type
    build_spec: Callable[[ModelConfig], ModelSpec]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, build_spec: Callable[[ModelConfig], ModelSpec]) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_cls, build_spec)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"config.json: architecture '{name}' is not registered; known: "
            f"{', '.join(known_architectures()) or '(none)'}") from None


def config_from_dict(raw: dict) -> ModelConfig:
    return get_architecture(architecture_name(raw)).config_cls.from_dict(raw)


def load_config(model_dir: str | Path) -> ModelConfig:
    return config_from_dict(read_config_json(model_dir))


def spec_for(cfg: ModelConfig) -> ModelSpec:
    return get_architecture(type(cfg).architecture).build_spec(cfg)


_builtin_done = False


def _ensure_builtin() -> None:
    global _builtin_done
    if not _builtin_done:
        _builtin_done = True
        from .models import qwen3  # noqa: F401  (registers itself)
