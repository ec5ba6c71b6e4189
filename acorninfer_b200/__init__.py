"""acorninfer_b200: a small, whole, single-GPU inference engine for NVIDIA B200 (sm_100a).

Public entry points: :func:`generate` (token ids in, token ids out), :class:`Engine`
(``submit`` / ``step`` / ``has_pending`` / ``drop``), :class:`ModelRunner` (the step
function), :class:`SamplingParams`, ``register_architecture`` and the part registries
under :mod:`acorninfer_b200.parts`.  ``python -m acorninfer_b200 generate ...`` is the
command line, ``bin/trace_run`` the trace replay.
"""

from .config.engine_config import EngineConfig  # noqa: F401
from .config.model_config import ConfigError, ModelConfig, Qwen3Config  # noqa: F401
from .registry import known_architectures, load_config, register_architecture  # noqa: F401
from .sampling.params import SamplingParams  # noqa: F401

__all__ = ["EngineConfig", "ConfigError", "ModelConfig", "Qwen3Config", "SamplingParams", "generate", "Engine",
           "ModelRunner", "register_architecture", "known_architectures", "load_config"]


def __getattr__(name):
    # Engine parts import torch and the kernels; load them on first use.
    if name == "generate":
        from .generation import generate
        return generate
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name == "ModelRunner":
        from .engine.runner import ModelRunner
        return ModelRunner
    raise AttributeError(name)
