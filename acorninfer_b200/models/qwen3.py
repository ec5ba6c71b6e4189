"""Qwen3 dense as data: which parts each layer has, with which sizes, in which order.

The computation this describes is the reference's ``acorninfer/models/qwen3.py``:
embedding (``:482,512``), per layer pre-norm attention with per-head q/k RMSNorm
and half-rotate RoPE (``:106-152``), SwiGLU feed-forward (``:385-396``), residual
sums (``:407-410``), final norm and output matrix (``:515-518``).  Tensor names are the
checkpoint's own (``:750-752`` strips ``model.``; ``lm_head.weight`` has no prefix).

The reference reads ``tie_word_embeddings`` and never uses it; here a tied model
uses the token table as output matrix, and ``lm_head.weight`` may be absent.
"""

from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture


def qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    rope = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                             "rotary_dim": cfg.head_dim, "pairing": "half"})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        norm = {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps}
        layers.append(LayerSpec(
            block=PartSpec("prenorm", {}, p),
            mixer=PartSpec("attention", {
                "hidden_size": cfg.hidden_size,
                "num_heads": cfg.num_attention_heads,
                "num_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim,
                "qk_norm_eps": cfg.rms_norm_eps,
                "position": "rope",
                "scale": cfg.head_dim ** -0.5,
                "window": None,
            }, p + "self_attn."),
            feed_forward=PartSpec("swiglu", {
                "hidden_size": cfg.hidden_size,
                "intermediate_size": cfg.intermediate_size,
            }, p + "mlp."),
            norms={
                "mixer": PartSpec("rmsnorm", norm, p + "input_layernorm."),
                "feed_forward": PartSpec("rmsnorm", norm, p + "post_attention_layernorm."),
            },
        ))
    return ModelSpec(
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        embedding="model.embed_tokens.weight",
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps}, "model.norm."),
        head=None if cfg.tie_word_embeddings else "lm_head.weight",
        positions={"rope": rope},
    )


register_architecture(Qwen3Config.architecture, Qwen3Config, qwen3_spec)
