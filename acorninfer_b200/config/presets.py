"""Sizes of published Qwen3 dense models as ``config.json`` dictionaries, for runs with random
weights (benchmarks, the random-weights mode): no checkpoint is needed to measure at a model's
layer sizes.  Only the keys the architecture reads are given."""

from __future__ import annotations


def _qwen3(layers: int, hidden: int, heads: int, kv_heads: int, intermediate: int, tied: bool) -> dict:
    return {"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": layers, "hidden_size": hidden,
            "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": 128,
            "intermediate_size": intermediate, "rms_norm_eps": 1e-6, "rope_theta": 1e6, "vocab_size": 151936,
            "tie_word_embeddings": tied, "eos_token_id": 151645}


PRESETS: dict[str, dict] = {
    "qwen3-0.6b": _qwen3(28, 1024, 16, 8, 3072, True),
    "qwen3-1.7b": _qwen3(28, 2048, 16, 8, 6144, True),
    "qwen3-4b": _qwen3(36, 2560, 32, 8, 9728, True),
    "qwen3-8b": _qwen3(36, 4096, 32, 8, 12288, False),
    "qwen3-14b": _qwen3(40, 5120, 40, 8, 17408, False),
    "qwen3-32b": _qwen3(64, 5120, 64, 8, 25600, False),
}


def preset(name: str) -> dict:
    try:
        return dict(PRESETS[name.lower()])
    except KeyError:
        raise ValueError(f"no preset {name!r}; there are {', '.join(sorted(PRESETS))}") from None
