"""Configuration: keys read from config.json, defaults, refusals, the registry."""

import json

import pytest

from acorninfer_b200.config.engine_config import EngineConfig
from acorninfer_b200.config.model_config import ConfigError, Qwen3Config
from acorninfer_b200.registry import config_from_dict, known_architectures, load_config, spec_for
from tests.tiny import TINIES

RAW_8B = {  # the sizes the reference's tests list for Qwen3-8B (tests/test_config.py:12-22)
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 36, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000, "vocab_size": 151936, "tie_word_embeddings": False,
    "bos_token_id": 151643, "eos_token_id": 151645, "sliding_window": None, "use_sliding_window": False,
    "rope_scaling": None, "torch_dtype": "bfloat16", "max_position_embeddings": 40960,
}


def test_reads_every_size_from_the_keys():
    cfg = config_from_dict(RAW_8B)
    assert isinstance(cfg, Qwen3Config)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (36, 4096, 32, 8)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (128, 12288, 151936)
    assert cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-6
    assert cfg.eos_token_id == (151645,) and cfg.tie_word_embeddings is False


def test_head_dim_defaults_to_width_over_heads_and_eos_may_be_a_list():
    raw = dict(RAW_8B, eos_token_id=[1, 2])
    del raw["head_dim"]
    cfg = config_from_dict(raw)
    assert cfg.head_dim == 128 and cfg.eos_token_id == (1, 2)


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                                 "intermediate_size", "rms_norm_eps", "rope_theta", "vocab_size"])
def test_missing_key_is_named(key):
    raw = dict(RAW_8B)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(raw)


@pytest.mark.parametrize("patch,word", [({"attention_bias": True}, "attention_bias"),
                                        ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
                                        ({"use_sliding_window": True}, "use_sliding_window"),
                                        ({"hidden_act": "gelu"}, "hidden_act"),
                                        ({"num_key_value_heads": 5}, "multiple"),
                                        ({"hidden_size": "big"}, "hidden_size")])
def test_unsupported_or_bad_values_are_refused(patch, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict(dict(RAW_8B, **patch))


def test_unknown_architecture_lists_known_ones():
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        config_from_dict(dict(RAW_8B, architectures=["NopeForCausalLM"]))
    assert "Qwen3ForCausalLM" in known_architectures()


def test_round_trip_through_a_folder(tmp_path):
    for tiny in TINIES.values():
        (tmp_path / "config.json").write_text(json.dumps(tiny["cfg"].to_dict()))
        assert load_config(tmp_path) == tiny["cfg"]


def test_spec_is_data_with_every_size_from_the_config():
    cfg = TINIES["tiny_b"]["cfg"]
    spec = spec_for(cfg)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    m = spec.layers[1].mixer
    assert m.kind == "attention" and m.params["num_heads"] == 8 and m.params["num_kv_heads"] == 1
    assert m.params["head_dim"] == 32 and m.params["qk_norm_eps"] == 1e-5
    assert spec.layers[2].feed_forward.params["intermediate_size"] == 160
    assert spec.positions["rope"].params["theta"] == 1e6
    assert spec.head == "lm_head.weight" and spec_for(TINIES["tiny_a"]["cfg"]).head is None


def test_engine_config_validation():
    assert EngineConfig(dtype="bf16").dtype == "bfloat16"
    for bad in (dict(num_blocks=0), dict(page_size=0), dict(max_running=0), dict(watermark_blocks=-1),
                dict(watermark_blocks=1024), dict(chunked_budget=0), dict(dtype="fp8")):
        with pytest.raises(ValueError):
            EngineConfig(**bad)


def test_presets_of_the_family_are_valid_configurations():
    from acorninfer_b200.config.presets import PRESETS, preset
    from acorninfer_b200.registry import config_from_dict, spec_for
    for name, raw in PRESETS.items():
        cfg = config_from_dict(raw)
        assert cfg.head_dim == 128 and cfg.num_attention_heads % cfg.num_key_value_heads == 0
        spec_for(cfg)                                    # builds the model description
    assert preset("Qwen3-8B")["hidden_size"] == 4096
    import pytest
    with pytest.raises(ValueError, match="qwen3-8b"):
        preset("qwen9")
