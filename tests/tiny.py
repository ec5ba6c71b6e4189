"""The tiny configurations the tests use, and helpers to make their model folders.

Tiny A and Tiny B differ in every size and option: layers, width, head counts and groups,
head size, feed-forward width, vocabulary, rope theta, eps, tied or separate output matrix,
weight scale and page size.  Tiny C has sizes that are no power of two anywhere and 5 query
heads per kv head.
"""

from __future__ import annotations

from pathlib import Path

import torch

from acorninfer_b200.config.model_config import Qwen3Config
from acorninfer_b200.weights.random_init import write_random_model
from acorninfer_b200.weights.safetensors_io import SafetensorsFile

TINY_A = dict(cfg=Qwen3Config(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                              head_dim=16, intermediate_size=128, rms_norm_eps=1e-6, rope_theta=1e4, vocab_size=256,
                              tie_word_embeddings=True, bos_token_id=0, eos_token_id=(1,)),
              sigma=0.02, sigma_norm=0.1, seed=101, page_size=4)
TINY_B = dict(cfg=Qwen3Config(num_hidden_layers=3, hidden_size=96, num_attention_heads=8, num_key_value_heads=1,
                              head_dim=32, intermediate_size=160, rms_norm_eps=1e-5, rope_theta=1e6, vocab_size=384,
                              tie_word_embeddings=False, bos_token_id=0, eos_token_id=(2, 3)),
              sigma=0.05, sigma_norm=0.1, seed=202, page_size=8)
TINY_C = dict(cfg=Qwen3Config(num_hidden_layers=2, hidden_size=120, num_attention_heads=10, num_key_value_heads=2,
                              head_dim=48, intermediate_size=200, rms_norm_eps=3e-6, rope_theta=5e5, vocab_size=331,
                              tie_word_embeddings=False, bos_token_id=None, eos_token_id=()),
              sigma=0.04, sigma_norm=0.2, seed=303, page_size=16)
# head size 128: the size the tcgen05 attention kernel takes, so that replay runs through it
TINY_D = dict(cfg=Qwen3Config(num_hidden_layers=2, hidden_size=192, num_attention_heads=4, num_key_value_heads=2,
                              head_dim=128, intermediate_size=320, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=500,
                              tie_word_embeddings=False, bos_token_id=None, eos_token_id=()),
              sigma=0.04, sigma_norm=0.1, seed=404, page_size=16)
TINIES = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C, "tiny_d": TINY_D}


def make_model_dir(tmp: Path, tiny: dict, dtype=torch.bfloat16) -> Path:
    return write_random_model(tmp, tiny["cfg"], tiny["seed"], tiny["sigma"], tiny["sigma_norm"], dtype)


def read_weights(model_dir: Path) -> dict[str, torch.Tensor]:
    f = SafetensorsFile(Path(model_dir) / "model.safetensors")
    return {n: f.tensor(n).clone() for n in f.entries}


def sizes_of(cfg: Qwen3Config) -> dict:
    return cfg.to_dict()


def random_tokens(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
