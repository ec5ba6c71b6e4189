"""Makes tests/golden/qwen3_reference_logits.json: logits of the reference's own model code
(ErnestW2019/acorninfer, acorninfer/models/qwen3.py, imported on the CPU in float32) on two tiny random
models, so that the plain implementation under tests/plain/ can be checked against the
reference without the reference being present.

Run from the repository root with the reference on the path:

    PYTHONPATH=<path to the acorninfer checkout> python tests/golden/make_golden.py

Weights come from a torch generator seeded per tensor name (values rounded to bfloat16, then
widened), token ids from a seeded generator; nothing is downloaded.  The tied configuration
assigns the token table to ``lm_head`` because the reference does not implement tying itself
(acorninfer/models/qwen3.py:485).
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

CONFIGS = {
    "tiny_a": dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                   intermediate_size=128, rms_norm_eps=1e-6, rope_theta=1e4, vocab_size=256,
                   tie_word_embeddings=True, sigma=0.02, seed=11, tokens=13),
    "tiny_b": dict(num_hidden_layers=3, hidden_size=96, num_attention_heads=8, num_key_value_heads=1, head_dim=32,
                   intermediate_size=160, rms_norm_eps=1e-5, rope_theta=1e6, vocab_size=384,
                   tie_word_embeddings=False, sigma=0.05, seed=12, tokens=23),
}


def golden_weights(c: dict) -> dict[str, torch.Tensor]:
    """Seeded weights by checkpoint name (bfloat16-representable float32 values)."""
    H, nq, nkv, d, I, V = (c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                           c["intermediate_size"], c["vocab_size"])
    shapes = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    if not c["tie_word_embeddings"]:
        shapes["lm_head.weight"] = (V, H)
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shapes.update({
            p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,),
            p + "self_attn.q_proj.weight": (nq * d, H), p + "self_attn.k_proj.weight": (nkv * d, H),
            p + "self_attn.v_proj.weight": (nkv * d, H), p + "self_attn.o_proj.weight": (H, nq * d),
            p + "self_attn.q_norm.weight": (d,), p + "self_attn.k_norm.weight": (d,),
            p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H), p + "mlp.down_proj.weight": (H, I),
        })
    out = {}
    for n, (name, shape) in enumerate(sorted(shapes.items())):
        g = torch.Generator().manual_seed(c["seed"] * 1000 + n)
        if len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        else:
            t = c["sigma"] * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def golden_tokens(c: dict) -> list[int]:
    g = torch.Generator().manual_seed(c["seed"])
    return torch.randint(0, c["vocab_size"], (c["tokens"],), generator=g).tolist()


def main() -> None:
    from acorninfer.config import Qwen3Config
    from acorninfer.models.qwen3 import Qwen3ForCausalLM

    result = {}
    for name, c in CONFIGS.items():
        cfg = Qwen3Config(
            num_hidden_layers=c["num_hidden_layers"], hidden_size=c["hidden_size"],
            num_attention_heads=c["num_attention_heads"], num_key_value_heads=c["num_key_value_heads"],
            head_dim=c["head_dim"], intermediate_size=c["intermediate_size"], rms_norm_eps=c["rms_norm_eps"],
            rope_theta=c["rope_theta"], vocab_size=c["vocab_size"], tie_word_embeddings=c["tie_word_embeddings"],
            bos_token_id=0, eos_token_id=[1])
        model = Qwen3ForCausalLM(cfg).float().eval()
        w = golden_weights(c)
        state = {k[len("model."):] if k.startswith("model.") else k: v for k, v in w.items()}
        if c["tie_word_embeddings"]:
            state["lm_head.weight"] = state["embed_tokens.weight"]
        model.load_state_dict(state, strict=True)
        ids = golden_tokens(c)
        with torch.inference_mode():
            logits = model(torch.tensor([ids]))[0]
        result[name] = {"tokens": ids, "logits_last": logits[-1].tolist(),
                        "logits_row_sums": logits.sum(-1).tolist(),
                        "logits_first4": logits[:, :4].tolist()}
    (HERE / "qwen3_reference_logits.json").write_text(json.dumps(result) + "\n")
    print("wrote", HERE / "qwen3_reference_logits.json")


if __name__ == "__main__":
    main()
