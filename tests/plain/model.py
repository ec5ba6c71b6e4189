"""Plain, slow implementation of the Qwen3 dense decoder for whole sequences.

No cache, no batching, one function per part, written from the reference's formulas
(each function cites the reference file and lines).  It shares no code with the
engine under ``acorninfer_b200/``: it takes a dict of sizes and a dict of tensors by
checkpoint name, and computes in the dtype it is given (float64 by default, so that it
can arbitrate between float32 results).  ``tests/golden/`` holds outputs of the
reference's own model (imported on the CPU) that this file is checked against once.
"""

from __future__ import annotations


import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """acorninfer/models/qwen3.py:56-60: x * rsqrt(mean(x^2, last) + eps) * w."""
    var = x.pow(2).mean(-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def rope_cos_sin(positions: torch.Tensor, rotary_dim: int, theta: float, dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """acorninfer/models/qwen3.py:71-84: inv_freq[j] = 1 / theta^(2j/d) (float32, as the
    reference's buffer), freqs = pos (x) inv_freq, cos/sin of cat(freqs, freqs)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
    freqs = torch.outer(positions.to(torch.float32), inv_freq).to(torch.float64)
    # The angle is a float32 product in the reference; cos/sin are then evaluated exactly here.
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """acorninfer/models/qwen3.py:63-65: cat(-x[d/2:], x[:d/2])."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """acorninfer/models/qwen3.py:87-95: x * cos + rotate_half(x) * sin.  x: [heads, S, d]."""
    return x * cos[None] + rotate_half(x) * sin[None]


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: int | None = None) -> torch.Tensor:
    """acorninfer/models/qwen3.py:98-103,135-149 and acorninfer/ops/paged_attention.py:54,147:
    query head h reads kv head h // rep; scores (q . k) * scale; query at position p sees keys
    0..p (with a window w: p-w+1..p); softmax over keys; weighted sum of values.
    q: [nq, S, d]; k, v: [nkv, S, d] -> [nq, S, d]."""
    nq, S, d = q.shape
    rep = nq // k.shape[0]
    k = k.repeat_interleave(rep, dim=0)
    v = v.repeat_interleave(rep, dim=0)
    scores = torch.einsum("hqd,hkd->hqk", q, k) * scale
    qi = torch.arange(S)[:, None]
    ki = torch.arange(S)[None, :]
    allowed = ki <= qi
    if window is not None:
        allowed &= ki > qi - window
    scores = scores.masked_fill(~allowed[None], float("-inf"))
    return torch.einsum("hqk,hkd->hqd", torch.softmax(scores, dim=-1), v)


def attention_keys_values(x, w, prefix, sizes, positions):
    """k, v of a layer (normed, rotated keys) from its input: acorninfer/models/qwen3.py:123-129."""
    nkv, d = sizes["num_key_value_heads"], sizes["head_dim"]
    S = x.shape[0]
    k = (x @ w[prefix + "k_proj.weight"].T).view(S, nkv, d).transpose(0, 1)
    v = (x @ w[prefix + "v_proj.weight"].T).view(S, nkv, d).transpose(0, 1)
    k = rms_norm(k, w[prefix + "k_norm.weight"], sizes["rms_norm_eps"])
    cos, sin = rope_cos_sin(positions, d, sizes["rope_theta"], x.dtype)
    return apply_rope(k, cos, sin), v


def attention_block(x, w, prefix, sizes, positions, window=None, shared_kv=None):
    """acorninfer/models/qwen3.py:119-152: projections (no bias), per-head q/k RMSNorm over
    head_dim with one weight for all heads, rope, causal attention, output projection.
    ``shared_kv``: keys/values of another layer to read instead of this layer's own."""
    nq, d = sizes["num_attention_heads"], sizes["head_dim"]
    S = x.shape[0]
    q = (x @ w[prefix + "q_proj.weight"].T).view(S, nq, d).transpose(0, 1)
    q = rms_norm(q, w[prefix + "q_norm.weight"], sizes["rms_norm_eps"])
    cos, sin = rope_cos_sin(positions, d, sizes["rope_theta"], x.dtype)
    q = apply_rope(q, cos, sin)
    k, v = shared_kv if shared_kv is not None else attention_keys_values(x, w, prefix, sizes, positions)
    out = causal_attention(q, k, v, d ** -0.5, window)
    return out.transpose(0, 1).reshape(S, nq * d) @ w[prefix + "o_proj.weight"].T, (k, v)


def swiglu_mlp(x, w, prefix):
    """acorninfer/models/qwen3.py:392-396: down(silu(gate(x)) * up(x)), silu(z) = z * sigmoid(z)."""
    g = x @ w[prefix + "gate_proj.weight"].T
    u = x @ w[prefix + "up_proj.weight"].T
    return (g * torch.sigmoid(g) * u) @ w[prefix + "down_proj.weight"].T


def decoder_layer(x, w, i, sizes, positions, window=None, shared_kv=None):
    """acorninfer/models/qwen3.py:407-410: x += attn(norm(x)); x += mlp(norm(x))."""
    p = f"model.layers.{i}."
    eps = sizes["rms_norm_eps"]
    a, kv = attention_block(rms_norm(x, w[p + "input_layernorm.weight"], eps), w, p + "self_attn.", sizes,
                            positions, window, shared_kv)
    x = x + a
    x = x + swiglu_mlp(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    return x, kv


def final_hidden(sizes: dict, weights: dict, token_ids, dtype=torch.float64, schedule=None, windows=None,
                 embedded: torch.Tensor | None = None) -> torch.Tensor:
    """acorninfer/models/qwen3.py:491-515: embedding, the layers, final norm.  Returns the normed
    hidden rows [S, hidden] that the output matrix multiplies.

    ``schedule``: list of (layer, reads_cache_of_entry | None), default each layer once;
    ``windows``: per layer, a window or None; ``embedded``: the token table's rows of
    ``token_ids`` [S, hidden], for a caller that does not hold the whole table."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.numel())
    x = embedded.to(dtype) if embedded is not None else w["model.embed_tokens.weight"][ids]
    n_layers = sizes["num_hidden_layers"]
    schedule = schedule or [(i, None) for i in range(n_layers)]
    kvs = []
    for layer, reads in schedule:
        window = windows[layer] if windows else None
        x, kv = decoder_layer(x, w, layer, sizes, positions, window, kvs[reads] if reads is not None else None)
        kvs.append(kv)
    return rms_norm(x, w["model.norm.weight"], sizes["rms_norm_eps"])


def forward(sizes: dict, weights: dict, token_ids, dtype=torch.float64, schedule=None, windows=None) -> torch.Tensor:
    """acorninfer/models/qwen3.py:516-518: the output matrix (the token table when tied) on the
    final hidden rows.  Returns logits [S, vocab] for every position."""
    x = final_hidden(sizes, weights, token_ids, dtype, schedule, windows)
    head = weights["lm_head.weight"] if "lm_head.weight" in weights and not sizes.get("tie_word_embeddings") \
        else weights["model.embed_tokens.weight"]
    return x @ head.to(dtype).T


def greedy_generate(sizes, weights, prompt, max_new_tokens, eos_ids=(), dtype=torch.float64) -> list[int]:
    """acorninfer/generate.py:20-51: argmax of the last position, append, stop after an eos id."""
    out = list(prompt)
    for _ in range(max_new_tokens):
        nxt = int(forward(sizes, weights, out, dtype)[-1].argmax())
        out.append(nxt)
        if nxt in eos_ids:
            break
    return out


# ------------------------------------------------------------------ sampling


def process_logits(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0) -> torch.Tensor:
    """acorninfer/sampler.py:38-56: / temperature; top-k keeps logits >= the k-th largest;
    top-p removes, ascending, tokens whose cumulative probability is <= 1 - top_p, never the largest."""
    x = logits.to(torch.float64) / temperature
    if top_k > 0:
        kth = torch.topk(x, min(top_k, x.numel())).values[-1]
        x = x.masked_fill(x < kth, float("-inf"))
    if top_p < 1.0:
        sorted_x, idx = torch.sort(x, descending=False)
        cum = sorted_x.softmax(-1).cumsum(-1)
        remove = cum <= (1.0 - top_p)
        remove[-1] = False
        x = x.masked_fill(torch.zeros_like(remove).scatter(0, idx, remove), float("-inf"))
    return x


def sample_with_uniform(processed: torch.Tensor, u: float) -> tuple[int, float, float]:
    """Inverse CDF in token order: the first token whose running probability exceeds u.
    Returns (token, its log-probability, distance of u to the nearest CDF step)."""
    p = processed.softmax(-1)
    cdf = p.cumsum(-1)
    tok = int(torch.searchsorted(cdf, torch.tensor(u, dtype=cdf.dtype), right=True).clamp(max=p.numel() - 1))
    margin = float((cdf - u).abs().min())
    return tok, float(torch.log(p[tok])), margin
