"""Two more toy parts, defined here and registered without touching the framework: a routed
feed-forward (router logits in float32, top-1 of three experts, each a small SwiGLU) and an
architecture whose attention uses another position encoding (interleaved pairs, only part of
the head rotated).  Built from a model folder, stepped through runner and replay in every cut,
compared with a plain computation written here.  They are test parts, not anyone's model."""

from dataclasses import dataclass
from typing import ClassVar

import numpy as np
import pytest
import torch

from acorninfer_b200.config.model_config import ModelConfig
from acorninfer_b200.parts.base import FEED_FORWARDS, FeedForward, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
from acorninfer_b200.registry import register_architecture, unregister_architecture
from tests import traces
from tests.plain import model as plain
from tests.tiny import random_tokens, read_weights

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class RoutedConfig(ModelConfig):
    architecture: ClassVar[str] = "ToyRoutedForCausalLM"
    hidden_size: int = 48
    vocab_size: int = 113
    num_heads: int = 3
    num_kv_heads: int = 1
    head_dim: int = 32
    rotary_dim: int = 16
    expert_size: int = 40
    num_experts: int = 3
    eps: float = 2e-6
    theta: float = 7e3

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: raw[k] for k in cls.__dataclass_fields__ if k in raw})


class Top1Experts(FeedForward):
    """y[t] = p * expert_e(x[t]), e = argmax of the router's float32 logits, p its softmax weight."""

    def __init__(self, ctx, width, expert_size, num_experts):
        self.ctx, self.width, self.size, self.n = ctx, width, expert_size, num_experts
        self.router = None
        self.experts = []

    def tensor_specs(self):
        specs = {"router.weight": TensorSpec((self.n, self.width))}
        for e in range(self.n):
            specs[f"experts.{e}.gate_up.weight"] = TensorSpec((2 * self.size, self.width))
            specs[f"experts.{e}.down.weight"] = TensorSpec((self.width, self.size))
        return specs

    def bind(self, tensors):
        self.router = tensors["router.weight"].float().contiguous()
        self.experts = [(tensors[f"experts.{e}.gate_up.weight"].contiguous(), tensors[f"experts.{e}.down.weight"].contiguous())
                        for e in range(self.n)]

    def forward(self, x, inputs):
        from acorninfer_b200.kernels import ops
        logits = ops.gemm_f32(ops.cast(x, torch.float32), self.router)          # router in float32
        prob = torch.softmax(logits, dim=-1)
        choice = logits.argmax(dim=-1)
        out = torch.zeros_like(x)
        for e, (w_gu, w_down) in enumerate(self.experts):
            idx = (choice == e).nonzero(as_tuple=True)[0]
            if idx.numel() == 0:
                continue
            h = ops.swiglu(ops.linear(x.index_select(0, idx).contiguous(), w_gu, out_dtype=self.ctx.dtype))
            y = ops.linear(h, w_down, out_dtype=self.ctx.dtype)
            out.index_copy_(0, idx, (y.float() * prob[idx, e].unsqueeze(1)).to(x.dtype))
        return out


def routed_spec(cfg: RoutedConfig) -> ModelSpec:
    norm = {"width": cfg.hidden_size, "eps": cfg.eps}
    layers = []
    for i in range(2):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            PartSpec("prenorm", {}, p),
            PartSpec("attention", {"hidden_size": cfg.hidden_size, "num_heads": cfg.num_heads,
                                   "num_kv_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim, "qk_norm_eps": None,
                                   "position": "rope_partial", "scale": cfg.head_dim ** -0.5, "window": None},
                     p + "self_attn."),
            PartSpec("toy_top1_experts", {"width": cfg.hidden_size, "expert_size": cfg.expert_size,
                                          "num_experts": cfg.num_experts}, p + "moe."),
            {"mixer": PartSpec("rmsnorm", norm, p + "ln1."), "feed_forward": PartSpec("rmsnorm", norm, p + "ln2.")}))
    return ModelSpec(cfg.vocab_size, cfg.hidden_size, "model.embed_tokens.weight", tuple(layers),
                     (ScheduleEntry(0), ScheduleEntry(1)), PartSpec("rmsnorm", norm, "model.norm."), "lm_head.weight",
                     {"rope_partial": PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.theta,
                                                        "rotary_dim": cfg.rotary_dim, "pairing": "interleaved"})})


def rope_interleaved(x, positions, rot, theta):
    """Pairs (x[2j], x[2j+1]) of the first ``rot`` dims rotated by pos * theta^(-2j/rot); the rest kept."""
    inv = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    ang = (positions.to(torch.float32)[:, None] * inv[None]).double()
    c, s = ang.cos()[None], ang.sin()[None]                  # x: [heads, S, d]
    out = x.clone()
    a, b = x[..., 0:rot:2], x[..., 1:rot:2]
    out[..., 0:rot:2], out[..., 1:rot:2] = a * c - b * s, b * c + a * s
    return out


def routed_plain(cfg: RoutedConfig, weights, ids):
    w = {k: v.double() for k, v in weights.items()}
    ids = torch.as_tensor(ids)
    S = len(ids)
    pos = torch.arange(S)
    x = w["model.embed_tokens.weight"][ids]
    for i in range(2):
        p = f"model.layers.{i}."
        h = plain.rms_norm(x, w[p + "ln1.weight"], cfg.eps)
        q = (h @ w[p + "self_attn.q_proj.weight"].T).view(S, cfg.num_heads, cfg.head_dim).transpose(0, 1)
        k = (h @ w[p + "self_attn.k_proj.weight"].T).view(S, cfg.num_kv_heads, cfg.head_dim).transpose(0, 1)
        v = (h @ w[p + "self_attn.v_proj.weight"].T).view(S, cfg.num_kv_heads, cfg.head_dim).transpose(0, 1)
        q, k = rope_interleaved(q, pos, cfg.rotary_dim, cfg.theta), rope_interleaved(k, pos, cfg.rotary_dim, cfg.theta)
        a = plain.causal_attention(q, k, v, cfg.head_dim ** -0.5)
        x = x + a.transpose(0, 1).reshape(S, -1) @ w[p + "self_attn.o_proj.weight"].T
        h = plain.rms_norm(x, w[p + "ln2.weight"], cfg.eps)
        logits = h @ w[p + "moe.router.weight"].T
        prob, choice = torch.softmax(logits, -1), logits.argmax(-1)
        y = torch.zeros_like(h)
        for t in range(S):
            e = int(choice[t])
            gu = h[t] @ w[p + f"moe.experts.{e}.gate_up.weight"].T
            g, u = gu[:cfg.expert_size], gu[cfg.expert_size:]
            y[t] = prob[t, e] * ((g * torch.sigmoid(g) * u) @ w[p + f"moe.experts.{e}.down.weight"].T)
        x = x + y
    return plain.rms_norm(x, w["model.norm.weight"], cfg.eps) @ w["lm_head.weight"].T, None


@pytest.fixture(scope="module")
def routed(tmp_path_factory):
    from acorninfer_b200.weights.random_init import write_random_model
    FEED_FORWARDS.register("toy_top1_experts", Top1Experts)
    register_architecture(RoutedConfig.architecture, RoutedConfig, routed_spec)
    cfg = RoutedConfig()
    d = write_random_model(tmp_path_factory.mktemp("routed"), cfg, seed=21, sigma=0.15, sigma_norm=0.1)
    yield cfg, d
    unregister_architecture(RoutedConfig.architecture)


def test_routed_feed_forward_and_partial_interleaved_rope_float32(routed):
    """float32 only: with bfloat16 rounding a token near a routing boundary may pick another expert,
    which is a property of routing, not a fault."""
    from acorninfer_b200.engine.runner import ModelRunner
    from acorninfer_b200.replay import TraceSession
    cfg, d = routed
    w = read_weights(d)
    reqs = {f"m{i}": random_tokens(n, cfg.vocab_size, 90 + i) for i, n in enumerate([41, 36, 50])}
    ref = {rid: routed_plain(cfg, w, toks)[0].numpy() for rid, toks in reqs.items()}
    for cut in ("whole", "decode_tail", "portions", "mixed"):
        steps = getattr(traces, cut)(reqs)
        runner = ModelRunner.from_model_dir(d, dtype="float32", num_blocks=-(-traces.max_live_tokens(steps) // 8),
                                            page_size=8, max_requests=4)
        assert not runner.decode_graph                      # the routed part reads the step on the host
        got = traces.collect(TraceSession(runner).step, steps)
        runner.manager.assert_balanced()
        for (rid, pos), row in got.items():
            assert np.abs(row - ref[rid][pos]).max() < 5e-5, (cut, rid, pos)
