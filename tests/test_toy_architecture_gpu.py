"""Another architecture, defined here and nowhere in the framework: a mixer with state of its
own (a running mean over the request's tokens, kept in a state slot) that reads a per-step array
it declared itself, a windowed attention layer beside it, a layer that runs twice, a run that
reads another run's cache, a scale after the token table and a cap on the logits.  It is
registered, built from a model folder and stepped through the same runner and replay, cut in
every way, and compared with a plain whole-sequence computation written here; its decode steps
are captured and replayed as CUDA graphs like the built-in model's."""

from dataclasses import dataclass
from typing import ClassVar

import numpy as np
import pytest
import torch

from acorninfer_b200.config.model_config import ModelConfig
from acorninfer_b200.parts.base import (MIXERS, STAGES, CacheNeeds, LayerSpec, Mixer, ModelSpec, PartSpec, ScheduleEntry,
                                        Stage, StateNeeds, TensorSpec)
from acorninfer_b200.registry import register_architecture, unregister_architecture
from tests import traces
from tests.plain import model as plain
from tests.tiny import random_tokens, read_weights

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    architecture: ClassVar[str] = "ToyStateForCausalLM"
    hidden_size: int = 40
    vocab_size: int = 97
    num_heads: int = 6
    num_kv_heads: int = 3
    head_dim: int = 16
    intermediate_size: int = 56
    window: int = 9
    eps: float = 1e-5
    theta: float = 3e4
    embedding_scale: float = 1.7
    logit_cap: float = 1.5

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: raw[k] for k in cls.__dataclass_fields__ if k in raw})


class RunningMean(Mixer):
    """out[t] = W . mean(x[0..t]) over the tokens of the request so far.  The sum and the count
    live in the request's state slot, so a portion continues where the last one stopped.

    Everything it needs of the step it reads on the device: the common arrays and one of its own,
    ``toy.token_slot`` (the state slot of every token), declared through ``step_arrays`` and built
    on the host by the step layer.  Nothing of the step is read on the host, so the mixer is
    ``graph_safe`` and the model's decode steps can be captured."""

    graph_safe = True

    def __init__(self, ctx, width):
        self.ctx, self.width, self.w = ctx, width, None

    def tensor_specs(self):
        return {"mean_proj.weight": TensorSpec((self.width, self.width))}

    def bind(self, tensors):
        self.w = tensors["mean_proj.weight"].contiguous()

    def cache_needs(self):
        return CacheNeeds(state=StateNeeds((self.width + 1,)))

    def step_arrays(self):
        return {"toy.token_slot": lambda plan: plan.row_slot[plan.token_row]}

    def forward(self, x, inputs, cache):
        from acorninfer_b200.kernels import ops
        T = x.shape[0]
        slot = inputs.extra["toy.token_slot"].long()                 # [T], on the device
        row = inputs.token_row.long()
        x32 = x.float()
        # sum over the tokens of the same row up to and including each token, as a masked product
        t = torch.arange(T, device=x.device)
        mask = ((row[:, None] == row[None, :]) & (t[None, :] <= t[:, None])).float()
        sums = cache.state[slot, :self.width] + mask @ x32
        counts = cache.state[slot, self.width] + mask.sum(1)
        out = (sums / counts[:, None]).to(x.dtype)
        cache.state.index_add_(0, slot, torch.cat([x32, torch.ones(T, 1, device=x.device)], dim=1))
        return ops.linear(out, self.w, out_dtype=self.ctx.dtype)


class ScaleRows(Stage):
    """x * factor, after the token table."""

    graph_safe = True

    def __init__(self, ctx, factor):
        self.factor = factor

    def forward(self, x, inputs):
        return x.mul_(self.factor)


class SoftCap(Stage):
    """cap * tanh(logits / cap), with a learned per-token bias on the logits to show that a stage
    may own tensors."""

    graph_safe = True

    def __init__(self, ctx, cap, vocab):
        self.cap, self.vocab, self.bias = cap, vocab, None

    def tensor_specs(self):
        return {"bias": TensorSpec((self.vocab,))}

    def bind(self, tensors):
        self.bias = tensors["bias"].float()

    def forward(self, x, inputs):
        return self.cap * torch.tanh((x + self.bias) / self.cap)


def toy_spec(cfg: ToyConfig) -> ModelSpec:
    norm = {"width": cfg.hidden_size, "eps": cfg.eps}
    ff = {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size}

    def attn(window):
        return {"hidden_size": cfg.hidden_size, "num_heads": cfg.num_heads, "num_kv_heads": cfg.num_kv_heads,
                "head_dim": cfg.head_dim, "qk_norm_eps": cfg.eps, "position": "rope", "scale": cfg.head_dim ** -0.5,
                "window": window}

    def layer(i, mixer):
        p = f"model.layers.{i}."
        return LayerSpec(PartSpec("prenorm", {}, p), mixer, PartSpec("swiglu", ff, p + "mlp."),
                         {"mixer": PartSpec("rmsnorm", norm, p + "input_layernorm."),
                          "feed_forward": PartSpec("rmsnorm", norm, p + "post_attention_layernorm.")})

    layers = (layer(0, PartSpec("toy_running_mean", {"width": cfg.hidden_size}, "model.layers.0.mixer.")),
              layer(1, PartSpec("attention", attn(cfg.window), "model.layers.1.self_attn.")),
              layer(2, PartSpec("attention", attn(None), "model.layers.2.self_attn.")))
    # layer 1 runs twice (each run keeps a cache of its own); the last run of layer 2 reads the
    # cache its first run wrote
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(1), ScheduleEntry(2, reads_cache_of=2))
    return ModelSpec(cfg.vocab_size, cfg.hidden_size, "model.embed_tokens.weight", layers, schedule,
                     PartSpec("rmsnorm", norm, "model.norm."), "lm_head.weight",
                     {"rope": PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.theta})},
                     after_embedding=(PartSpec("toy_scale", {"factor": cfg.embedding_scale}),),
                     after_head=(PartSpec("toy_softcap", {"cap": cfg.logit_cap, "vocab": cfg.vocab_size}, "logit_cap."),))


def toy_plain(cfg: ToyConfig, weights, ids):
    """Whole-sequence computation of the toy model in float64 from the plain formulas."""
    w = {k: v.double() for k, v in weights.items()}
    sizes = {"num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
             "rms_norm_eps": cfg.eps, "rope_theta": cfg.theta}
    ids = torch.as_tensor(ids)
    pos = torch.arange(len(ids))
    x = w["model.embed_tokens.weight"][ids] * cfg.embedding_scale
    kv_of_entry = {}
    for entry, (layer, reads) in enumerate([(0, None), (1, None), (2, None), (1, None), (2, 2)]):
        p = f"model.layers.{layer}."
        h = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg.eps)
        if layer == 0:
            mean = torch.cumsum(h, 0) / torch.arange(1, len(ids) + 1, dtype=torch.float64)[:, None]
            a = mean @ w[p + "mixer.mean_proj.weight"].T
        else:
            a, kv = plain.attention_block(h, w, p + "self_attn.", sizes, pos, cfg.window if layer == 1 else None,
                                          kv_of_entry.get(reads))
            kv_of_entry[entry] = kv
        x = x + a
        x = x + plain.swiglu_mlp(plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg.eps), w, p + "mlp.")
    logits = plain.rms_norm(x, w["model.norm.weight"], cfg.eps) @ w["lm_head.weight"].T
    return cfg.logit_cap * torch.tanh((logits + w["logit_cap.bias"]) / cfg.logit_cap)


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from acorninfer_b200.weights.random_init import write_random_model
    MIXERS.register("toy_running_mean", RunningMean)
    STAGES.register("toy_scale", ScaleRows)
    STAGES.register("toy_softcap", SoftCap)
    register_architecture(ToyConfig.architecture, ToyConfig, toy_spec)
    cfg = ToyConfig()
    d = write_random_model(tmp_path_factory.mktemp("toy"), cfg, seed=9, sigma=0.08, sigma_norm=0.1)
    yield cfg, d
    unregister_architecture(ToyConfig.architecture)


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 8e-2)])
def test_toy_architecture_runs_through_the_same_runner_and_replay(toy, dtype, tol):
    from acorninfer_b200.engine.runner import ModelRunner
    from acorninfer_b200.replay import TraceSession

    cfg, d = toy
    w = read_weights(d)
    reqs = {f"t{i}": random_tokens(n, cfg.vocab_size, 70 + i) for i, n in enumerate([45, 38, 61, 50, 33])}
    ref = {rid: toy_plain(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    for cut in ("whole", "decode_tail", "portions", "mixed"):
        steps = getattr(traces, cut)(reqs)
        runner = ModelRunner.from_model_dir(d, dtype=dtype, num_blocks=-(-traces.max_live_tokens(steps) // 8),
                                            page_size=8, max_requests=4)
        assert len(runner.manager.groups) == 2 and len(runner.manager.state) == 1   # window, full; one state
        assert runner.decode_graph and "toy.token_slot" in runner.step_arrays         # every part is graph_safe
        got = traces.collect(TraceSession(runner).step, steps)
        runner.manager.assert_balanced()
        if cut == "decode_tail":
            assert runner.graph_replays >= 5 * 29          # 32 single-token steps a request: seen, captured, replayed
        for (rid, pos), row in got.items():
            assert np.abs(row - ref[rid][pos]).max() < tol, (cut, rid, pos)


def test_toy_architecture_through_the_engine_with_a_tight_pool(toy):
    """The same toy model (state slots, a windowed group beside a full one) under the scheduler:
    greedy generation with a token budget and so few pages that requests are preempted and
    recomputed; every generated token is the plain computation's best (float32)."""
    from acorninfer_b200.engine.engine import Engine
    from acorninfer_b200.engine.runner import ModelRunner
    from acorninfer_b200.sampling.params import SamplingParams

    cfg, d = toy
    w = read_weights(d)
    prompts = [random_tokens(n, cfg.vocab_size, 500 + n) for n in (14, 9, 21, 5)]
    runner = ModelRunner.from_model_dir(d, dtype="float32", num_blocks=9, page_size=8, max_requests=3)
    eng = Engine(runner, max_running=3, watermark_blocks=0, chunked_budget=10)
    ids = [eng.submit(p, SamplingParams(temperature=0.0), max_tokens=24, eos_ids=()) for p in prompts]
    steps = 0
    while eng.has_pending():
        eng.step()
        steps += 1
        assert steps < 1000
    assert sum(eng.seqs[i].preemptions for i in ids) >= 1          # the pool was tight enough to preempt
    for i, p in zip(ids, prompts):
        out = eng.seqs[i].all_ids
        assert len(out) == len(p) + 24
        logits = toy_plain(cfg, w, out[:-1])
        for j in range(len(p), len(out)):
            row = logits[j - 1]
            assert float(row.max() - row[out[j]]) < 1e-5, (i, j)
    eng.assert_balanced()
