"""Each part alone, built from its parameters only, against the plain formulas: norm,
position encoding, attention mixer (also windowed, and with the step cut in two), feed-forward,
and their arrangement in a block.  Sizes differ from every model configuration in the tests."""

import pytest
import torch

from acorninfer_b200.parts.base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, BuildContext,
                                        PartSpec, build_part)
from tests.plain import model as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
SIZES = {"num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 48, "rms_norm_eps": 2e-5, "rope_theta": 7e4}
H, I = 72, 136


def context(dtype):
    import acorninfer_b200.parts  # noqa: F401
    ctx = BuildContext(dtype=dtype, device=DEV, page_size=8)
    ctx.positions["rope"] = build_part(POSITION_ENCODINGS, PartSpec("rope", {"head_dim": 48, "theta": 7e4}), ctx)
    return ctx


def random_bind(part, dtype, seed, sigma=0.1):
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, spec in part.tensor_specs().items():
        t = torch.randn(spec.shape, generator=g)
        t = (1 + 0.1 * t) if spec.init == "norm" else sigma * t
        tensors[name] = t.to(torch.bfloat16).float() if dtype == torch.bfloat16 else t
    part.bind({k: v.to(DEV, dtype) for k, v in tensors.items()})
    return {k: v.double() for k, v in tensors.items()}


class MixerHarness:
    """A cache manager, workspace and entry cache for one mixer, driven like the runner does."""

    def __init__(self, mixer, dtype):
        from acorninfer_b200.cache.manager import CacheManager
        from acorninfer_b200.engine.batch import StepWorkspace
        from acorninfer_b200.models.decoder import EntryCache
        needs = mixer.cache_needs()
        self.manager = CacheManager({0: needs.kv}, {}, 64, 8, 4, dtype=dtype, device=DEV)
        k, v = self.manager.kv_pages(0)
        self.cache = EntryCache(0, 0, k, v, True, None)
        self.ws = StepWorkspace(DEV, 1 << 16)
        self.mixer = mixer

    def step(self, rows):
        """rows: list of (RequestCache, x [n, H]); returns the mixer's output per row."""
        from acorninfer_b200.engine.batch import StepEntry, plan_step
        entries = [StepEntry(rc, [0] * x.shape[0], []) for rc, x in rows]
        for e in entries:
            self.manager.extend(e.cache, e.cache.length + len(e.tokens))
        inputs = self.ws.upload(plan_step(entries, self.manager, self.mixer.step_arrays()))
        out = self.mixer.forward(torch.cat([x for _, x in rows]).contiguous(), inputs, self.cache)
        for e in entries:
            self.manager.commit(e.cache, e.cache.length + len(e.tokens))
        return out


TOL = {torch.float32: dict(atol=2e-5, rtol=1e-4), torch.bfloat16: dict(atol=3e-2, rtol=3e-2)}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    ctx = context(dtype)
    norm = build_part(NORMS, PartSpec("rmsnorm", {"width": H, "eps": 2e-5}), ctx)
    w = random_bind(norm, dtype, 1)
    x = torch.randn(11, H, device=DEV)
    d = torch.randn(11, H, device=DEV).to(dtype)
    assert torch.allclose(norm.forward(x.clone()).double().cpu(),
                          plain.rms_norm(x.double().cpu(), w["weight"], 2e-5), **TOL[dtype])
    r = x.clone()
    out = norm.add_forward(r, d)
    assert torch.allclose(r, x + d.float())
    assert torch.allclose(out.double().cpu(), plain.rms_norm((x + d.float()).double().cpu(), w["weight"], 2e-5), **TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 10])
def test_attention_mixer_part_whole_and_cut(dtype, window):
    ctx = context(dtype)
    params = {"hidden_size": H, "num_heads": 6, "num_kv_heads": 2, "head_dim": 48, "qk_norm_eps": 2e-5,
              "position": "rope", "scale": 48 ** -0.5, "window": window}
    mixer = build_part(MIXERS, PartSpec("attention", params), ctx)
    w = {"p." + k: v for k, v in random_bind(mixer, dtype, 2).items()}
    xs = [torch.randn(n, H).to(dtype) for n in (37, 20)]
    want = [plain.attention_block(x.double(), w, "p.", SIZES, torch.arange(x.shape[0]), window)[0] for x in xs]
    hz = MixerHarness(mixer, dtype)
    a, b = hz.manager.open("a"), hz.manager.open("b")
    # step 1: all of a, the first 9 tokens of b; step 2: the rest of b in one portion; then b token by token
    o1 = hz.step([(a, xs[0].to(DEV)), (b, xs[1][:9].to(DEV))])
    o2 = hz.step([(b, xs[1][9:17].to(DEV))])
    o3 = [hz.step([(b, xs[1][i:i + 1].to(DEV))]) for i in range(17, 20)]
    got_a = o1[:37]
    got_b = torch.cat([o1[37:], o2] + o3)
    assert torch.allclose(got_a.double().cpu(), want[0], **TOL[dtype])
    assert torch.allclose(got_b.double().cpu(), want[1], **TOL[dtype])
    hz.manager.close(a)
    hz.manager.close(b)
    hz.manager.assert_balanced()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    ctx = context(dtype)
    ff = build_part(FEED_FORWARDS, PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}), ctx)
    w = {"p." + k: v for k, v in random_bind(ff, dtype, 3).items()}
    x = torch.randn(15, H).to(dtype)
    assert torch.allclose(ff.forward(x.to(DEV), None).double().cpu(), plain.swiglu_mlp(x.double(), w, "p."), **TOL[dtype])


def test_feed_forward_part_with_only_its_gate_up_product_on_the_paired_kernel(monkeypatch):
    """Between the few rows of the one-CTA kernel and the many of a wholly fused layer, the gate/up
    product alone may run on the paired kernel with SwiGLU as its epilogue (its tiles fill the device
    first); forced here for 40 rows of a small part, the down product on the library."""
    from acorninfer_b200.kernels import ops
    monkeypatch.setattr(ops, "GEMM_PAIR_MIN_ROWS", 33)
    monkeypatch.setattr(ops, "GEMM_PAIR_MIN_FILL_ALONE", 0.0)
    monkeypatch.setattr(ops, "GEMM_PAIR_ALONE_MIN_K", 0)
    monkeypatch.setattr(ops, "fused_rows_ok", lambda rows, dtype, widths=None, num_sms=148: dtype == torch.bfloat16 and rows <= 32)
    ctx = context(torch.bfloat16)
    hidden, inter = 96, 192                          # intermediate size a multiple of 64: blocks of gate and up rows
    ff = build_part(FEED_FORWARDS, PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inter}), ctx)
    w = {"p." + k: v for k, v in random_bind(ff, torch.bfloat16, 5).items()}
    x = torch.randn(40, hidden).to(torch.bfloat16)
    before = dict(ops.COUNTS)
    got = ff.forward(x.to(DEV), None)
    ran = {k: v - before.get(k, 0) for k, v in ops.COUNTS.items() if v - before.get(k, 0)}
    assert ran.get("gemm_tc_pair") == 1 and "swiglu" not in ran
    assert torch.allclose(got.double().cpu(), plain.swiglu_mlp(x.double(), w, "p."), **TOL[torch.bfloat16])


@pytest.mark.parametrize("pairing,rot", [("half", 48), ("interleaved", 32)])
def test_position_encoding_part_constants(pairing, rot):
    ctx = context(torch.float32)
    rope = build_part(POSITION_ENCODINGS, PartSpec("rope", {"head_dim": 48, "theta": 7e4, "rotary_dim": rot,
                                                            "pairing": pairing}), ctx)
    want = 1.0 / (7e4 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    assert torch.equal(rope.inv_freq.cpu(), want) and rope.interleaved == (pairing == "interleaved")
    with pytest.raises(ValueError):
        build_part(POSITION_ENCODINGS, PartSpec("rope", {"head_dim": 48, "theta": 1e4, "rotary_dim": 50}), ctx)
    with pytest.raises(KeyError, match="known"):
        build_part(POSITION_ENCODINGS, PartSpec("alibi", {}), ctx)


def test_block_arrangement_part_float32():
    dtype = torch.float32
    ctx = context(dtype)
    params = {"hidden_size": H, "num_heads": 6, "num_kv_heads": 2, "head_dim": 48, "qk_norm_eps": 2e-5,
              "position": "rope", "scale": 48 ** -0.5, "window": None}
    mixer = build_part(MIXERS, PartSpec("attention", params), ctx)
    ff = build_part(FEED_FORWARDS, PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}), ctx)
    norms = {k: build_part(NORMS, PartSpec("rmsnorm", {"width": H, "eps": 2e-5}), ctx) for k in ("mixer", "feed_forward")}
    block = BLOCKS.get("prenorm")(ctx=ctx, mixer=mixer, feed_forward=ff, norms=norms)
    w = {}
    w.update({"model.layers.0.self_attn." + k: v for k, v in random_bind(mixer, dtype, 4).items()})
    w.update({"model.layers.0.mlp." + k: v for k, v in random_bind(ff, dtype, 5).items()})
    w["model.layers.0.input_layernorm.weight"] = random_bind(norms["mixer"], dtype, 6)["weight"]
    w["model.layers.0.post_attention_layernorm.weight"] = random_bind(norms["feed_forward"], dtype, 7)["weight"]
    x = torch.randn(29, H)
    want, _ = plain.decoder_layer(x.double(), w, 0, SIZES, torch.arange(29))
    hz = MixerHarness(mixer, dtype)
    rc = hz.manager.open("a")

    class BlockAsMixer:
        step_arrays = mixer.step_arrays

        def forward(self, xin, inputs, cache):
            resid, delta = block.forward(xin.float().clone(), None, inputs, cache)
            return resid + delta.float()
    hz.mixer = BlockAsMixer()
    got = hz.step([(rc, x.to(DEV))])
    assert torch.allclose(got.double().cpu(), want, atol=3e-5, rtol=1e-4)
    with pytest.raises(ValueError, match="norms"):
        BLOCKS.get("prenorm")(ctx=ctx, mixer=mixer, feed_forward=ff, norms={})
