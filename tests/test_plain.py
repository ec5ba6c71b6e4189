"""The plain implementation against the reference's own model code (golden outputs), and
against itself where a property must hold (causality, window)."""

import json
from pathlib import Path

import torch

from tests.golden.make_golden import CONFIGS, golden_tokens, golden_weights
from tests.plain import model as plain

GOLDEN = json.loads((Path(__file__).parent / "golden" / "qwen3_reference_logits.json").read_text())


def test_plain_matches_reference_model_outputs():
    for name, c in CONFIGS.items():
        g = GOLDEN[name]
        ids = golden_tokens(c)
        assert ids == g["tokens"]
        logits = plain.forward(c, golden_weights(c), ids, dtype=torch.float64)
        last = torch.tensor(g["logits_last"], dtype=torch.float64)
        assert (logits[-1] - last).abs().max() < 2e-5, name
        sums = torch.tensor(g["logits_row_sums"], dtype=torch.float64)
        assert (logits.sum(-1) - sums).abs().max() < 2e-3, name
        first = torch.tensor(g["logits_first4"], dtype=torch.float64)
        assert (logits[:, :4] - first).abs().max() < 2e-5, name


def test_plain_is_causal():
    c = CONFIGS["tiny_b"]
    w = golden_weights(c)
    ids = golden_tokens(c)
    full = plain.forward(c, w, ids)
    part = plain.forward(c, w, ids[:9])
    assert (full[:9] - part).abs().max() < 1e-9


def test_plain_window_equals_full_when_wide_and_differs_when_narrow():
    c = CONFIGS["tiny_a"]
    w = golden_weights(c)
    ids = golden_tokens(c)
    full = plain.forward(c, w, ids)
    wide = plain.forward(c, w, ids, windows=[len(ids), len(ids)])
    narrow = plain.forward(c, w, ids, windows=[3, 3])
    assert (full - wide).abs().max() < 1e-12
    assert (full[:3] - narrow[:3]).abs().max() < 1e-12
    assert (full[5:] - narrow[5:]).abs().max() > 1e-6


def test_plain_sampling_processing():
    x = torch.tensor([0.1, 2.0, 1.0, -1.0, 1.5])
    p = plain.process_logits(x, 1.0, top_k=2)
    assert torch.isinf(p).tolist() == [True, False, True, True, False]
    p = plain.process_logits(x, 0.5, top_p=0.5)
    assert not torch.isinf(p[1])
    tok, lp, _ = plain.sample_with_uniform(plain.process_logits(x, 1.0), 0.0)
    assert tok == 0 and lp < 0


def test_plain_sampling_processing_matches_the_reference_sampler():
    """``process_logits`` against what the reference's own ``Sampler.process`` kept and left, for a
    dozen settings (tests/golden/make_sampler_golden.py wrote the file from the reference's code)."""
    cases = json.loads((Path(__file__).parent / "golden" / "sampler_reference_processing.json").read_text())
    assert len(cases) >= 12
    for c in cases:
        logits = torch.tensor([float(x) for x in c["logits"]], dtype=torch.float32)
        got = plain.process_logits(logits, c["temperature"], c["top_k"], c["top_p"])
        kept = torch.isfinite(got).nonzero().flatten().tolist()
        assert kept == c["kept"], (c["temperature"], c["top_k"], c["top_p"])
        want = torch.tensor([float(x) for x in c["processed_kept"]], dtype=torch.float64)
        assert (got[kept] - want).abs().max() < 1e-6
