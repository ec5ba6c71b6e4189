"""Generation through the entry point and the engine: greedy against the plain
implementation, the first tokens of a sequence, long decoding, sampling with known uniforms,
a token budget, and what happens when pages run out (preemption and recomputation give
the same tokens; a request that can never fit is stopped)."""

import pytest

from tests.plain import model as plain
from tests.tiny import TINY_A, TINY_B, TINY_C, TINY_D, make_model_dir, random_tokens, read_weights, sizes_of

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, tiny in (("a", TINY_A), ("b", TINY_B), ("c", TINY_C), ("d", TINY_D)):
        d = make_model_dir(tmp_path_factory.mktemp(name), tiny)
        out[name] = (tiny, d, read_weights(d))
    return out


def follows_plain(sizes, weights, prompt, ids, slack):
    """Every generated token is the plain model's best at its place, or within ``slack`` of it."""
    logits = plain.forward(sizes, weights, ids[:-1])
    for i in range(len(prompt), len(ids)):
        row = logits[i - 1]
        if float(row.max() - row[ids[i]]) > slack:
            return False
    return True


@pytest.mark.parametrize("which", ["a", "b", "c"])
def test_greedy_generate_matches_plain_float32(folders, which):
    from acorninfer_b200 import generate
    tiny, d, w = folders[which]
    cfg = tiny["cfg"]
    prompts = [random_tokens(n, cfg.vocab_size, 10 + n) for n in (5, 9, 13, 1)]
    got = generate(d, prompts, max_new_tokens=8, temperature=0.0, dtype="float32", page_size=tiny["page_size"],
                   num_blocks=64, eos_ids=())
    for p, ids in zip(prompts, got):
        assert ids[:len(p)] == p and len(ids) == len(p) + 8
        assert ids == plain.greedy_generate(sizes_of(cfg), w, p, 8) or follows_plain(sizes_of(cfg), w, p, ids, 1e-5)


def test_greedy_generate_bfloat16_follows_plain_within_rounding(folders):
    from acorninfer_b200 import generate
    tiny, d, w = folders["b"]
    cfg = tiny["cfg"]
    prompts = [random_tokens(n, cfg.vocab_size, 30 + n) for n in (7, 16, 23)]
    got = generate(d, prompts, max_new_tokens=10, dtype="bfloat16", page_size=8, num_blocks=64, eos_ids=())
    for p, ids in zip(prompts, got):
        assert follows_plain(sizes_of(cfg), w, p, ids, 0.06)


def test_first_tokens_and_eos(folders):
    """A one-token prompt; and generation stops after an eos id, which is kept."""
    from acorninfer_b200 import generate
    tiny, d, w = folders["a"]
    cfg = tiny["cfg"]
    ref = plain.greedy_generate(sizes_of(cfg), w, [17], 6)
    assert generate(d, [[17]], max_new_tokens=6, dtype="float32", page_size=4, num_blocks=16, eos_ids=())[0] == ref
    eos = ref[3]
    stopped = generate(d, [[17]], max_new_tokens=6, dtype="float32", page_size=4, num_blocks=16, eos_ids=(eos,))[0]
    assert stopped == ref[:ref.index(eos, 1) + 1]


def test_long_decoding_float32(folders):
    """300 decoded tokens, crossing many pages, checked against the plain model's logits."""
    from acorninfer_b200 import generate
    tiny, d, w = folders["c"]
    cfg = tiny["cfg"]
    p = random_tokens(6, cfg.vocab_size, 4)
    ids = generate(d, [p], max_new_tokens=300, dtype="float32", page_size=16, num_blocks=32, eos_ids=())[0]
    assert len(ids) == 306 and follows_plain(sizes_of(cfg), w, p, ids, 1e-5)


def test_temperature_sampling_uses_the_request_stream(folders):
    from acorninfer_b200 import generate
    from acorninfer_b200.kernels import ops
    tiny, d, w = folders["b"]
    cfg = tiny["cfg"]
    prompts = [random_tokens(n, cfg.vocab_size, 60 + n) for n in (1, 7, 16, 23)]
    kw = dict(max_new_tokens=10, temperature=0.7, seed=5, dtype="float32", page_size=8, num_blocks=64, eos_ids=())
    got = generate(d, prompts, chunked_budget=5, **kw)
    assert got == generate(d, prompts, **kw)             # same tokens whatever the batching
    alone = generate(d, prompts[2:3], **dict(kw, seed=7))[0]   # request 2 has seed 5 + 2
    assert alone == got[2]
    agree = total = 0
    for i, (p, ids) in enumerate(zip(prompts, got)):
        logits = plain.forward(sizes_of(cfg), w, ids[:-1])
        for j in range(len(p), len(ids)):
            u = ops.uniform(5 + i, j - len(p))
            want, _, margin = plain.sample_with_uniform(plain.process_logits(logits[j - 1], 0.7), u)
            if margin > 1e-4:
                total += 1
                agree += int(want == ids[j])
    assert total >= 20 and agree == total


def test_pages_run_out_preempts_and_recomputes_the_same_tokens(folders):
    from acorninfer_b200.generation import build_engine, generate_with_engine
    tiny, d, w = folders["a"]
    cfg = tiny["cfg"]
    prompts = [random_tokens(n, cfg.vocab_size, 80 + n) for n in (12, 12, 9)]
    roomy = build_engine(d, dtype="float32", page_size=4, num_blocks=64, watermark_blocks=0, max_running=3)
    want = generate_with_engine(roomy, prompts, max_new_tokens=12, eos_ids=())
    tight = build_engine(d, dtype="float32", page_size=4, num_blocks=9, watermark_blocks=0, max_running=3)
    got = generate_with_engine(tight, prompts, max_new_tokens=12, eos_ids=())
    assert got == want
    tight.assert_balanced()


def test_preemption_is_counted_and_capacity_stops_a_request_that_cannot_fit(folders):
    from acorninfer_b200.generation import build_engine
    from acorninfer_b200.sampling.params import SamplingParams
    tiny, d, w = folders["a"]
    eng = build_engine(d, dtype="float32", page_size=4, num_blocks=6, watermark_blocks=0, max_running=2)
    a = eng.submit(list(range(1, 13)), SamplingParams(temperature=0.0), max_tokens=8, eos_ids=())
    b = eng.submit(list(range(21, 33)), SamplingParams(temperature=0.0), max_tokens=3, eos_ids=())
    while eng.has_pending():
        eng.step()
    assert eng.seqs[a].preemptions >= 1 and len(eng.seqs[a].generated_ids) == 8 and len(eng.seqs[b].generated_ids) == 3
    ref = plain.greedy_generate(sizes_of(tiny["cfg"]), w, list(range(1, 13)), 8)
    assert eng.seqs[a].all_ids == ref
    # 4 + 40 tokens need 11 pages; the pool has 6: stopped with a reason, not waiting for ever
    c = eng.submit([5, 6, 7, 8], SamplingParams(temperature=0.0), max_tokens=40, eos_ids=())
    steps = 0
    while eng.has_pending():
        eng.step()
        steps += 1
        assert steps < 200
    assert eng.seqs[c].stop_reason == "capacity" and 16 <= len(eng.seqs[c].generated_ids) < 40
    eng.assert_balanced()
    with pytest.raises(ValueError, match="never be admitted"):
        eng.submit(list(range(1, 30)), max_tokens=1)


def test_command_line(folders, capsys):
    from acorninfer_b200.cli import main
    tiny, d, w = folders["a"]
    rc = main(["generate", "--model-dir", str(d), "--prompt-ids", "5,6,7", "--max-new-tokens", "4", "--dtype", "float32",
               "--page-size", "4", "--num-blocks", "16"])
    out = capsys.readouterr().out.strip().splitlines()[-1]
    ids = [int(t) for t in out.split(",")]
    ref = plain.greedy_generate(sizes_of(tiny["cfg"]), w, [5, 6, 7], 4)
    eos = set(tiny["cfg"].eos_token_id)
    stop = next((i for i in range(3, len(ref)) if ref[i] in eos), len(ref) - 1)     # the configuration's eos ids apply
    assert rc == 0 and (ids == ref[:stop + 1] or follows_plain(sizes_of(tiny["cfg"]), w, [5, 6, 7], ids, 1e-5))
    assert len(ids) == stop + 1


def run_engine(runner, prompts, lookahead, eos_ids, max_running=4, budget=11, watermark=1, base_tokens=9):
    from acorninfer_b200.engine.engine import Engine
    from acorninfer_b200.sampling.params import SamplingParams
    eng = Engine(runner, max_running=max_running, watermark_blocks=watermark, chunked_budget=budget, lookahead=lookahead)
    ids = []
    for i, p in enumerate(prompts):
        sp = SamplingParams(temperature=0.0) if i % 2 == 0 else SamplingParams(temperature=0.8, top_k=20, seed=i)
        ids.append(eng.submit(p, sp, max_tokens=base_tokens + i % 7, eos_ids=eos_ids))
    steps = 0
    while eng.has_pending():
        eng.step()
        steps += 1
        assert steps < 2000
    eng.assert_balanced()
    return [(eng.seqs[i].all_ids, eng.seqs[i].stop_reason) for i in ids], sum(eng.seqs[i].preemptions for i in ids)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_lookahead_gives_the_same_tokens_as_reading_every_step(folders, dtype):
    """One step ahead (ids stay on the device, the host reads them a call later) and step by step
    give the same sequences: greedy and sampled, with eos stops, a token budget and a tight pool."""
    from acorninfer_b200.engine.runner import ModelRunner
    tiny, d, w = folders["b"]
    cfg = tiny["cfg"]
    prompts = [random_tokens(n, cfg.vocab_size, 300 + n) for n in (3, 17, 9, 26, 1, 12)]
    make = lambda: ModelRunner.from_model_dir(d, dtype=dtype, num_blocks=14, page_size=8, max_requests=4)
    # eos ids taken from what the requests generate when nothing stops them: some tokens from the
    # middle of two generations, so that stops by eos (the wasted row of a step ahead) do happen
    free_run, _ = run_engine(make(), prompts, False, ())
    eos = (free_run[0][0][len(prompts[0]) + 4], free_run[3][0][len(prompts[3]) + 6])
    results = {look: run_engine(make(), prompts, look, eos)[0] for look in (False, True)}
    assert results[True] == results[False]
    assert sum(reason == "stop" for _, reason in results[True]) >= 2
    assert any(reason == "length" for _, reason in results[True])


def test_a_warmed_runner_serves_a_lookahead_engine_and_a_step_by_step_engine_alike(folders):
    """Graphs captured by ``warm_up`` (no row takes its id from the device) are replayed by an engine a
    step ahead (every decoded row does), then by one that reads every step, on the same runner: the
    place of every array a graph reads must not depend on how many ids come from the device."""
    from acorninfer_b200.engine.runner import ModelRunner
    tiny, d, w = folders["d"]
    cfg = tiny["cfg"]
    runner = ModelRunner.from_model_dir(d, dtype="bfloat16", num_blocks=96, page_size=16, max_requests=8)
    runner.warm_up(prompt_tokens=(16,), decode_rows=(1, 2, 3, 4, 5, 6))
    prompts = [random_tokens(n, cfg.vocab_size, 700 + n) for n in (5, 19, 33, 8, 27, 12)]
    replays = runner.graph_replays
    ahead, _ = run_engine(runner, prompts, True, (), max_running=6, budget=64, base_tokens=12)
    assert runner.graph_replays > replays + 5
    by_step, _ = run_engine(runner, prompts, False, (), max_running=6, budget=64, base_tokens=12)
    assert ahead == by_step
    cold = ModelRunner.from_model_dir(d, dtype="bfloat16", num_blocks=96, page_size=16, max_requests=8, decode_graph=False)
    assert run_engine(cold, prompts, False, (), max_running=6, budget=64, base_tokens=12)[0] == by_step
    for i in range(0, len(prompts), 2):                       # the greedy ones follow the plain model
        assert follows_plain(sizes_of(cfg), w, prompts[i], by_step[i][0], 0.06)


@pytest.mark.parametrize("lookahead", [False, True])
def test_more_than_32_requests_decode_together(folders, lookahead):
    """44 requests at once: decode batches above 32 rows (buckets 40 and 48 with padding rows, library
    products), a step ahead (ids from the device) and step by step; greedy ones against the plain model."""
    from acorninfer_b200.engine.runner import ModelRunner
    tiny, d, w = folders["d"]
    cfg = tiny["cfg"]
    prompts = [random_tokens(3 + (7 * i) % 18, cfg.vocab_size, 900 + i) for i in range(44)]
    runner = ModelRunner.from_model_dir(d, dtype="bfloat16", num_blocks=44 * 3 + 8, page_size=16, max_requests=44)
    got, _ = run_engine(runner, prompts, lookahead, (), max_running=44, budget=256, watermark=2, base_tokens=10)
    assert runner.graph_replays >= 3 and any(key[1] >= 40 for key in runner._graphs)      # a bucket above 32 rows was captured
    for i in range(0, len(prompts), 2):
        assert follows_plain(sizes_of(cfg), w, prompts[i], got[i][0], 0.06), i
    if lookahead:
        ref_runner = ModelRunner.from_model_dir(d, dtype="bfloat16", num_blocks=44 * 3 + 8, page_size=16, max_requests=44)
        assert got == run_engine(ref_runner, prompts, False, (), max_running=44, budget=256, watermark=2, base_tokens=10)[0]


def test_preemption_and_recomputation_in_bfloat16_follow_the_plain_model(folders):
    """A pool so tight that requests are preempted and recomputed, on the fast kernels (head size 128,
    bfloat16, a step ahead): the greedy tokens are still the plain model's within rounding."""
    from acorninfer_b200.engine.runner import ModelRunner
    tiny, d, w = folders["d"]
    cfg = tiny["cfg"]
    prompts = [random_tokens(n, cfg.vocab_size, 1100 + n) for n in (40, 23, 35, 18, 29)]
    runner = ModelRunner.from_model_dir(d, dtype="bfloat16", num_blocks=11, page_size=16, max_requests=4)
    from acorninfer_b200.engine.engine import Engine
    from acorninfer_b200.sampling.params import SamplingParams
    eng = Engine(runner, max_running=4, watermark_blocks=0, chunked_budget=48, lookahead=True)
    ids = [eng.submit(p, SamplingParams(temperature=0.0), max_tokens=40, eos_ids=()) for p in prompts]
    steps = 0
    while eng.has_pending():
        eng.step()
        steps += 1
        assert steps < 2000
    eng.assert_balanced()
    assert sum(eng.seqs[i].preemptions for i in ids) >= 2
    for i, p in zip(ids, prompts):
        assert len(eng.seqs[i].all_ids) == len(p) + 40
        assert follows_plain(sizes_of(cfg), w, p, eng.seqs[i].all_ids, 0.06), i


def test_padded_prompt_graphs_change_no_token_in_float32(folders):
    """One request at a time, so that every prompt (and every portion of a prompt cut by the budget) is
    alone in its step: with graphs such steps are padded to 32 tokens and replayed, without graphs they run
    as they are.  The float32 kernels give a row the same bits whatever else is in the step, so the two
    engines must generate exactly the same tokens, greedy and sampled; lengths repeat so that buckets are
    captured and replayed."""
    from acorninfer_b200.engine.runner import ModelRunner
    tiny, d, w = folders["b"]
    cfg = tiny["cfg"]
    lengths = (3, 17, 40, 33, 2, 31, 64, 17, 40, 5, 50, 33, 20, 61)
    prompts = [random_tokens(n, cfg.vocab_size, 900 + i) for i, n in enumerate(lengths)]
    out = {}
    for graphs in (False, True):
        runner = ModelRunner.from_model_dir(d, dtype="float32", num_blocks=40, page_size=8, max_requests=2, decode_graph=graphs)
        out[graphs] = run_engine(runner, prompts, True, (), max_running=1, budget=48, watermark=1)[0]
        if graphs:
            assert runner.prefill_graph and runner.graph_replays > 20
    assert out[False] == out[True]
