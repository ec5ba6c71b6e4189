"""Captured, padded all-decode steps give the same logits as plain launches of the same steps;
and the reference-style benchmark module runs on a tiny random model."""

import json

import numpy as np
import pytest

from tests.tiny import TINY_B, TINY_D, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tiny", [TINY_B, TINY_D], ids=["tiny_b", "tiny_d"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_with_padding_equals_plain_launches(tmp_path, tiny, dtype):
    from acorninfer_b200.engine.batch import StepEntry
    from acorninfer_b200.engine.runner import ModelRunner

    d = make_model_dir(tmp_path / "m", tiny)
    V = tiny["cfg"].vocab_size
    results = {}
    for graphs in (False, True):
        runner = ModelRunner.from_model_dir(d, dtype=dtype, num_blocks=64, page_size=tiny["page_size"], max_requests=8,
                                            decode_graph=graphs)
        reqs = [runner.open(i) for i in range(5)]
        for i, rc in enumerate(reqs):                       # prompts of different lengths
            runner.step([StepEntry(rc, random_tokens(3 + 4 * i, V, i), [])])
        outs = []
        for step in range(8):                               # 5 rows (bucket 5), then 3 rows, wanting 2 of them
            live = reqs if step < 4 else reqs[:3]
            want = (lambda i: [0]) if step < 4 else (lambda i: [0] if i != 1 else [])
            logits = runner.step([StepEntry(rc, [(7 * step + i) % V], want(i)) for i, rc in enumerate(live)])
            outs.append(logits.float().cpu().numpy().copy())
        if graphs:
            assert runner.graph_replays >= 4               # the repeated shapes were replayed
        results[graphs] = outs
        for rc in reqs:
            runner.close(rc)
        runner.manager.assert_balanced()
    tol = 1e-6 if dtype == "float32" else 2e-2
    for a, b in zip(results[False], results[True]):
        assert a.shape == b.shape and np.abs(a - b).max() <= tol


def test_bench_module_runs(tmp_path, capsys):
    from acorninfer_b200.bench import main
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(TINY_B["cfg"].to_dict()))
    rc = main(["--random-config", str(cfg), "--num-blocks", "64", "--page-size", "8", "--max-running", "4",
               "--watermark-blocks", "2", "--in-tokens", "12", "--out-tokens", "5", "--concurrency", "1", "3",
               "--chunked-budget", "16"])
    out = capsys.readouterr().out
    assert rc == 0 and out.count("RESULT C=") == 2 and "tok_s=" in out


def test_warm_up_captures_graphs_and_gives_everything_back(tmp_path):
    from acorninfer_b200.engine.batch import StepEntry
    from acorninfer_b200.engine.runner import ModelRunner
    from tests.tiny import TINY_D, make_model_dir
    d = make_model_dir(tmp_path / "m", TINY_D)
    runner = ModelRunner.from_model_dir(d, dtype="bfloat16", num_blocks=64, page_size=TINY_D["page_size"], max_requests=4)
    runner.warm_up(prompt_tokens=(16, 100, 10 ** 6), decode_rows=(1, 2, 9))     # sizes beyond the pools are left out
    runner.manager.assert_balanced()
    assert min(runner.manager.free_pages()) == 64 and runner.manager.slots.num_free == 4
    before = runner.graph_replays
    a = runner.open("a")
    runner.step([StepEntry(a, [1, 2, 3], [])])
    runner.step([StepEntry(a, [4], [0])])
    assert runner.graph_replays == before + 1          # the first decode step of a request replays a warmed graph


def test_a_step_too_large_for_the_workspace_is_refused_and_holds_nothing(tmp_path):
    """The step's arrays (here: block tables of many rows) do not fit the workspace: the step raises before
    anything is launched, the pages it had reserved go back, and the runner carries on."""
    from acorninfer_b200.engine.batch import BatchError, StepEntry
    from acorninfer_b200.engine.runner import ModelRunner
    d = make_model_dir(tmp_path / "m", TINY_B)
    runner = ModelRunner.from_model_dir(d, dtype="float32", num_blocks=64, page_size=TINY_B["page_size"], max_requests=8,
                                        workspace_ints=96)
    V = TINY_B["cfg"].vocab_size
    a = runner.open("a")
    logits = runner.step([StepEntry(a, random_tokens(5, V, 1), [4])])        # small steps fit
    assert logits.shape == (1, V)
    free = runner.manager.free_pages()
    others = [runner.open(i) for i in range(6)]
    with pytest.raises(BatchError, match="workspace holds"):
        runner.step([StepEntry(rc, random_tokens(9, V, 2), [8]) for rc in others])
    assert runner.manager.free_pages() == free and all(rc.length == 0 and rc.tables == [[]] for rc in others)
    again = runner.step([StepEntry(a, [7], [0])])
    assert again.shape == (1, V)
    for rc in [a] + others:
        runner.close(rc)
    runner.manager.assert_balanced()


@pytest.mark.parametrize("tiny", [TINY_B, TINY_D], ids=["tiny_b", "tiny_d"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_prompts_replay_padded_graphs_and_what_the_padding_wrote_is_never_read(tmp_path, tiny, dtype):
    """A prompt portion alone in its step is padded to a bucket of token counts and replayed from a
    captured graph.  Three prompts of 45 tokens (bucket 64): the third replays; every logit against
    the plain model.  The padding wrote keys and values at positions 45 .. 63 of the request's pages
    (and into the padding page beyond them): the request then decodes 30 tokens through those
    positions, and continues with a portion of 40 tokens that starts inside a page, all against the
    plain model."""
    import torch
    from acorninfer_b200.engine.batch import StepEntry
    from acorninfer_b200.engine.runner import ModelRunner
    from tests.plain import model as plain
    from tests.tiny import read_weights, sizes_of

    d = make_model_dir(tmp_path / "m", tiny)
    w, sizes, V = read_weights(d), sizes_of(tiny["cfg"]), tiny["cfg"].vocab_size
    tol = 2e-5 if dtype == "float32" else 6e-2
    runner = ModelRunner.from_model_dir(d, dtype=dtype, num_blocks=64, page_size=tiny["page_size"], max_requests=4)
    assert runner.prefill_graph
    seqs = [random_tokens(45 + 30 + 40, V, 70 + i) for i in range(3)]
    rcs = []
    for i, ids in enumerate(seqs):
        rc = runner.open(i)
        rcs.append(rc)
        before = runner.graph_replays
        got = runner.step([StepEntry(rc, ids[:45], list(range(45)))]).float().cpu().numpy()
        assert (runner.graph_replays == before + 1) == (i == 2)          # seen, captured, replayed
        want = plain.forward(sizes, w, ids[:45]).numpy()
        assert np.abs(got - want).max() < tol, f"prompt {i}"
    ids, rc = seqs[2], rcs[2]
    want = plain.forward(sizes, w, ids).numpy()
    for t in range(45, 75):                                              # through the slots the padding wrote
        got = runner.step([StepEntry(rc, [ids[t]], [0])]).float().cpu().numpy()
        assert np.abs(got[0] - want[t]).max() < tol, f"decoded token at {t}"
    got = runner.step([StepEntry(rc, ids[75:115], list(range(40)))]).float().cpu().numpy()     # a padded portion that starts at 75
    assert np.abs(got - want[75:115]).max() < tol
    # the other requests' pages were not touched: they decode on as the plain model says
    for i in (0, 1):
        full = plain.forward(sizes, w, seqs[i][:46]).numpy()
        got = runner.step([StepEntry(rcs[i], [seqs[i][45]], [0])]).float().cpu().numpy()
        assert np.abs(got[0] - full[45]).max() < tol
    for rc in rcs:
        runner.close(rc)
    runner.manager.assert_balanced()
    torch.cuda.synchronize()


def test_the_graph_replayed_longest_ago_makes_room(tmp_path, monkeypatch):
    """With room for two graphs, a third shape evicts the one replayed longest ago; the evicted shape is
    captured again when it comes back, and every step's logits stay what plain launches give."""
    from acorninfer_b200.engine import runner as runner_module
    from acorninfer_b200.engine.batch import StepEntry
    d = make_model_dir(tmp_path / "m", TINY_B)
    V = TINY_B["cfg"].vocab_size
    monkeypatch.setattr(runner_module, "MAX_GRAPHS", 2)
    plain = runner_module.ModelRunner.from_model_dir(d, dtype="float32", num_blocks=64, page_size=8, max_requests=8, decode_graph=False)
    graphs = runner_module.ModelRunner.from_model_dir(d, dtype="float32", num_blocks=64, page_size=8, max_requests=8)
    reqs = {r: [r.open(i) for i in range(3)] for r in (plain, graphs)}
    for r in (plain, graphs):
        for i, rc in enumerate(reqs[r]):
            r.step([StepEntry(rc, random_tokens(4 + i, V, i), [])])
    for step in range(18):
        rows = (1, 2, 3)[(step // 3) % 3]                                 # three shapes in turn, three steps each
        outs = []
        for r in (plain, graphs):
            logits = r.step([StepEntry(rc, [(5 * step + i) % V], [0]) for i, rc in enumerate(reqs[r][:rows])])
            outs.append(logits.float().cpu().numpy().copy())
        assert np.abs(outs[0] - outs[1]).max() <= 1e-6, step
        assert len(graphs._graphs) <= 2
    assert graphs.graph_replays >= 6                                      # the third step of every visit replays
    for r in (plain, graphs):
        for rc in reqs[r]:
            r.close(rc)
        r.manager.assert_balanced()
