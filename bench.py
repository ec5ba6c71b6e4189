"""Benchmark of acorninfer_b200: decode tokens/s at Qwen3-8B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers N] [--impl ours|reference]

Prints ONE JSON line.  A step is one decode step of a batch of 8 requests at the context
length of the reference configuration (2,048-token prompts + 2,048 generated tokens: the
timed steps end at context 4,096).  ``value`` is decoded tokens per second timed on the
device with CUDA events (token ids prepared beforehand, sampling kernel included);
``e2e`` is the same through ``Engine.step()``: host token ids in, sampled ids out, every
step.  ``prefill`` is one 2,048-token prompt in one step; ``points`` are decode at batch
1 and 64 (and all three batches again at context 3,072, the middle of the generation); ``roofline`` compares the bytes a decode step must read (every weight once,
the cache of the live requests) with the measured copy bandwidth.  Weights are random
(seeded N(0, 0.02), norms 1), token ids uniform random: synthetic data.  Weights
(15 GB) are far larger than L2, so no L2 flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                intermediate_size=12288, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=151936,
                tie_word_embeddings=False, bos_token_id=None, eos_token_id=())
CONTEXT = 4096
PROMPT = 2048
PAGE = 16


def shared_config(args, peaks_source: str) -> dict:
    """The workload, printed alike by both arms (flat, at most 20 keys)."""
    return {"model": "Qwen3-8B sizes, random weights", "layers": args.layers,
            "layers_of_config": QWEN3_8B["num_hidden_layers"], "hidden": 4096, "q_heads": 32, "kv_heads": 8,
            "head_dim": 128, "intermediate": 12288, "vocab": 151936, "global_batch": args.batch,
            "seq_len": CONTEXT, "prompt": PROMPT, "page_size": PAGE, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (15 GB of weights per step)", "peaks": peaks_source,
            "kv": "device-timed value: synthetic pages (random K and V at full context); e2e: prompts prefilled by the engine under test"}


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows: list[list[str]] = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def model_numbers(c: dict, layers: int) -> dict:
    H, nq, nkv, d, I, V = (c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                           c["intermediate_size"], c["vocab_size"])
    per_layer = H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I
    return {"layer_params": per_layer, "weight_bytes": 2 * (layers * per_layer + V * H),
            "kv_bytes_per_token": 2 * layers * 2 * nkv * d, "nq": nq, "d": d, "H": H, "V": V}


def prefill_flops(nums: dict, layers: int, T: int) -> float:
    gemm = 2.0 * T * layers * nums["layer_params"] + 2.0 * nums["V"] * nums["H"]
    attn = layers * nums["nq"] * nums["d"] * 4.0 * (T * (T + 1) / 2)
    return gemm + attn


def synthetic_requests(runner, B: int, length: int, tag: str):
    """B live requests that hold ``length`` tokens each: pages taken through the manager, their
    contents random (what a prefill of random weights and tokens would leave, in distribution)."""
    out = []
    for i in range(B):
        rc = runner.open(f"{tag}{i}")
        runner.manager.extend(rc, length)
        runner.manager.commit(rc, length)
        out.append(rc)
    return out


def time_decode(runner, sampler, B: int, steps: int, warmup: int, ctx_end: int, torch):
    """Device-timed decode at batch B ending at context ``ctx_end``: tokens prepared beforehand,
    one step function call and one sampling launch per step, no host read in the loop."""
    from acorninfer_b200.engine.batch import StepEntry
    from acorninfer_b200.kernels import ops
    from acorninfer_b200.sampling.params import SamplingParams

    reqs = synthetic_requests(runner, B, ctx_end - steps - warmup, f"b{B}_")
    g = torch.Generator().manual_seed(B)
    toks = torch.randint(0, runner.vocab_size, (steps + warmup, B), generator=g).tolist()
    greedy = [SamplingParams(temperature=0.0)] * B
    dev = runner.device
    t_par = torch.zeros(B, dtype=torch.float32, device=dev)
    k_par = torch.zeros(B, dtype=torch.int32, device=dev)
    p_par = torch.ones(B, dtype=torch.float32, device=dev)
    s_par = torch.zeros(B, dtype=torch.int64, device=dev)

    def one(i):
        logits = runner.step([StepEntry(rc, [toks[i][r]], [0]) for r, rc in enumerate(reqs)])
        return ops.sample(logits, t_par, k_par, p_par, s_par, s_par)[0]

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    launches0 = ops.LAUNCHES + getattr(runner, "graph_kernel_launches", 0)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(warmup, warmup + steps):
        last = one(i)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    launches = ops.LAUNCHES + getattr(runner, "graph_kernel_launches", 0) - launches0
    assert int(last.min()) >= 0
    mean_ctx = ctx_end - steps / 2
    for rc in reqs:
        runner.close(rc)
    return {"ms_per_step": ms / steps, "tok_s": B * steps / (ms / 1e3), "launches": launches, "mean_context": mean_ctx}


def time_prefill(runner, T: int, repeats: int, torch):
    from acorninfer_b200.engine.batch import StepEntry
    g = torch.Generator().manual_seed(7)
    toks = torch.randint(0, runner.vocab_size, (T,), generator=g).tolist()
    best = None
    for i in range(repeats + 1):
        rc = runner.open(f"p{i}")
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry(rc, toks, [T - 1])])
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        runner.close(rc)
        if i > 0:
            best = ms if best is None else min(best, ms)
    return best


def time_first_token(runner, T: int, torch) -> float:
    """Milliseconds from a lone prompt of ``T`` host tokens to its first sampled token on the host (median of
    seven after three warm-up prompts): the step is padded to a bucket of token counts and replayed from a graph."""
    import statistics
    from acorninfer_b200.engine.batch import StepEntry
    from acorninfer_b200.kernels import ops
    g = torch.Generator().manual_seed(T)
    z32, zf, z64 = (torch.zeros(1, dtype=d, device=runner.device) for d in (torch.int32, torch.float32, torch.int64))
    one = torch.ones(1, dtype=torch.float32, device=runner.device)
    times = []
    for i in range(10):
        toks = torch.randint(0, runner.vocab_size, (T,), generator=g).tolist()
        rc = runner.open(f"ttft{T}_{i}")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        logits = runner.step([StepEntry(rc, toks, [T - 1])])
        tok = int(ops.sample(logits, zf, z32, one, z64, z64)[0].item())
        times.append((time.perf_counter() - t0) * 1e3)
        assert 0 <= tok < runner.vocab_size
        runner.close(rc)
    return statistics.median(times[3:])


def time_e2e(runner, B: int, steps: int, warmup: int, ctx_end: int, torch):
    """The same metric through the public engine: ``Engine.submit`` then ``Engine.step()``;
    every step copies that step's token ids and tables from pinned host memory to the device and
    reads the sampled token ids back."""
    from acorninfer_b200.engine.engine import Engine
    from acorninfer_b200.sampling.params import SamplingParams

    engine = Engine(runner, max_running=B, watermark_blocks=0, chunked_budget=2048, default_eos_ids=())
    # Prompts go through the engine in portions of 2,048 tokens; requests that finish their prompt
    # early decode while the others are still being read, so the prompts are shortened by the
    # number of such steps and the timed steps end at the context length.
    prefill_steps = -(-B * ctx_end // 2048)
    prompt_len = ctx_end - steps - warmup - prefill_steps
    g = torch.Generator().manual_seed(100 + B)
    prompts = torch.randint(0, runner.vocab_size, (B, prompt_len), generator=g).tolist()
    for p in prompts:
        engine.submit(p, SamplingParams(temperature=0.0), max_tokens=ctx_end, eos_ids=())
    while any(not r.generated_ids for r in engine.seqs.values()):
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    n = steps
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    produced = 0
    for _ in range(n):
        produced += len(engine.step())
    end.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms = max(start.elapsed_time(end), wall * 1e3)
    context_now = max(r.num_tokens for r in engine.seqs.values())
    lay_ints = 3 * B + (B + 1) + 2 * B + B + sum(2 * B + B * g.block_table.shape[1]
                                                   for g in runner.last_plan.groups) if hasattr(runner, "last_plan") else 0
    for sid in list(engine.seqs):
        engine.abort(sid)
    while engine.has_pending():          # the step still in flight is read and dropped
        engine.step()
    for sid in list(engine.seqs):
        engine.drop(sid)
    engine.assert_balanced()
    return {"value": produced / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms / n, "steps": n,
            "context_end": context_now,
            "h2d_bytes_per_step": 4 * lay_ints + 8 * 5 * B + 16 * B, "d2h_bytes_per_step": 4 * B}


def _mean_by_tag(records) -> dict:
    acc: dict = {}
    for what, tag, us in records:
        e = acc.setdefault((what, tag), [0, 0.0])
        e[0] += 1
        e[1] += us
    return {k: (n, total / n) for k, (n, total) in acc.items()}


def _in_step_contributions(runner, step, order: list, torch) -> dict:
    """Per (entry point, tag): the mean of what its launches add to the end time of a captured, replayed
    step (kernels overlap under programmatic dependent launch, so durations would count time twice),
    from the profiler's kernel records.  ``order`` is the step's launch list from an eager run, which the
    records must match in number; {} when they do not or the profiler is not to be had."""
    try:
        from torch.profiler import ProfilerActivity, profile
        for _ in range(4):              # seen, captured, replayed
            step()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "emcpy" not in e.name
               and "emset" not in e.name]
        evs.sort(key=lambda e: e.time_range.start)
        if len(evs) != len(order):
            return {}
        ends = sorted(range(len(evs)), key=lambda i: evs[i].time_range.end)
        prev = evs[0].time_range.start
        acc: dict = {}
        for i in ends:
            e = acc.setdefault(order[i], [0, 0.0])
            e[0] += 1
            e[1] += evs[i].time_range.end - prev
            prev = evs[i].time_range.end
        return {k: total / n for k, (n, total) in acc.items()}
    except Exception:
        return {}


def kernel_table(runner, nums: dict, conf: dict, B: int, ctx: int, T: int, pk: dict, torch) -> dict:
    """Every launch of one decode step (batch B at context ctx) and of one prefill step (T tokens),
    each timed alone with CUDA events in an eager step; the products, attention and the output
    matrix with the bytes they must read or the flops they do, against the measured peaks."""
    from acorninfer_b200.engine.batch import StepEntry
    from acorninfer_b200.kernels import ops

    H, nq, nkv, d, I, V = (conf["hidden_size"], conf["num_attention_heads"], conf["num_key_value_heads"],
                           conf["head_dim"], conf["intermediate_size"], conf["vocab_size"])
    hbm, tf = pk["hbm_gbs"], pk["bf16_tflops"]
    graphs, runner.decode_graph = runner.decode_graph, False

    def run_ahead():
        """Keeps the device busy for some 20 ms so that the host has queued the whole step before its
        first kernel starts: the events then bracket device time, not the host's launch latency."""
        torch.cuda.synchronize()
        torch.cuda._sleep(40_000_000)

    try:
        reqs = synthetic_requests(runner, B, ctx - 4, "kt")
        step = lambda: runner.step([StepEntry(rc, [7], [0]) for rc in reqs])
        step()
        run_ahead()
        with ops.kernel_timer() as timer:
            step()
        records = timer.records()
        dec = _mean_by_tag(records)
        # the same step captured and replayed, under the profiler: what each kernel adds to the step's end
        runner.decode_graph = graphs
        in_step = _in_step_contributions(runner, step, [(w, t) for w, t, _ in records], torch) if graphs else {}
        runner.decode_graph = False
        for rc in reqs:
            runner.close(rc)
        rc = runner.open("ktp")
        g = torch.Generator().manual_seed(11)
        toks = torch.randint(0, runner.vocab_size, (T,), generator=g).tolist()
        run_ahead()
        with ops.kernel_timer() as timer:
            runner.step([StepEntry(rc, toks, [T - 1])])
        pre = _mean_by_tag(timer.records())
        runner.close(rc)
    finally:
        runner.decode_graph = graphs

    def mem(key, nbytes):
        n, us = dec.get(key, (0, None))
        if us is None:
            return {"us": None}
        gbs = nbytes / us / 1e3
        out = {"us": round(us, 2), "calls": n, "MB": round(nbytes / 1e6, 2), "GBps": round(gbs, 1), "frac_hbm": round(gbs / hbm, 3)}
        if key in in_step:
            out["in_step_us"] = round(in_step[key], 2)
            out["in_step_frac_hbm"] = round(nbytes / in_step[key] / 1e3 / hbm, 3)
        return out

    def flop(key, flops):
        n, us = pre.get(key, (0, None))
        if us is None:
            return {"us": None}
        t = flops / us / 1e6
        return {"us": round(us, 1), "calls": n, "TFLOPS": round(t, 1), "frac_bf16": round(t / tf, 3)}

    qkv_n = (nq + 2 * nkv) * d
    decode = {
        "qkv_norm_rope_kvwrite": mem(("gemm_tc_qkv_rope", f"{B}x{qkv_n}x{H}"), 2 * qkv_n * H),
        "attention_decode": mem(("attention_decode_tma", ""), 2 * 2 * B * ctx * nkv * d),
        "attention_merge": {"us": round(dec.get(("attention_decode_merge", ""), (0, 0.0))[1], 2)},
        "o_add_norm": mem(("gemm_tc", f"{B}x{H}x{nq * d}"), 2 * H * nq * d),
        "gate_up_swiglu": mem(("gemm_tc", f"{B}x{2 * I}x{H}"), 2 * 2 * I * H),
        "down_add_norm": mem(("gemm_tc", f"{B}x{H}x{I}"), 2 * H * I),
        "lm_head": mem(("gemm_tc", f"{B}x{V}x{H}"), 2 * V * H),
        "sum_us_layer": round(sum(us for (what, tag), (n, us) in dec.items()
                                  if what.startswith(("gemm_tc", "attention")) and not tag.startswith(f"{B}x{V}x")), 1),
        "in_step_us_layer": round(sum(us for (what, tag), us in in_step.items()
                                      if what.startswith(("gemm_tc", "attention")) and not tag.startswith(f"{B}x{V}x")), 1),
    }
    def product(own: str, tag: str, flops: float):
        """A product of the prefill step: on the paired tcgen05 kernel of this library (with its fused
        epilogue) where the step's size lets its tiles fill the device, else the library's."""
        res = flop((own, tag), flops)
        if res["us"] is not None:
            return dict(res, kernel=own)
        return dict(flop(("library_gemm", tag), flops), kernel="library")

    prefill = {
        "attention_prefill": flop(("attention_prefill_tc", ""), nq * d * 4.0 * (T * (T + 1) / 2)),
        "qkv_norm_rope_kvwrite": product("gemm_tc_pair_qkv_rope", f"{T}x{qkv_n}x{H}", 2.0 * T * qkv_n * H),
        "o_add_norm": product("gemm_tc_pair", f"{T}x{H}x{nq * d}", 2.0 * T * H * nq * d),
        "gate_up_swiglu": product("gemm_tc_pair", f"{T}x{2 * I}x{H}", 2.0 * T * 2 * I * H),
        "down_add_norm": product("gemm_tc_pair", f"{T}x{H}x{I}", 2.0 * T * H * I),
        "library_products_us_step": round(sum(n * us for (what, tag), (n, us) in pre.items() if what == "library_gemm"), 1),
        "other_own_kernels_us_step": round(sum(n * us for (what, tag), (n, us) in pre.items()
                                          if what in ("add_rmsnorm", "swiglu", "qk_rope_kv", "rope_table", "embed")), 1),
    }
    return {"timing": "us: CUDA events around each launch of one eager step queued behind a busy device, each kernel alone; "
                      "in_step_us: what a launch adds to the end time of the captured, replayed step (profiler records; "
                      "kernels overlap through programmatic dependent launch); means over the layers",
            f"decode_b{B}_ctx{ctx}": decode, f"prefill_{T}": prefill}


def continuous_batching(torch) -> dict:
    """Qwen3-0.6B layer sizes, 128 requests arriving at once (prompts uniform in 16..1,024, outputs in
    16..512), token budget 2,048 a step, through ``Engine.submit/step``.  Run twice; the second run
    (graphs and library kernels warm) is timed by the wall clock."""
    from acorninfer_b200.bench import random_prompts
    from acorninfer_b200.config.presets import preset
    from acorninfer_b200.engine.engine import Engine
    from acorninfer_b200.engine.runner import ModelRunner
    from acorninfer_b200.registry import config_from_dict
    from acorninfer_b200.sampling.params import SamplingParams

    n_req, budget = 128, 2048
    cfg = config_from_dict(preset("qwen3-0.6b"))
    runner = ModelRunner.from_random(cfg, seed=0, dtype="bfloat16", num_blocks=n_req * (1024 + 512) // PAGE + 64,
                                     page_size=PAGE, max_requests=n_req, max_step_tokens=budget)
    gen = torch.Generator().manual_seed(4)
    lens = torch.randint(16, 1025, (n_req,), generator=gen).tolist()
    outs = torch.randint(16, 513, (n_req,), generator=gen).tolist()
    prompts = random_prompts(n_req, lens, runner.vocab_size, 4)
    result = {}
    for timed in (False, True):
        engine = Engine(runner, max_running=n_req, watermark_blocks=8, chunked_budget=budget, default_eos_ids=())
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        sids = [engine.submit(p, SamplingParams(temperature=0.0), max_tokens=n, eos_ids=()) for p, n in zip(prompts, outs)]
        while engine.has_pending():
            engine.step()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        total = sum(len(engine.seqs[i].generated_ids) for i in sids)
        assert total == sum(outs)
        for i in sids:
            engine.drop(i)
        engine.assert_balanced()
        result = {"model": "Qwen3-0.6B sizes, random weights, bf16", "requests": n_req, "token_budget": budget,
                  "prompt_tokens": sum(lens), "output_tokens": total, "output_tok_s": round(total / wall, 1),
                  "total_tok_s": round((total + sum(lens)) / wall, 1), "wall_s": round(wall, 3), "steps": engine.steps,
                  "mean_rows_per_step": round(engine.rows_launched / max(engine.steps, 1), 1),
                  "host_ms_per_step": round(engine.host_seconds / max(engine.steps, 1) * 1e3, 3),
                  "ms_per_step": round(wall / max(engine.steps, 1) * 1e3, 3)}
    del engine, runner
    return result


def long_context(steps: int, warmup: int, pk: dict, torch) -> dict:
    """Qwen3-32B layer sizes (64 layers, 65.5 GB of bfloat16 weights), 8 requests at context 16,384:
    device-timed decode steps on synthetic pages, and the fraction of the memory roofline."""
    from acorninfer_b200.config.presets import preset
    from acorninfer_b200.engine.runner import ModelRunner
    from acorninfer_b200.registry import config_from_dict

    raw = preset("qwen3-32b")
    cfg = config_from_dict(raw)
    B, ctx = 8, 16384
    runner = ModelRunner.from_random(cfg, seed=0, dtype="bfloat16", num_blocks=B * ctx // PAGE + 64, page_size=PAGE,
                                     max_requests=B + 1, max_step_tokens=4096)
    for g in runner.manager.groups:
        g.storage.normal_(0, 1)
    nums = model_numbers(raw, raw["num_hidden_layers"])
    res = time_decode(runner, None, B, steps, warmup, ctx, torch)
    step_bytes = nums["weight_bytes"] + B * res["mean_context"] * nums["kv_bytes_per_token"]
    gbs = step_bytes / (res["ms_per_step"] / 1e3) / 1e9
    del runner
    return {"model": "Qwen3-32B sizes, random weights, bf16", "layers": raw["num_hidden_layers"], "batch": B,
            "context": ctx, "ms_per_step": round(res["ms_per_step"], 3), "tok_s": round(res["tok_s"], 1),
            "step_GB": round(step_bytes / 1e9, 2), "GBps": round(gbs, 1), "frac_hbm": round(gbs / pk["hbm_gbs"], 4)}


def float32_path(pk: dict, torch) -> dict:
    """The true 32-bit path at Qwen3-8B layer sizes with 4 of the 36 layers (float32 weights, cache
    and products on the CUDA cores): a decode step at batch 8, context 4,096, and a 2,048-token
    prefill, device-timed.  It is the correctness path; the figures say how long a check takes."""
    from acorninfer_b200.config.model_config import Qwen3Config
    from acorninfer_b200.engine.runner import ModelRunner

    layers, B, steps, warmup = 4, 8, 8, 3
    conf = dict(QWEN3_8B, num_hidden_layers=layers)
    runner = ModelRunner.from_random(Qwen3Config(**conf), seed=0, sigma=0.02, dtype="float32",
                                     num_blocks=B * CONTEXT // PAGE + 2 * (PROMPT // PAGE) + 64, page_size=PAGE,
                                     max_requests=B + 2, max_step_tokens=4096)
    for g in runner.manager.groups:
        g.storage.normal_(0, 1)
    nums = model_numbers(conf, layers)
    res = time_decode(runner, None, B, steps, warmup, CONTEXT, torch)
    step_bytes = 2 * (nums["weight_bytes"] + B * res["mean_context"] * nums["kv_bytes_per_token"])   # 4-byte elements
    pre_ms = time_prefill(runner, PROMPT, 1, torch)
    del runner
    return {"model": "Qwen3-8B layer sizes, random weights, float32", "layers": layers,
            "layers_of_config": QWEN3_8B["num_hidden_layers"], "batch": B, "context": CONTEXT,
            "decode_ms_per_step": round(res["ms_per_step"], 3),
            "decode_GBps": round(step_bytes / (res["ms_per_step"] / 1e3) / 1e9, 1),
            "decode_frac_hbm": round(step_bytes / (res["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 4),
            "prefill_tokens": PROMPT, "prefill_ms": round(pre_ms, 2),
            "prefill_tflops": round(prefill_flops(nums, layers, PROMPT) / (pre_ms / 1e3) / 1e12, 2)}


def reference_arm(args) -> int:
    """The unmodified reference (installed under baseline/_ref) through its own public API:
    ``from_pretrained`` + ``Engine.submit/step`` with its fastest documented settings (Triton paged
    attention, fused ops, CUDA graph for decode).  Same metric and sizes: batch 8, context 4,096,
    Qwen3-8B layer sizes, random weights written to a temporary folder first."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "acorninfer").is_dir():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this box"}))
        return 0
    import shutil
    import tempfile
    tmp = Path(tempfile.mkdtemp(prefix="acorn_ref_model_"))
    try:
        import torch

        from acorninfer_b200.config.model_config import Qwen3Config, dump_config
        from acorninfer_b200.models.decoder import expected_tensors
        from acorninfer_b200.registry import spec_for
        from acorninfer_b200.weights.random_init import random_state
        from acorninfer_b200.weights.safetensors_io import write_safetensors

        conf = dict(QWEN3_8B, num_hidden_layers=args.layers, bos_token_id=0, eos_token_id=(151645,))
        cfg = Qwen3Config(**conf)
        dump_config(cfg, tmp)
        tensors = random_state(expected_tensors(spec_for(cfg)), 0, 0.02, 0.0, torch.bfloat16, "cuda:0")
        tensors = {k: v.cpu() for k, v in tensors.items()}
        write_safetensors(tmp / "model.safetensors", tensors)
        (tmp / "model.safetensors.index.json").write_text(json.dumps(
            {"weight_map": {k: "model.safetensors" for k in tensors}}))
        del tensors
        torch.cuda.empty_cache()

        sys.path.insert(0, str(ref))
        from acorninfer.engine.engine import Engine as RefEngine
        from acorninfer.models.qwen3 import from_pretrained
        from acorninfer.sampler import SamplingParams as RefParams

        model = from_pretrained(str(tmp), "cuda:0", torch.bfloat16)
        model.attention_backend = "triton"
        model.fused_ops = True
        model.decode_graph = True
        B, steps, warmup = args.batch, args.steps, max(args.warmup, 3)
        engine = RefEngine(model, None, num_blocks=B * CONTEXT // PAGE + 64, page_size=PAGE, max_running=B,
                           watermark_blocks=8)
        prompt_len = CONTEXT - steps - warmup - 1
        g = torch.Generator().manual_seed(100 + B)
        prompts = torch.randint(0, QWEN3_8B["vocab_size"], (B, prompt_len), generator=g).tolist()
        for p in prompts:
            engine.submit(p, RefParams(temperature=0.0), max_tokens=steps + warmup + 1, eos_ids=frozenset())
        while any(not engine.seqs[i].generated_ids for i in engine.seqs):
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        clocks = ClockSampler()
        clocks.start()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        produced = 0
        for _ in range(steps):
            produced += len(engine.step())
        end.record()
        torch.cuda.synchronize()
        ms = max(start.elapsed_time(end), (time.perf_counter() - t0) * 1e3)
        clock_info = clocks.stop()
        # What its decode step copies, counted from its own staging tensors: two pinned blocks to the
        # device (ids, positions, page and slot targets; lengths and block tables), one argmax list back.
        h2d = d2h = None
        runner_ = getattr(engine, "graph_runner", None)
        if runner_ is not None:
            st = runner_.states[min(b for b in runner_.states if b >= B)]
            h2d = st.pin_long.numel() * st.pin_long.element_size() + st.pin_i32.numel() * st.pin_i32.element_size()
            d2h = 8 * B
        line = {"impl": "reference", "metric": "decode tok/s at batch 8, context 4096 (Qwen3-8B layer sizes, 1 B200)",
                "value": round(produced / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
                "warmup": warmup, "ms_per_step": round(ms / steps, 4), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": shared_config(args, peaks()["source"]),
                "settings": "triton attention, fused ops, decode graph",
                "e2e": {"value": round(produced / (ms / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(ms / steps, 4),
                        "steps": steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
                "clocks": clock_info}
        print(json.dumps(line))
    except Exception as exc:  # the reference could not run here: say why, in one line
        reason = f"{type(exc).__name__}: {exc}".replace("\n", " ")[:300]
        print(json.dumps({"impl": "reference", "unavailable": reason}))
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"],
                    help="fewer layers than the configuration has (sizes of a layer stay)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="only the batch of the headline value")
    ap.add_argument("--skip-extra", action="store_true",
                    help="leave out the per-kernel table, the continuous-batching, long-context and float32 runs")
    args = ap.parse_args()
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from acorninfer_b200.config.model_config import Qwen3Config
    from acorninfer_b200.engine.runner import ModelRunner
    from acorninfer_b200.kernels import ops

    pk = peaks()
    conf = dict(QWEN3_8B, num_hidden_layers=args.layers)
    cfg = Qwen3Config(**conf)
    nums = model_numbers(conf, args.layers)
    max_b = max(args.batch, 1 if args.skip_points else 64)
    num_blocks = max_b * CONTEXT // PAGE + 2 * (PROMPT // PAGE) + 64
    runner = ModelRunner.from_random(cfg, seed=0, sigma=0.02, dtype="bfloat16", num_blocks=num_blocks, page_size=PAGE,
                                     max_requests=max_b + 2, max_step_tokens=4096)
    for g in runner.manager.groups:
        g.storage.normal_(0, 1)
    sampler = None

    clocks = ClockSampler()
    clocks.start()
    head = time_decode(runner, sampler, args.batch, args.steps, args.warmup, CONTEXT, torch)
    clock_info = clocks.stop()
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(time_decode(runner, sampler, b, args.steps, args.warmup, CONTEXT, torch)["tok_s"], 1)
        # the same three batches in the middle of the generation (context 3,072: prompt 2,048 + 1,024 generated)
        mid = PROMPT + (CONTEXT - PROMPT) // 2 + (args.steps + args.warmup) // 2
        for b in (1, 8, 64):
            points[f"decode_b{b}_ctx3072"] = round(time_decode(runner, sampler, b, args.steps, args.warmup, mid, torch)["tok_s"], 1)
    pre_ms = time_prefill(runner, PROMPT, 6, torch)
    if not args.skip_points:
        points["first_token_ms_prompt128"] = round(time_first_token(runner, 128, torch), 3)
    e2e = time_e2e(runner, args.batch, args.steps, args.warmup, CONTEXT, torch)
    extra = {}
    if not args.skip_extra:
        extra["kernels"] = kernel_table(runner, nums, conf, args.batch, CONTEXT, PROMPT, pk, torch)
        del runner                      # the other workloads build models of their own: free this one's memory first
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        extra["continuous_batching"] = continuous_batching(torch)
        gc.collect()
        torch.cuda.empty_cache()
        extra["long_context"] = long_context(min(args.steps, 32), 4, pk, torch)
        gc.collect()
        torch.cuda.empty_cache()
        extra["float32_path"] = float32_path(pk, torch)
        points["cb_0.6b_128req_output_tok_s"] = extra["continuous_batching"]["output_tok_s"]
        points["decode_32b_b8_ctx16384"] = extra["long_context"]["tok_s"]

    step_bytes = nums["weight_bytes"] + args.batch * head["mean_context"] * nums["kv_bytes_per_token"]
    achieved = step_bytes / (head["ms_per_step"] / 1e3) / 1e9
    flops = prefill_flops(nums, args.layers, PROMPT)
    line = {
        "metric": "decode tok/s at batch 8, context 4096 (Qwen3-8B layer sizes, 1 B200)",
        "value": round(head["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(head["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": shared_config(args, pk["source"]),
        "settings": "lookahead engine, captured decode steps, one-CTA tcgen05 products up to 32 rows, paired tcgen05 products "
                    "with fused epilogues where their tiles fill the device (the 2,048-token prefill), library products between",
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": head["launches"],
        "prefill": {"value": round(PROMPT / (pre_ms / 1e3), 1), "tokens": PROMPT, "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_info,
        **extra,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
