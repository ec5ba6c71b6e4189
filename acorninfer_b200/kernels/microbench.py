"""Times one kernel of the library alone, at given sizes, with CUDA events.

    python -m acorninfer_b200.kernels.microbench gemm --m 8 --n 24576 --k 4096
    python -m acorninfer_b200.kernels.microbench attn-decode --batch 64 --context 4096
    python -m acorninfer_b200.kernels.microbench attn-prefill --tokens 2048
    python -m acorninfer_b200.kernels.microbench step --layers 8 --batch 8

Prints the time per call and the achieved GB/s (bytes the kernel must read) or TFLOPS.
Inputs are larger than L2 or rotated over several copies, so DRAM figures mean something;
calls are captured in a CUDA graph so that host launch time is not measured.  The same
command under ``ncu`` profiles the kernel (few launches: ``--reps 2 --graph 0``).
"""

from __future__ import annotations

import argparse

import torch

from . import ops
from .attention import decode_splits

DEV = "cuda:0"


def _time(fns, reps: int, graph: bool) -> float:
    """Microseconds per call of the callables in ``fns`` (cycled)."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(reps):
                fns[i % len(fns)]()
        g.replay()
        torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    if graph:
        g.replay()
    else:
        for i in range(reps):
            fns[i % len(fns)]()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / reps * 1e3


def bench_gemm(a) -> None:
    copies = max(2, int(400e6 // (a.n * a.k * 2)) + 1)
    ws = [torch.randn(a.n, a.k, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(a.m, a.k, device=DEV, dtype=torch.bfloat16)
    splits, per_sm = (a.splits, a.per_sm) if a.splits else ops.gemm_tc_plan(a.m, a.n, a.k)
    resid = torch.randn(a.m, a.n, device=DEV)
    norm_w = torch.ones(a.n, device=DEV)
    xin = x
    if a.normed:       # x arrives as rows that lack their RMS factor (32 partial sums a row)
        xin = ops.NormedRows(x, torch.rand(32, a.m, device=DEV) + 1.0, 1e-6, a.k)
    ep = ops.AddNormEpilogue(resid, norm_w, 1e-6) if a.epilogue == "add_norm" else None
    if a.kernel == "pair":
        us = _time([lambda w=w: ops.gemm_tc_pair(xin, w, torch.bfloat16, epilogue=ep, swiglu=a.epilogue == "swiglu")
                    for w in ws], a.reps, a.graph)
        lib = _time([lambda w=w: torch.mm(x, w.t()) for w in ws], a.reps, a.graph) if a.library else float("nan")
        fl = 2.0 * a.m * a.n * a.k
        print(f"gemm_tcgen05_pair M={a.m} N={a.n} K={a.k} epilogue={a.epilogue} normed={a.normed}: {us:.1f} us, "
              f"{fl / us / 1e6:.1f} TFLOPS; library product {lib:.1f} us, {fl / lib / 1e6:.1f} TFLOPS; "
              f"error flag {ops.gemm_tc_pair_error()}")
        return
    us = _time([lambda w=w: ops.gemm_tc(xin, w, torch.bfloat16, splits=splits, epilogue=ep,
                                        swiglu=a.epilogue == "swiglu", per_sm=per_sm) for w in ws], a.reps, a.graph)
    lib = _time([lambda w=w: torch.mm(x, w.t()) for w in ws], a.reps, a.graph) if a.library else float("nan")
    gb, fl = a.n * a.k * 2 / 1e9, 2.0 * a.m * a.n * a.k
    print(f"gemm_tcgen05 M={a.m} N={a.n} K={a.k} splits={splits} per_sm={per_sm} epilogue={a.epilogue} normed={a.normed}: {us:.1f} us, {gb / us * 1e6:.0f} GB/s of weights, "
          f"{fl / us / 1e6:.1f} TFLOPS; library product {lib:.1f} us; error flag {ops.gemm_tc_error()}")


def bench_attn_decode(a) -> None:
    nq, nkv, d, P, B, ctx = a.heads, a.kv_heads, a.head_dim, a.page, a.batch, a.context
    pages_per = ctx // P
    k_pages = torch.randn(B * pages_per, nkv, P, d, device=DEV, dtype=torch.bfloat16)
    v_pages = torch.randn_like(k_pages)
    table = torch.randperm(B * pages_per, device=DEV).to(torch.int32).view(B, pages_per).contiguous()
    base = torch.zeros(B, dtype=torch.int32, device=DEV)
    rows = torch.arange(B, dtype=torch.int32, device=DEV)
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=DEV)
    qkv = torch.randn(B, (nq + 2 * nkv) * d, device=DEV, dtype=torch.bfloat16)
    splits = a.splits or decode_splits(B, nkv, ctx, d)
    us = _time([lambda: ops.attention_decode(qkv, qkv.stride(0), k_pages, v_pages, table, base, rows, pos, B, nq, nkv,
                                             d, d ** -0.5, None, splits, use_tma=a.kernel != "mma")],
               a.reps, a.graph)
    gb = B * ctx * nkv * d * 2 * 2 / 1e9
    print(f"attention_decode[{'cp.async' if a.kernel == 'mma' else 'tma'}] B={B} context={ctx} heads={nq}/{nkv} d={d} page={P} splits={splits}: {us:.1f} us, "
          f"{gb / us * 1e6:.0f} GB/s of K and V")


def bench_attn_prefill(a) -> None:
    nq, nkv, d, P, T = a.heads, a.kv_heads, a.head_dim, a.page, a.tokens
    pages = -(-T // P)
    k_pages = torch.randn(pages, nkv, P, d, device=DEV, dtype=torch.bfloat16)
    v_pages = torch.randn_like(k_pages)
    table = torch.randperm(pages, device=DEV).to(torch.int32).view(1, pages).contiguous()
    base = torch.zeros(1, dtype=torch.int32, device=DEV)
    row_start = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    row_pos = torch.zeros(1, dtype=torch.int32, device=DEV)
    tiles = torch.tensor([(0, q0) for q0 in range(0, T, 64)], dtype=torch.int32, device=DEV)
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device=DEV, dtype=torch.bfloat16)
    if a.kernel == "tc":
        # the kernel starts CTAs in list order: the tiles that read the most keys first
        tiles = torch.tensor([(0, q0) for q0 in reversed(range(0, T, 128))], dtype=torch.int32, device=DEV)
        fn = lambda: ops.attention_prefill_tc(qkv, qkv.stride(0), k_pages, v_pages, table, base, row_start, row_pos,
                                              tiles, T, nq, nkv, d, d ** -0.5, None)
    else:
        fn = lambda: ops.attention_prefill(qkv, qkv.stride(0), k_pages, v_pages, table, base, row_start, row_pos,
                                           tiles, T, nq, nkv, d, d ** -0.5, None)
    us = _time([fn], a.reps, a.graph)
    fl = nq * d * 4.0 * (T * (T + 1) / 2)
    print(f"attention_prefill[{a.kernel}] tokens={T} heads={nq}/{nkv} d={d} page={P}: {us:.1f} us, {fl / us / 1e6:.0f} TFLOPS (causal)")


def bench_step(a) -> None:
    """What each kernel of one decode step adds to the step's end time (kernels overlap under
    programmatic dependent launch, so the sum of durations would count time twice), from the torch
    profiler's kernel records of a replayed step on a model of Qwen3-8B layer sizes."""
    import collections

    from torch.profiler import ProfilerActivity, profile

    from ..config.model_config import Qwen3Config
    from ..engine.batch import StepEntry
    from ..engine.runner import ModelRunner

    cfg = Qwen3Config(num_hidden_layers=a.layers, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                      head_dim=128, intermediate_size=12288, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=151936)
    runner = ModelRunner.from_random(cfg, seed=0, dtype="bfloat16", num_blocks=a.batch * a.context // 16 + 64,
                                     page_size=16, max_requests=a.batch + 1)
    for g in runner.manager.groups:
        g.storage.normal_(0, 1)
    reqs = []
    for i in range(a.batch):
        rc = runner.open(i)
        runner.manager.extend(rc, a.context - 16)
        runner.manager.commit(rc, a.context - 16)
        reqs.append(rc)
    one = lambda: runner.step([StepEntry(rc, [5], [0]) for rc in reqs])
    for _ in range(5):
        one()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(2):
            one()
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "emcpy" not in e.name]
    evs.sort(key=lambda e: e.time_range.start)
    starts = [i for i, e in enumerate(evs) if "embed_kernel" in e.name]
    evs = sorted(evs[starts[-1]:], key=lambda e: e.time_range.end)
    prev = evs[0].time_range.start
    t0 = prev
    agg = collections.OrderedDict()
    for e in evs:
        name = e.name.split("(")[0].split("<")[0].replace("void ", "")[-44:]
        entry = agg.setdefault(name, [0, 0.0])
        entry[0] += 1
        entry[1] += e.time_range.end - prev
        prev = e.time_range.end
    print(f"decode step, batch {a.batch}, context {a.context}, {a.layers} layers: {prev - t0:.1f} us, {len(evs)} kernels")
    for name, (n, total) in agg.items():
        print(f"  {name:46s} n={n:4d}  adds {total / n:7.2f} us a call  ({total:8.1f} us in all)")


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="microbench")
    sub = p.add_subparsers(dest="what", required=True)
    common = argparse.ArgumentParser(add_help=False)
    common.add_argument("--reps", type=int, default=20)
    common.add_argument("--graph", type=int, default=1, help="1: time a CUDA graph of the calls; 0: plain launches")
    g = sub.add_parser("gemm", parents=[common])
    g.add_argument("--m", type=int, default=8)
    g.add_argument("--n", type=int, default=24576)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--splits", type=int, default=0)
    g.add_argument("--per-sm", type=int, default=2, help="with --splits: CTAs to an SM (2: deep ring, 3: short ring)")
    g.add_argument("--library", type=int, default=1, help="also time the library product")
    g.add_argument("--kernel", default="one", choices=["one", "pair"],
                   help="one: the one-CTA kernel (few rows); pair: the paired kernel (many rows)")
    g.add_argument("--epilogue", default="none", choices=["none", "add_norm", "swiglu"])
    g.add_argument("--normed", type=int, default=0, help="1: x is NormedRows (row factors applied in the epilogue)")
    for name in ("attn-decode", "attn-prefill"):
        s = sub.add_parser(name, parents=[common])
        s.add_argument("--heads", type=int, default=32)
        s.add_argument("--kv-heads", type=int, default=8)
        s.add_argument("--head-dim", type=int, default=128)
        s.add_argument("--page", type=int, default=16)
        s.add_argument("--batch", type=int, default=64)
        s.add_argument("--context", type=int, default=4096)
        s.add_argument("--tokens", type=int, default=2048)
        s.add_argument("--splits", type=int, default=0)
        s.add_argument("--kernel", default="mma", choices=["mma", "tc"], help="prefill: mma.sync or tcgen05 kernel")
    st = sub.add_parser("step", help="per-kernel contributions to one decode step (torch profiler)")
    st.add_argument("--layers", type=int, default=8)
    st.add_argument("--batch", type=int, default=8)
    st.add_argument("--context", type=int, default=4096)
    a = p.parse_args(argv)
    {"gemm": bench_gemm, "attn-decode": bench_attn_decode, "attn-prefill": bench_attn_prefill,
     "step": bench_step}[a.what](a)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
