"""Times single kernels at given sizes with CUDA events: ``python -m glint_b200.bench_kernels``.

Each case rotates through enough copies of its large operands that consecutive launches never
find them in the 126 MB L2; times are medians over the launches after warm-up.  Prints one
line per case with the achieved GB/s (bytes the kernel has to move) and TFLOP/s.
"""
from __future__ import annotations

import argparse
import json
import math

import numpy as np
import torch

DEV = "cuda:0"
L2_BYTES = 126 << 20


def _time(fn, n_variants, iters=20, warmup=5):
    """Median microseconds per launch.  The launches of one round over all variants are captured
    in a CUDA graph, so that the time between the events is device time, not host enqueue time."""
    for i in range(max(warmup, n_variants)):
        fn(i % n_variants)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(n_variants):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(max(3, iters // n_variants + 1)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3 / n_variants)
    times.sort()
    return times[len(times) // 2]


def _copies(nbytes):
    return max(2, int(math.ceil(2.5 * L2_BYTES / max(nbytes, 1))))


def bench_gemm(M, N, K, gated=False, splits=0, iters=20, path=None):
    """A product at the given sizes with the kernel the runtime would take (``path`` names one instead:
    "skinny" or "tcgen05")."""
    from . import ops_tensor
    rows = 2 * N if gated else N
    n = min(_copies(rows * K * 2), 64)
    ws = [torch.randn(rows, K, device=DEV).to(torch.bfloat16) * 0.05 for _ in range(n)]
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16 if gated else torch.float32)
    if gated:
        fn = lambda i: ops_tensor.gemm_gated(x, ws[i], out, "gelu_tanh", force_splits=splits, path=path)
    else:
        fn = lambda i: ops_tensor.gemm(x, ws[i], out, force_splits=splits, path=path)
    us = _time(fn, n, iters)
    nbytes = rows * K * 2 + M * K * 2 + out.numel() * out.element_size()
    flops = 2.0 * M * rows * K
    return {"kernel": ("gemm_gated" if gated else "gemm") + ("_" + path if path else ""), "M": M, "N": N, "K": K, "splits": splits, "us": round(us, 2),
            "GB/s": round(nbytes / us / 1e3, 1), "TFLOP/s": round(flops / us / 1e6, 1)}


def bench_attention_decode(batch, context, nh=8, nkv=4, hd=256, page=16, window=None, cap=50.0, splits=None, iters=20,
                           kernel=None, spread=0.0):
    """Single tokens of ``batch`` requests with ``context`` tokens cached (``spread`` > 0: uniformly between
    (1 - spread) x context and context, seeded).  ``kernel``: "cluster", "stream", or None for the runtime's choice."""
    from . import ops_tensor
    rng = np.random.default_rng(11)
    contexts = [max(1, int(round(context * (1.0 - spread * rng.random())))) for _ in range(batch)]
    pages = [(c + page - 1) // page for c in contexts]
    n_pages = sum(pages)
    keys = [min(c, window) if window else c for c in contexts]
    nbytes = 2 * sum(keys) * nkv * hd * 2
    n = min(_copies(nbytes), 16)
    pools = [(torch.randn(n_pages, nkv, page, hd, device=DEV).to(torch.bfloat16),
              torch.randn(n_pages, nkv, page, hd, device=DEV).to(torch.bfloat16)) for _ in range(n)]
    table = torch.full((batch, max(pages)), -1, dtype=torch.int32)
    at = 0
    for i, p in enumerate(pages):
        table[i, :p] = torch.arange(at, at + p, dtype=torch.int32)
        at += p
    table = table.to(DEV)
    q = torch.randn(batch, nh * hd, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(q)
    pos = torch.tensor([c - 1 for c in contexts], dtype=torch.int32, device=DEV)
    seq = torch.arange(batch, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    share = sum(contexts) / (batch * max(contexts))
    uneven = 0 if share > 0.7 else 1 if share > 0.35 else 2 if share > 0.175 else 3
    if kernel is None:
        kernel = "stream" if ops_tensor.decode_streams(batch, nh, nkv, max(contexts), uneven=uneven) else "cluster"
    res = {"kernel": "attention_decode", "batch": batch, "context": context, "spread": spread}
    if kernel == "stream":
        blocks = 2 * ops_tensor.sm_count()
        plan = ops_tensor.attention_decode_stream_plan(pos, seq, batch, window, page, hd, nkv, blocks)
        partials = torch.empty(ops_tensor.stream_workspace_floats(blocks, nh, nkv, hd), dtype=torch.float32, device=DEV)
        arrive = torch.zeros(batch * nkv, dtype=torch.int32, device=DEV)
        fn = lambda i: ops_tensor.attention_decode_stream(q, pools[i][0], pools[i][1], pos, seq, table, out, nh, nkv,
                                                          hd, page, n_pages, 1 / 16.0, cap, window, status, plan,
                                                          partials, arrive)
        res["blocks"] = blocks
    else:
        sp = splits or ops_tensor.decode_splits(batch, nkv, max(contexts), uneven=uneven)
        fn = lambda i: ops_tensor.attention_decode(q, pools[i][0], pools[i][1], pos, seq, table, out, nh, nkv, hd, page,
                                                   n_pages, 1 / 16.0, cap, window, status, sp)
        res["splits"] = sp
    us = _time(fn, n, iters)
    res.update({"variant": kernel, "us": round(us, 2), "GB/s": round(nbytes / us / 1e3, 1)})
    return res


def bench_attention_prefill(tokens, before=0, nh=8, nkv=4, hd=256, page=16, window=None, cap=50.0, iters=10,
                            kernel="tcgen05"):
    from . import ops_tensor
    total = before + tokens
    n_pages = (total + page - 1) // page
    k = torch.randn(n_pages, nkv, page, hd, device=DEV).to(torch.bfloat16)
    v = torch.randn(n_pages, nkv, page, hd, device=DEV).to(torch.bfloat16)
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(1, n_pages)
    q = torch.randn(tokens, nh * hd, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(q)
    cu = torch.tensor([0, tokens], dtype=torch.int32, device=DEV)
    start = torch.tensor([before], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    run = ops_tensor.attention_tcgen05 if kernel == "tcgen05" else ops_tensor.attention_prefill
    fn = lambda i: run(q, k, v, cu, start, table, out, 1, tokens, nh, nkv, hd, page, n_pages, 1 / 16.0, cap, window,
                       status)
    us = _time(fn, 1, iters)
    keys = sum(min(p + 1, window) if window else p + 1 for p in range(before, total))
    flops = 4.0 * nh * hd * keys
    return {"kernel": "attention_" + kernel, "tokens": tokens, "before": before, "window": window, "us": round(us, 2),
            "TFLOP/s": round(flops / us / 1e6, 1)}


def bench_rows(rows, H=2304, iters=20):
    from . import ops
    x = torch.randn(rows, H, device=DEV)
    y = torch.randn(rows, H, device=DEV)
    w = torch.randn(H, device=DEV)
    out = torch.empty(rows, H, device=DEV, dtype=torch.bfloat16)
    res = []
    us = _time(lambda i: ops.rmsnorm(x, w, out, 1e-6, 1.0), 8, iters)
    res.append({"kernel": "rmsnorm", "rows": rows, "H": H, "us": round(us, 2), "GB/s": round(rows * H * 6 / us / 1e3, 1)})
    us = _time(lambda i: ops.add_rmsnorm(x, y, (w, 1e-6, 1.0), out, (w, 1e-6, 1.0)), 8, iters)
    res.append({"kernel": "add_rmsnorm", "rows": rows, "H": H, "us": round(us, 2),
                "GB/s": round(rows * H * 14 / us / 1e3, 1)})
    return res


def prefill_step(tokens, layers, iters):
    """One prompt portion through an engine of the Gemma-2-2B layer sizes with ``layers`` layers.  The
    last step runs between cudaProfilerStart and cudaProfilerStop, so that a profiler started with
    ``--profile-from-start off`` lists the launches of exactly one step."""
    from . import bench as B
    llm = B.open_llm("2b", layers=layers, cache_tokens=2 * tokens + 256, max_active=2, max_step_tokens=max(tokens, 16))
    ms = B.time_prefill(llm.engine, tokens, iters=iters, warmup=3, seed=30)[0]
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    B.time_prefill(llm.engine, tokens, iters=1, warmup=0, seed=31)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    return {"kernel": "prefill step", "tokens": tokens, "layers": layers, "ms": round(ms, 4)}


def engine_step(shape, layers, batch, context, tokens, timeline=False, spread=0.0):
    """One step of an engine of a named shape with ``layers`` layers: ``batch`` requests with ``context``
    tokens cached (with ``spread`` > 0: uniformly between (1 - spread) x context and context, seeded) bring one
    token each and, with ``tokens`` > 0, one more request brings a portion of that many tokens.  The last step
    runs between cudaProfilerStart and cudaProfilerStop (for a profiler started with ``--profile-from-start off``).  ``timeline``: a step of single tokens is replayed from its CUDA graph
    under the PyTorch profiler and every kernel's start, end and duration in microseconds are printed, which
    shows what runs under what (a launch list shows each kernel alone)."""
    from . import bench as B
    from . import ops
    from .engine.step import StepEntry
    llm = B.open_llm(shape, layers=layers, cache_tokens=(batch + 2) * (context + 64) + 2 * tokens + 64,
                     max_active=batch + 2, max_step_tokens=max(4096, tokens))
    eng = llm.engine
    V = eng.vocab_size
    slots = [eng.open() for _ in range(batch)]
    rng = np.random.default_rng(11)
    contexts = [max(1, int(round(context * (1.0 - spread * rng.random())))) for _ in range(batch)]
    B.fill_cache(eng, slots, [B.random_prompt(c, V, 100 + i) for i, c in enumerate(contexts)])
    out = torch.ones(max(batch, 1), dtype=torch.int32, device=DEV)

    def step():
        entries = [StepEntry(s, [5], [0]) for s in slots]
        if tokens:
            extra = eng.open()
            entries.append(StepEntry(extra, B.random_prompt(tokens, V, 7), [tokens - 1]))
        logits = eng.step(entries)
        ops.argmax(logits, out[:logits.shape[0]]) if logits.shape[0] <= out.shape[0] else None
        if tokens:
            eng.close(extra)

    for _ in range(4):
        step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    step()
    b.record()
    torch.cuda.synchronize()
    res = [{"kernel": "engine step", "shape": shape, "layers": layers, "batch": batch, "context": context,
            "spread": spread, "portion": tokens, "ms": round(a.elapsed_time(b), 4), "graphs": dict(eng.graph_counts)}]
    if timeline:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                     key=lambda e: e.time_range.start)
        t0 = evs[0].time_range.start if evs else 0
        for e in evs:
            res.append({"start_us": round(e.time_range.start - t0, 1), "end_us": round(e.time_range.end - t0, 1),
                        "us": round(e.time_range.end - e.time_range.start, 1), "kernel": e.name[:60]})
    torch.cuda.profiler.start()
    step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    return res


def bench_sampling(rows, V, iters=20):
    """The sampling kernel on random logits: temperature alone, with top-k, and with every stage."""
    from . import ops
    logits = torch.randn(rows, V, device=DEV) * 3
    work = torch.empty(rows, V, device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    f32 = lambda v: torch.full((rows,), v, dtype=torch.float32, device=DEV)
    i32 = lambda v: torch.full((rows,), v, dtype=torch.int32, device=DEV)
    past = torch.arange(0, 2048, dtype=torch.int32, device=DEV).repeat(rows)
    pens = (torch.arange(0, rows + 1, dtype=torch.int32, device=DEV) * 2048, past, torch.ones_like(past), f32(1.1))
    res = []
    for name, k, p, mp, pen in (("temperature", 0, 1.0, 0.0, None), ("top-k 40", 40, 1.0, 0.0, None),
                                ("top-p 0.9", 0, 0.9, 0.0, None), ("top-k, top-p, min-p, penalty", 40, 0.9, 0.02, pens)):
        args = (logits, work, f32(0.8), i32(k), f32(p), f32(mp), f32(0.37), out)
        us = _time(lambda i: ops.sample_rows(*args, penalties=pen), 1, iters)
        res.append({"kernel": "sample_rows", "rows": rows, "V": V, "stages": name, "us": round(us, 2)})
    return res


def gemma2_2b_decode_cases(batch):
    H, I, V, QKV, Q = 2304, 9216, 256000, 4096, 2048
    return [("qkv", batch, QKV, H, False), ("o", batch, H, Q, False), ("gate_up", batch, I, H, True),
            ("down", batch, H, I, False), ("lm_head", batch, V, H, False)]


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("what", choices=["gemm", "gated", "decode-shapes", "prefill-shapes", "attention-decode",
                                     "attention-prefill", "rows", "prefill-step", "sampling", "step"])
    ap.add_argument("--shape", default="2b", help="step: 2b, 9b, 27b or a model folder")
    ap.add_argument("--portion", type=int, default=0, help="step: tokens of a prompt portion beside the single tokens")
    ap.add_argument("--spread", type=float, default=0.0,
                    help="step, attention-decode: contexts uniform between (1 - spread) x context and context "
                         "instead of all equal")
    ap.add_argument("--kernel", default=None, choices=["cluster", "stream"],
                    help="attention-decode: the kernel (default: the runtime's choice)")
    ap.add_argument("--heads", type=int, default=8, help="attention-decode: query heads")
    ap.add_argument("--kv-heads", type=int, default=4, help="attention-decode: kv heads")
    ap.add_argument("--head-dim", type=int, default=256, help="attention-decode: head size")
    ap.add_argument("--timeline", action="store_true", help="step: kernel starts and ends inside a graph replay")
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=2304)
    ap.add_argument("--splits", type=int, default=0, help="attention-decode: blocks per token (default: the runtime's choice)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2176)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--layers", type=int, default=2, help="prefill-step: layers of the engine")
    a = ap.parse_args()
    out = []
    if a.what == "gemm":
        out.append(bench_gemm(a.m, a.n, a.k, False, 0, a.iters))
    elif a.what == "gated":
        out.append(bench_gemm(a.m, a.n, a.k, True, 0, a.iters))
    elif a.what == "decode-shapes":
        for name, M, N, K, gated in gemma2_2b_decode_cases(a.batch):
            out.append(dict(bench_gemm(M, N, K, gated, 0, a.iters), name=name))
        out.append(bench_attention_decode(a.batch, a.context, iters=a.iters))
        out.extend(bench_rows(a.batch))
    elif a.what == "prefill-shapes":
        for name, M, N, K, gated in gemma2_2b_decode_cases(a.tokens)[:4]:
            out.append(dict(bench_gemm(M, N, K, gated, 0, a.iters), name=name))
        out.append(bench_attention_prefill(a.tokens, iters=a.iters))
        out.append(bench_attention_prefill(a.tokens, iters=a.iters, kernel="mma"))
        out.extend(bench_rows(a.tokens))
    elif a.what == "attention-decode":
        out.append(bench_attention_decode(a.batch, a.context, nh=a.heads, nkv=a.kv_heads, hd=a.head_dim, page=a.page,
                                          window=a.window or None, splits=a.splits or None, iters=a.iters,
                                          kernel=a.kernel, spread=a.spread))
    elif a.what == "attention-prefill":
        out.append(bench_attention_prefill(a.tokens, page=a.page, window=a.window or None, iters=a.iters))
    elif a.what == "rows":
        out.extend(bench_rows(a.batch))
    elif a.what == "sampling":
        out.extend(bench_sampling(a.batch, a.n if a.n != 4096 else 256000, a.iters))
    elif a.what == "step":
        out.extend(engine_step(a.shape, a.layers, a.batch, a.context, a.portion, a.timeline, a.spread))
    elif a.what == "prefill-step":
        out.append(prefill_step(a.tokens, a.layers, a.iters))
    for row in out:
        print(json.dumps(row))


if __name__ == "__main__":
    main()
