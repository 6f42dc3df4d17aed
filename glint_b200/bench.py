"""Throughput measurement shared by ``bench.py`` at the repository root and the ``bench`` verb.

The reference's runner warms up, then times iterations: prefill tok/s = prompt length / prefill
seconds (src/bench/mod.rs:60-107), decode tok/s from the time per token after a prefill
(:110-189), concurrency tok/s = sequences x decoded tokens / elapsed with all sessions stepped
together (:198-264).  Here every kernel timing is taken on the device with CUDA events around
whole steps of the engine's own step function, and the serving workload runs through the
scheduler (the reference's engine loop, src/server/engine.rs:449-671).  Weights (GBs) are far
larger than the 126 MB L2, so no flush is needed between steps.

Rooflines come from the model itself: every part answers for the bytes it reads and the
operations it performs (``CausalLM.decode_read_bytes``, ``CausalLM.flops``), so nothing here knows
an architecture.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np
import torch

from .engine.step import StepEntry

# Layer sizes of the published Gemma 2 checkpoints, as config.json content (random weights are made
# for them on the device; nothing is downloaded).
_COMMON = {"architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "vocab_size": 256000, "rope_theta": 10000.0,
           "sliding_window": 4096, "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0,
           "rms_norm_eps": 1e-6, "max_position_embeddings": 8192, "tie_word_embeddings": True,
           "hidden_activation": "gelu_pytorch_tanh"}
SHAPES = {
    "2b": dict(_COMMON, num_hidden_layers=26, hidden_size=2304, num_attention_heads=8, num_key_value_heads=4,
               head_dim=256, intermediate_size=9216, query_pre_attn_scalar=256),
    "9b": dict(_COMMON, num_hidden_layers=42, hidden_size=3584, num_attention_heads=16, num_key_value_heads=8,
               head_dim=256, intermediate_size=14336, query_pre_attn_scalar=256),
    "27b": dict(_COMMON, num_hidden_layers=46, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16,
                head_dim=128, intermediate_size=36864, query_pre_attn_scalar=144),
}
SHAPE_SEEDS = {"2b": 2, "9b": 3, "27b": 4}


def peaks(root=None):
    """Measured peaks of this machine (``MEASURED_PEAKS.json`` beside the package, written by whoever
    measured them), else the figures of an earlier measurement on the same kind of GPU."""
    root = root or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def shape_config(shape, layers=None, context=None):
    """config.json content of a named shape, optionally with fewer layers and another context limit."""
    if shape not in SHAPES:
        raise ValueError(f"unknown shape '{shape}' (known: {', '.join(SHAPES)}, or a model folder)")
    cfg = dict(SHAPES[shape])
    if layers:
        cfg["num_hidden_layers"] = int(layers)
    if context:
        cfg["max_position_embeddings"] = int(context)
    return cfg


def open_llm(shape, dtype="bfloat16", device="cuda:0", layers=None, context=None, **kw):
    """An ``LLM`` for a named shape (random weights N(0, 0.02) made on the device with the shape's
    seed) or for a model folder."""
    from .engine.api import LLM
    if shape in SHAPES:
        return LLM.from_config(shape_config(shape, layers, context), seed=SHAPE_SEEDS[shape], std=0.02, norm_std=0.02,
                               dtype=dtype, device=device, **kw)
    if layers or context:
        raise ValueError("--layers and --context apply to named shapes, not to a model folder")
    return LLM(shape, dtype=dtype, device=device, **kw)


def random_prompt(n, vocab, seed):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=n)]


def element_size(model):
    return torch.empty((), dtype=model.rt.dtype).element_size()


def fill_cache(engine, slots, prompts, chunk=2048):
    """Prefill each prompt in portions of ``chunk`` tokens, wanting nothing."""
    for slot, toks in zip(slots, prompts):
        for at in range(0, len(toks), chunk):
            engine.step([StepEntry(slot, toks[at:at + chunk], [])])


def time_decode(engine, batch, prompt_len, steps, warmup, seed=0, repeats=1):
    """Device-timed decode: ``batch`` requests with ``prompt_len`` tokens cached each, then ``warmup``
    steps and ``repeats`` timed regions of ``steps`` steps of one token per request, a device argmax
    feeding the next step.  Returns a dictionary: ``ms`` per step (median over the regions), ``spread``
    (fastest and slowest region), ``positions`` of the tokens at the middle of the median region,
    ``launches_per_step`` (kernels of this package launched per timed step, replayed ones included)."""
    from . import ops
    vocab = engine.vocab_size
    slots = [engine.open() for _ in range(batch)]
    try:
        fill_cache(engine, slots, [random_prompt(prompt_len, vocab, seed + i) for i in range(batch)])
        out = torch.ones(batch, dtype=torch.int32, device=engine.rt.device)
        placeholder = [StepEntry(s, [0], [0]) for s in slots]

        def one():
            # the sampled tokens stay on the device: no host round trip inside the timed region
            logits = engine.step(placeholder, device_tokens=out)
            ops.argmax(logits, out)

        for _ in range(warmup):
            one()
        regions = []
        launches = ops.launches()
        for r in range(repeats):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(steps):
                one()
            stop.record()
            torch.cuda.synchronize()
            regions.append((start.elapsed_time(stop) / steps, prompt_len + warmup + r * steps + steps // 2))
        launches = (ops.launches() - launches) / (repeats * steps)
        engine.rt.check_status()
        order = sorted(regions)
        ms, mid = order[len(order) // 2]
        return {"ms": ms, "spread": [order[0][0], order[-1][0]], "positions": [mid] * batch,
                "launches_per_step": launches}
    finally:
        for s in slots:
            engine.close(s)


def decode_point(engine, batch, prompt_len, steps, warmup, seed=0, repeats=1, hbm_gbs=None):
    """``time_decode`` with its roofline: tokens a second, and the bytes the step has to read (every
    weight it uses once, and what the live requests' mixers read of the cache) over its time."""
    t = time_decode(engine, batch, prompt_len, steps, warmup, seed, repeats)
    model = engine.model
    step_bytes = model.decode_read_bytes(t["positions"], element_size(model))
    gbs = step_bytes / (t["ms"] * 1e-3) / 1e9
    hbm = hbm_gbs or peaks()["hbm_gbs"]
    return {"batch": batch, "context": t["positions"][0], "tok_per_s": batch * 1e3 / t["ms"], "ms_per_step": t["ms"],
            "spread_ms": t["spread"], "bytes_per_step": int(step_bytes), "gb_per_s": gbs, "frac": gbs / hbm,
            "launches_per_step": t["launches_per_step"]}


def time_prefill(engine, n_tokens, iters, warmup, seed=0):
    """Device-timed prefill of one ``n_tokens`` prompt in one step, logits at its last token.  Returns
    (median ms, fastest ms, slowest ms)."""
    vocab = engine.vocab_size
    toks = random_prompt(n_tokens, vocab, seed)
    times = []
    for i in range(warmup + iters):
        slot = engine.open()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([StepEntry(slot, toks, [n_tokens - 1])])
        stop.record()
        torch.cuda.synchronize()
        engine.close(slot)
        if i >= warmup:
            times.append(start.elapsed_time(stop))
    engine.rt.check_status()
    return float(np.median(times)), float(min(times)), float(max(times))


def prefill_point(engine, n_tokens, iters, warmup, seed=0, pk=None):
    """``time_prefill`` with its roofline: the step's operations over its time, against the peak of a
    matrix product measured as a burst and as a seconds-long loop under the power cap."""
    pk = pk or peaks()
    ms, lo, hi = time_prefill(engine, n_tokens, iters, warmup, seed)
    flops = engine.model.flops([(0, n_tokens)], 1)
    tf = flops / (ms * 1e-3) / 1e12
    return {"tokens": n_tokens, "tok_per_s": n_tokens / ms * 1e3, "ms": ms, "spread_ms": [lo, hi], "tflops": tf,
            "frac": tf / pk["bf16_tflops"], "frac_sustained": tf / pk["bf16_tflops_sustained"]}


def check_generate(llm, prompts, new_tokens=6, margin_fraction=0.025):
    """Before anything is timed: the entry point's path (CUDA graphs, the next step launched ahead, the
    scheduler) must choose, at every step, a token whose logit in a plain step-by-step run of the same
    model (no graphs, one request at a time) is the largest within the bfloat16 rounding of a logit
    (``margin_fraction`` of the largest magnitude).  Raises ``AssertionError`` otherwise, so that a fast
    wrong run cannot print a number."""
    from .engine.loading import build_engine
    got = llm.generate(prompts, max_tokens=new_tokens, stop_at_eos=False)
    room = max(len(p) for p in prompts) + new_tokens + 64
    plain_engine = build_engine(llm.model, room, num_slots=1, page_size=llm.engine.cache.page_size, use_graphs=False)
    worst = 0.0
    for p, out in zip(prompts, got):
        assert len(out) == new_tokens, f"generate returned {len(out)} tokens instead of {new_tokens}"
        slot = plain_engine.open()
        fill_cache(plain_engine, [slot], [p[:-1]]) if len(p) > 1 else None
        feed = p[-1]
        for t in out:
            logits = plain_engine.step([StepEntry(slot, [feed], [0])])[0].float()
            top = float(logits.max())
            scale = float(logits.abs().max())
            gap = top - float(logits[t])
            worst = max(worst, gap / max(scale, 1e-9))
            assert gap <= margin_fraction * scale, (
                f"the entry point chose token {t} whose logit lies {gap:.4f} below the largest ({top:.4f}) "
                f"of a plain step-by-step run")
            feed = t
        plain_engine.close(slot)
    llm.model.rt.check_status()
    del plain_engine
    return worst


def serve(llm, n_requests=64, prompt_range=(128, 4096), output_range=(64, 512), seed=0, temperature=0.0):
    """The continuous-batching workload: ``n_requests`` requests, all queued at t = 0, prompts of
    uniform-random ids with lengths uniform in ``prompt_range`` and output lengths uniform in
    ``output_range`` (seeded), run through the scheduler to the end.  Total tok/s is generated tokens
    over the wall time from the first step to the last token (the reference's concurrency figure,
    src/bench/mod.rs:198-251); TTFT is the time until a request's first token reached the host, TPOT
    the time per token after it.  Steps are counted by kind (only single tokens / prompt portions beside
    them / only portions) with the host's time in the step call against the device's time between the
    step boundaries (CUDA events)."""
    from .engine.scheduler import Request
    from .sampling import SamplingParams
    sch = llm.scheduler
    vocab = llm.model.spec.vocab_size
    rng = np.random.default_rng(seed)
    p_lens = rng.integers(prompt_range[0], prompt_range[1] + 1, size=n_requests)
    o_lens = rng.integers(output_range[0], output_range[1] + 1, size=n_requests)
    requests = []
    for i in range(n_requests):
        params = SamplingParams(temperature=temperature, seed=seed + i)
        requests.append(Request(("serve", i), random_prompt(int(p_lens[i]), vocab, seed * 1000 + i), int(o_lens[i]),
                                params, None))
    torch.cuda.synchronize()
    sch.step_log.clear()
    events = [torch.cuda.Event(enable_timing=True)]
    t0 = time.perf_counter()
    for r in requests:
        sch.add(r)
    events[0].record()
    while not sch.idle:
        n_log = len(sch.step_log)
        sch.step()
        if len(sch.step_log) > n_log:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            events.append(ev)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    llm.model.rt.check_status()
    log = list(sch.step_log)[-(len(events) - 1):]
    kinds = {}
    for i, s in enumerate(log):
        kind = "decode" if s["prefill_tokens"] == 0 else ("mixed" if s["decode_rows"] else "prefill")
        k = kinds.setdefault(kind, {"steps": 0, "host_s": 0.0, "device_s": 0.0, "tokens": 0})
        k["steps"] += 1
        k["host_s"] += s["seconds"]
        k["device_s"] += events[i].elapsed_time(events[i + 1]) * 1e-3
        k["tokens"] += s["prefill_tokens"] + s["decode_rows"]
    for k in kinds.values():
        k["host_s"], k["device_s"] = round(k["host_s"], 4), round(k["device_s"], 4)
    generated = sum(len(r.output) for r in requests)
    assert all(len(r.output) == int(n) for r, n in zip(requests, o_lens)), "a request ended early"
    ttft = np.array([r.t_first - t0 for r in requests])
    tpot = np.array([(r.t_finish - r.t_first) / max(len(r.output) - 1, 1) for r in requests])
    last = max(r.t_finish for r in requests)
    return {"requests": n_requests, "prompt_tokens": int(p_lens.sum()), "generated_tokens": int(generated),
            "seconds": last - t0, "tok_per_s": generated / (last - t0),
            "total_tok_per_s": (generated + int(p_lens.sum())) / (last - t0),
            "ttft_ms_mean": float(ttft.mean() * 1e3), "ttft_ms_p95": float(np.percentile(ttft, 95) * 1e3),
            "tpot_ms_mean": float(tpot.mean() * 1e3), "tpot_ms_p95": float(np.percentile(tpot, 95) * 1e3),
            "steps": kinds, "preemptions": sch.counters["preemptions"], "wall_s": t1 - t0}


def serve_cache_tokens(n_requests, prompt_range, output_range):
    """Room for every request of the workload at its longest, rounded up to pages."""
    return n_requests * (prompt_range[1] + output_range[1] + 64)


def release(llm):
    """Give the device memory of a model and its engine back (the next shape needs it)."""
    llm.engine._graphs.clear()
    llm.engine._graph_pool = None
    import gc
    gc.collect()
    torch.cuda.empty_cache()


# ---- the ``bench`` verb ------------------------------------------------------------------------------------


def run_cli_bench(args):
    """Rows of tok/s with their roofline fraction for a named shape or a model folder: ``prefill``,
    ``decode`` at each batch size, ``serve`` (the continuous-batching workload)."""
    pk = peaks()
    shape = args.shape or args.file
    if not shape:
        raise ValueError("bench needs --shape 2b|9b|27b|<folder> (or -f <folder>)")
    if args.batch:
        batches = [int(b) for b in str(args.batch).replace(",", " ").split()]
    else:
        batches = [n for n in (1, 2, 4, 8, 16, 32, 64) if n <= args.max_concurrent]
    modes = ("prefill", "decode", "serve") if args.mode == "all" else (("decode",) if args.mode == "concurrency" else (args.mode,))
    if shape in SHAPES:
        context = shape_config(shape, args.layers, args.context)["max_position_embeddings"]
    else:
        from .config import load_config
        context = load_config(shape).model_spec().max_positions
    # the workload's lengths, cut down for a model with a short context
    serve_ranges = ((min(128, max(1, context // 8)), min(4096, context // 2)), (min(64, max(1, context // 16)), min(512, context // 4)))
    if args.prompt_len + args.decode_tokens + args.warmup + 1 > context:
        raise ValueError(f"--prompt-len {args.prompt_len} and --decode-tokens {args.decode_tokens} exceed the model's "
                         f"context of {context} tokens")
    need = max(batches) * (args.prompt_len + args.decode_tokens + args.warmup + 64) if ("decode" in modes or "prefill" in modes) else 0
    if "serve" in modes:
        need = max(need, serve_cache_tokens(args.requests, *serve_ranges))
    need = max(need, args.prompt_len + 64)
    llm = open_llm(shape, args.dtype, args.device, args.layers, args.context, cache_tokens=need,
                   max_active=max(max(batches), args.requests if "serve" in modes else 1),
                   max_step_tokens=max(2048, min(args.prompt_len, 8192)))
    engine, model = llm.engine, llm.model
    rows = []
    if "prefill" in modes:
        p = prefill_point(engine, args.prompt_len, args.iters, args.warmup, pk=pk)
        rows.append({"mode": "prefill", "tokens": args.prompt_len, "ms": round(p["ms"], 3), "tok_per_s": round(p["tok_per_s"], 1),
                     "tflops": round(p["tflops"], 1), "frac_of_bf16_peak": round(p["frac"], 4)})
    if "decode" in modes:
        for b in batches:
            d = decode_point(engine, b, args.prompt_len, args.decode_tokens, args.warmup, hbm_gbs=pk["hbm_gbs"])
            rows.append({"mode": "decode", "batch": b, "context": d["context"], "ms_per_step": round(d["ms_per_step"], 4),
                         "tok_per_s": round(d["tok_per_s"], 1), "gb_per_s": round(d["gb_per_s"], 1),
                         "frac_of_hbm_peak": round(d["frac"], 4)})
    if "serve" in modes:
        s = serve(llm, args.requests, *serve_ranges, seed=3)
        rows.append({"mode": "serve", "requests": s["requests"], "generated_tokens": s["generated_tokens"],
                     "tok_per_s": round(s["tok_per_s"], 1), "ttft_ms_mean": round(s["ttft_ms_mean"], 1),
                     "ttft_ms_p95": round(s["ttft_ms_p95"], 1), "tpot_ms_mean": round(s["tpot_ms_mean"], 2),
                     "tpot_ms_p95": round(s["tpot_ms_p95"], 2), "steps": s["steps"]})
    return {"model": shape, "dtype": args.dtype, "layers": len(model.run_order), "peaks": pk, "rows": rows,
            "model_info": model.spec.info}
