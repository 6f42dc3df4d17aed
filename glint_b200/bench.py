"""Throughput measurement shared by ``bench.py`` at the repository root and the ``bench`` verb.

The reference's runner warms up, then times iterations: prefill tok/s = prompt length / prefill
seconds (src/bench/mod.rs:60-107), decode tok/s from the time per token after a prefill
(:110-189), concurrency tok/s with all sessions stepped together (:198-264).  Here every timing
is taken on the device with CUDA events around whole steps of the engine's own step function.
Weights (GBs) are far larger than the 126 MB L2, so no flush is needed between steps.
"""
from __future__ import annotations

import numpy as np
import torch

from .engine.step import StepEntry


def random_prompt(n, vocab, seed):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=n)]


def matmul_params_per_layer(c):
    return ((c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim * c.hidden_size
            + c.hidden_size * c.num_attention_heads * c.head_dim + 3 * c.hidden_size * c.intermediate_size)


def attended(c, layer, pos):
    """Keys a query at ``pos`` reads in ``layer``."""
    w = c.layer_window(layer)
    return pos + 1 if w is None else min(pos + 1, w)


def prefill_flops(c, n_tokens, n_layers, logit_rows=1):
    flops = 2.0 * n_tokens * matmul_params_per_layer(c) * n_layers
    flops += 2.0 * logit_rows * c.vocab_size * c.hidden_size
    for layer in range(n_layers):
        keys = sum(attended(c, layer, p) for p in range(n_tokens))
        flops += 4.0 * c.num_attention_heads * c.head_dim * keys
    return flops


def decode_bytes(model, c, n_layers, contexts, elem_size):
    """Bytes one decode step has to read: every weight it uses once, and the cache of the live
    requests (keys and values of the positions each layer attends)."""
    total = model.parameter_bytes()
    per_key = 2 * c.num_key_value_heads * c.head_dim * elem_size
    for ctx in contexts:
        for layer in range(n_layers):
            total += attended(c, layer, ctx) * per_key
    return total


def fill_cache(engine, slots, prompts, chunk=2048):
    """Prefill each prompt in portions of ``chunk`` tokens, wanting nothing."""
    for slot, toks in zip(slots, prompts):
        for at in range(0, len(toks), chunk):
            engine.step([StepEntry(slot, toks[at:at + chunk], [])])


def time_decode(engine, batch, prompt_len, steps, warmup, seed=0):
    """Device-timed decode: ``batch`` requests with ``prompt_len`` tokens cached each, then
    ``warmup`` + ``steps`` steps of one token per request with a device argmax feeding the next
    step.  Returns (ms per step, contexts at the middle of the timed region)."""
    from . import ops
    vocab = engine.vocab_size
    slots = [engine.open() for _ in range(batch)]
    try:
        fill_cache(engine, slots, [random_prompt(prompt_len, vocab, seed + i) for i in range(batch)])
        out = torch.ones(batch, dtype=torch.int32, device=engine.rt.device)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        placeholder = [StepEntry(s, [0], [0]) for s in slots]

        def one():
            # the sampled tokens stay on the device: no host round trip inside the timed region
            logits = engine.step(placeholder, device_tokens=out)
            ops.argmax(logits, out)

        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            one()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        engine.rt.check_status()
        mid = prompt_len + warmup + steps // 2
        return ms, [mid] * batch
    finally:
        for s in slots:
            engine.close(s)


def time_prefill(engine, n_tokens, iters, warmup, seed=0):
    """Device-timed prefill of one ``n_tokens`` prompt in one step, logits at its last token."""
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
    return float(np.median(times))


def run_cli_bench(args):
    """The ``bench`` verb: prefill, decode and concurrency rows for a model folder."""
    from .engine.loading import build_engine, load_model
    model = load_model(args.file, args.dtype, args.device)
    c = model.config
    levels = [n for n in (1, 2, 4, 8, 16, 32, 64) if n <= args.max_concurrent]
    need = max(levels) * (args.prompt_len + args.decode_tokens + args.warmup + 64)
    engine = build_engine(model, need, num_slots=max(levels))
    rows = []
    if args.mode in ("all", "prefill"):
        ms = time_prefill(engine, args.prompt_len, args.iters, args.warmup)
        rows.append({"mode": "prefill", "tokens": args.prompt_len, "ms": round(ms, 3),
                     "tok_per_s": round(args.prompt_len / ms * 1e3, 1)})
    if args.mode in ("all", "decode"):
        ms, _ = time_decode(engine, 1, args.prompt_len, args.decode_tokens, args.warmup)
        rows.append({"mode": "decode", "batch": 1, "ms_per_token": round(ms, 3), "tok_per_s": round(1e3 / ms, 1)})
    if args.mode in ("all", "concurrency"):
        for n in levels:
            ms, _ = time_decode(engine, n, args.prompt_len, args.decode_tokens, args.warmup)
            rows.append({"mode": "concurrency", "batch": n, "ms_per_step": round(ms, 3),
                         "tok_per_s": round(n * 1e3 / ms, 1)})
    return {"model": args.file, "dtype": args.dtype, "rows": rows, "model_info": c.model_info()}
