#!/usr/bin/env python3
"""Headline benchmark: Gemma-2-2B-shaped bfloat16 decode and prefill throughput on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 (device-timed, K decode
steps of the engine's step function with a device argmax); ``e2e`` is the same through the
Python entry point ``LLM.generate`` with host token ids in and out; ``prefill`` is one prompt
of 2,048 tokens; ``roofline`` is the bytes the decode step has to read over its time, against
the measured HBM bandwidth; ``points`` holds decode at batch 1 and 64.  Random weights
N(0, 0.02) seed 2, uniform-random prompts of 2,048 tokens, context limit 8,192.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "Gemma-2-2B bf16 decode tok/s @ batch 8 (prefill tok/s @ 2048 and batch 1/64 alongside)"

PROMPT_LEN = 2048
PREFILL_TOKENS = 2048
BATCH = 8
REPEATS = 5


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines = []
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
            self.lines.append((time.time(), line.strip()))

    def mark(self):
        return time.time()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, spans):
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.lines:
            if not any(a <= t <= b for a, b in spans):
                continue
            parts = [p.strip() for p in line.split(",")]
            try:
                sm.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm():
    print(json.dumps({"impl": "reference",
                      "unavailable": "HamadAndrabi/glint is a Rust crate built by maturin: no Rust toolchain and no "
                                     "maturin in this image, offline pip install fails (No module named 'maturin')"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--skip-points", action="store_true", help="only the headline decode (for profiling)")
    ap.add_argument("--skip-large", action="store_true", help="leave out the 9B serving workload and the 27B decode")
    ap.add_argument("--batch", type=int, default=BATCH)
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from glint_b200 import bench as B

    pk = B.peaks(ROOT)
    full_layers = B.SHAPES["2b"]["num_hidden_layers"]
    max_batch = 64 if not args.skip_points else args.batch
    cache_tokens = max_batch * (PROMPT_LEN + REPEATS * args.steps + args.warmup + 128)
    llm = B.open_llm("2b", layers=args.layers, cache_tokens=cache_tokens, max_active=max_batch, max_step_tokens=4096)
    engine, model = llm.engine, llm.model
    c = model.config
    L = len(model.run_order)
    clocks = ClockSampler()
    clocks.start()
    spans = []

    # ---- before anything is timed: the entry point's tokens against a plain step-by-step run ------------
    check_prompts = [B.random_prompt(PROMPT_LEN, c.vocab_size, 70 + i) for i in range(args.batch)]
    checked = B.check_generate(llm, check_prompts, new_tokens=6)

    # ---- decode at the headline batch, device-timed: REPEATS regions of --steps steps, the median ------------
    t0 = clocks.mark()
    d = B.decode_point(engine, args.batch, PROMPT_LEN, args.steps, args.warmup, seed=10, repeats=REPEATS,
                       hbm_gbs=pk["hbm_gbs"])
    spans.append((t0, clocks.mark()))
    launches = d["launches_per_step"] * args.steps          # this package's kernels in one timed region
    out = {
        "metric": METRIC, "value": round(d["tok_per_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(d["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights N(0,0.02) seed 2, uniform-random token ids",
        "impl": "ours",
        "spread": {"repeats": REPEATS, "ms_per_step_min": round(d["spread_ms"][0], 4),
                   "ms_per_step_max": round(d["spread_ms"][1], 4)},
        "config": {"model": "gemma-2-2b shape", "layers": L, "layers_of_config": full_layers,
                   "hidden": c.hidden_size, "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                   "head_dim": c.head_dim, "intermediate": c.intermediate_size, "vocab": c.vocab_size,
                   "sliding_window": c.sliding_window, "global_batch": args.batch, "seq_len": PROMPT_LEN,
                   "context_limit": c.max_position_embeddings, "page_size": engine.cache.page_size,
                   "parallelism": "single GPU", "l2": "weights 5.2 GB per step exceed the 126 MB L2; no flush",
                   "peaks": pk["source"], "repeats": REPEATS},
        "roofline": {"bound": "hbm", "achieved": round(d["gb_per_s"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(d["frac"], 4), "bytes_per_step": d["bytes_per_step"]},
        "gpu_launches": int(launches),
        "checked": {"what": "tokens of LLM.generate (graphs, launch-ahead) against a plain step-by-step run",
                    "worst_gap_over_scale": round(checked, 5)},
    }

    if not args.skip_points:
        points, detail = {}, {}
        # ---- decode at batch 1 and 64 --------------------------------------------------------------
        for b, key in ((1, "decode_b1"), (64, "decode_b64")):
            t0 = clocks.mark()
            p = B.decode_point(engine, b, PROMPT_LEN, max(16, args.steps // 2), args.warmup, seed=20 + b, repeats=3,
                               hbm_gbs=pk["hbm_gbs"])
            spans.append((t0, clocks.mark()))
            points[key] = round(p["tok_per_s"], 1)
            points[key + "_frac"] = round(p["frac"], 4)
            detail[key] = {"ms_per_step": round(p["ms_per_step"], 4), "bytes_per_step": p["bytes_per_step"],
                           "spread_ms": [round(x, 4) for x in p["spread_ms"]]}
        # ---- prefill of 2,048 tokens ---------------------------------------------------------------
        t0 = clocks.mark()
        pf = B.prefill_point(engine, PREFILL_TOKENS, iters=7, warmup=3, seed=30, pk=pk)
        spans.append((t0, clocks.mark()))
        out["prefill"] = {"value": round(pf["tok_per_s"], 1), "tokens": PREFILL_TOKENS, "ms": round(pf["ms"], 3),
                          "frac": round(pf["frac"], 4), "frac_sustained": round(pf["frac_sustained"], 4),
                          "tflops": round(pf["tflops"], 1), "spread_ms": [round(x, 3) for x in pf["spread_ms"]]}
        # ---- end to end through LLM.generate -------------------------------------------------------
        def end_to_end(batch, seed):
            """--steps full decode steps of ``batch`` requests through the entry point, by the wall clock between
            the ends of the steps (host token ids in, sampled tokens read back every step)."""
            prompts = [B.random_prompt(PROMPT_LEN, c.vocab_size, seed + i) for i in range(batch)]
            llm.generate(prompts, max_tokens=4, stop_at_eos=False)          # warm-up of the whole path
            ahead = batch * PROMPT_LEN // 4096 + 8           # tokens the first request is ahead when the last joins
            t0 = clocks.mark()
            llm.generate(prompts, max_tokens=args.steps + ahead, stop_at_eos=False)
            spans.append((t0, clocks.mark()))
            log = list(llm.scheduler.step_log)
            full = [i for i, s in enumerate(log) if s["prefill_tokens"] == 0 and s["decode_rows"] == batch]
            last = full[-1]
            first = last - args.steps                   # the step before the first of the --steps timed ones
            assert first >= 0 and all(i in full for i in range(first + 1, last + 1)), "too few full decode steps"
            seconds = log[last]["t_end"] - log[first]["t_end"]
            timed = log[first + 1:last + 1]
            return {"value": round(batch * args.steps / seconds, 1), "unit": "tok/s",
                    "h2d_bytes_per_step": int(sum(s["h2d_bytes"] for s in timed) / len(timed)),
                    "d2h_bytes_per_step": int(sum(s["d2h_bytes"] for s in timed) / len(timed)),
                    "steps": len(timed)}

        out["e2e"] = end_to_end(args.batch, 40)
        for b, key in ((1, "e2e_b1"), (64, "e2e_b64")):
            points[key] = end_to_end(b, 200 + b)["value"]
        out["points"] = points
        out["detail"] = detail
        if not args.skip_large:
            del engine, model
            B.release(llm)
            del llm
            large(B, args, pk, clocks, spans, points, detail)
    clocks.stop()
    out["clocks"] = clocks.summary(spans)
    print(json.dumps(out))
    return 0


def large(B, args, pk, clocks, spans, points, detail):
    """The serving workload at the 9B layer sizes (64 requests at t = 0 through the scheduler) and decode at
    the 27B layer sizes (batch 1 and 16, prompts of 4,096 tokens: past the window)."""
    import gc
    import torch
    gc.collect()
    torch.cuda.empty_cache()
    ranges = ((128, 4096), (64, 512))
    llm = B.open_llm("9b", cache_tokens=B.serve_cache_tokens(64, *ranges), max_active=64, max_step_tokens=4096)
    B.serve(llm, 8, (128, 1024), (8, 16), seed=1)                 # warm-up of the path: kernels, buffers, graphs
    t0 = clocks.mark()
    s = B.serve(llm, 64, *ranges, seed=3)
    spans.append((t0, clocks.mark()))
    points["serve_9b"] = round(s["tok_per_s"], 1)
    points["serve_9b_ttft_ms"] = round(s["ttft_ms_mean"], 1)
    points["serve_9b_tpot_ms"] = round(s["tpot_ms_mean"], 2)
    detail["serve_9b"] = {k: (round(v, 3) if isinstance(v, float) else v) for k, v in s.items()}
    detail["serve_9b"]["max_step_tokens"] = 4096
    B.release(llm)
    del llm
    gc.collect()
    torch.cuda.empty_cache()
    llm = B.open_llm("27b", cache_tokens=16 * (4096 + 256), max_active=16, max_step_tokens=4096)
    for b in (1, 16):
        t0 = clocks.mark()
        p = B.decode_point(llm.engine, b, 4096, 24, 4, seed=60 + b, repeats=3, hbm_gbs=pk["hbm_gbs"])
        spans.append((t0, clocks.mark()))
        points[f"decode_27b_b{b}"] = round(p["tok_per_s"], 1)
        points[f"decode_27b_b{b}_frac"] = round(p["frac"], 4)
        detail[f"decode_27b_b{b}"] = {"ms_per_step": round(p["ms_per_step"], 4), "bytes_per_step": p["bytes_per_step"],
                                      "context": p["context"], "layers": len(llm.model.run_order)}
    B.release(llm)


if __name__ == "__main__":
    sys.exit(main())
