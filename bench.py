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

GEMMA2_2B = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 26, "hidden_size": 2304, "num_attention_heads": 8, "num_key_value_heads": 4,
    "head_dim": 256, "intermediate_size": 9216, "vocab_size": 256000, "rope_theta": 10000.0,
    "sliding_window": 4096, "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0,
    "query_pre_attn_scalar": 256, "rms_norm_eps": 1e-6, "max_position_embeddings": 8192,
    "tie_word_embeddings": True, "hidden_activation": "gelu_pytorch_tanh",
}
PROMPT_LEN = 2048
PREFILL_TOKENS = 2048
BATCH = 8


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


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
    ap.add_argument("--skip-points", action="store_true", help="skip batch 1 and 64, prefill and e2e (for profiling)")
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
    from glint_b200 import ops
    from glint_b200.config import config_from_dict
    from glint_b200.engine.api import LLM

    pk = peaks()
    cfg = dict(GEMMA2_2B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    c = config_from_dict(cfg)
    L = c.num_hidden_layers
    max_batch = 64 if not args.skip_points else args.batch
    cache_tokens = max_batch * (PROMPT_LEN + args.steps + args.warmup + 64)
    llm = LLM.from_config(c, seed=2, std=0.02, norm_std=0.02, dtype="bfloat16", cache_tokens=cache_tokens,
                          max_active=max_batch, max_step_tokens=4096)
    engine, model = llm.engine, llm.model
    clocks = ClockSampler()
    clocks.start()
    spans = []

    # ---- decode at the headline batch, device-timed ------------------------------------------------
    launches0 = ops.launch_count
    t0 = clocks.mark()
    ms, contexts = B.time_decode(engine, args.batch, PROMPT_LEN, args.steps, args.warmup, seed=10)
    spans.append((t0, clocks.mark()))
    launches = (ops.launch_count - launches0) * args.steps // (args.steps + args.warmup + 1)
    launches = getattr(engine, "timed_launches", None) or launches
    value = args.batch * 1e3 / ms
    step_bytes = B.decode_bytes(model, c, L, contexts, 2)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    out = {
        "metric": METRIC, "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights N(0,0.02) seed 2, uniform-random token ids",
        "impl": "ours",
        "config": {"model": "gemma-2-2b shape", "layers": L, "layers_of_config": full_layers,
                   "hidden": c.hidden_size, "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                   "head_dim": c.head_dim, "intermediate": c.intermediate_size, "vocab": c.vocab_size,
                   "sliding_window": c.sliding_window, "global_batch": args.batch, "seq_len": PROMPT_LEN,
                   "context_limit": c.max_position_embeddings, "page_size": engine.cache.page_size,
                   "parallelism": "single GPU", "l2": "weights 5.2 GB per step exceed the 126 MB L2; no flush",
                   "peaks": pk["source"]},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "gpu_launches": int(launches),
    }

    if not args.skip_points:
        # ---- decode at batch 1 and 64 --------------------------------------------------------------
        points = {}
        for b, key in ((1, "decode_b1"), (64, "decode_b64")):
            t0 = clocks.mark()
            ms_b, _ = B.time_decode(engine, b, PROMPT_LEN, max(16, args.steps // 2), args.warmup, seed=20 + b)
            spans.append((t0, clocks.mark()))
            points[key] = round(b * 1e3 / ms_b, 1)
        out["points"] = points
        # ---- prefill of 2,048 tokens ---------------------------------------------------------------
        t0 = clocks.mark()
        pms = B.time_prefill(engine, PREFILL_TOKENS, iters=5, warmup=3, seed=30)
        spans.append((t0, clocks.mark()))
        flops = B.prefill_flops(c, PREFILL_TOKENS, L)
        out["prefill"] = {"value": round(PREFILL_TOKENS / pms * 1e3, 1), "tokens": PREFILL_TOKENS,
                          "ms": round(pms, 3), "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                          "tflops": round(flops / (pms * 1e-3) / 1e12, 1)}
        # ---- end to end through LLM.generate -------------------------------------------------------
        prompts = [B.random_prompt(PROMPT_LEN, c.vocab_size, 40 + i) for i in range(args.batch)]
        llm.generate(prompts, max_tokens=4, stop_at_eos=False)          # warm-up of the whole path
        t0 = clocks.mark()
        llm.generate(prompts, max_tokens=args.steps + 1, stop_at_eos=False)
        spans.append((t0, clocks.mark()))
        log = [s for s in llm.scheduler.step_log if s["prefill_tokens"] == 0 and s["decode_rows"] == args.batch]
        log = log[-args.steps:]
        e2e_s = sum(s["seconds"] for s in log)
        out["e2e"] = {"value": round(sum(s["decode_rows"] for s in log) / e2e_s, 1), "unit": "tok/s",
                      "h2d_bytes_per_step": int(sum(s["h2d_bytes"] for s in log) / len(log)),
                      "d2h_bytes_per_step": int(sum(s["d2h_bytes"] for s in log) / len(log)),
                      "steps": len(log)}
    clocks.stop()
    out["clocks"] = clocks.summary(spans)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
