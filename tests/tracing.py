"""Builds replay traces (lists of steps in bin/trace_run's JSON form) and runs them, either
through ``bin/trace_run`` as a child process or through the same engine calls in-process."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np

from tests.helpers import ROOT


def whole(requests):
    """Each request alone and whole, one step each, logits wanted everywhere."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail_decode(requests, tail=32):
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def chunked(requests, sizes=(7, 2, 16, 3, 2, 33, 5, 1, 17, 2)):
    """Portions of changing size, down to two tokens (and single ones)."""
    steps = []
    for rid, toks in requests.items():
        at, k = 0, 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            steps.append({"step": len(steps),
                          "entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}],
                          "end": [rid] if at + n == len(toks) else []})
            at += n
    return steps


def mixed(requests, seed=0, max_live=4, decode_tail=12, max_chunk=19):
    """Up to ``max_live`` live requests; each step holds portions of some beside single tokens
    of others; a request sometimes sits a step out.  The last ``decode_tail`` tokens of every
    request go one by one."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live = {}   # rid -> position
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, end = [], []
        for rid in list(live):
            toks = requests[rid]
            at = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue  # sits this step out
            left = len(toks) - at
            if left <= decode_tail:
                n = 1
            else:
                n = int(min(left - decode_tail, rng.integers(2, max_chunk + 1)))
            entries.append({"id": rid, "tokens": toks[at:at + n], "want": list(range(n))})
            live[rid] = at + n
            if at + n == len(toks):
                end.append(rid)
                del live[rid]
        if not entries:
            continue
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def max_live_tokens(steps, round_to=64):
    """The --max-tokens a trace needs: the most tokens live requests hold at any time, each
    request's count rounded up to a multiple of ``round_to``."""
    held, most = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(-(-h // round_to) * round_to for h in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return most


def collect(steps, outputs, vocab):
    """Per request, logits [tokens, vocab] in position order from per-step outputs
    (``outputs[step]`` is a float32 array [wanted, vocab] or ``None``)."""
    got = {}
    for s in steps:
        out = outputs.get(s["step"])
        row = 0
        for e in s["entries"]:
            for _ in e["want"]:
                got.setdefault(e["id"], []).append(out[row])
                row += 1
        assert out is None or row == out.shape[0]
    return {rid: np.stack(rows) for rid, rows in got.items()}


def run_in_process(engine, steps):
    """The same calls bin/trace_run makes, on an engine in this process."""
    from glint_b200.engine.step import StepEntry
    slots, outputs = {}, {}
    for s in steps:
        entries = []
        for e in s["entries"]:
            if e["id"] not in slots:
                slots[e["id"]] = engine.open()
            entries.append(StepEntry(slots[e["id"]], list(e["tokens"]), list(e["want"])))
        logits = engine.step(entries)
        if logits is not None:
            outputs[s["step"]] = logits.float().cpu().numpy()
        engine.rt.check_status()
        for rid in s["end"]:
            engine.close(slots.pop(rid))
        engine.cache.check_consistency()
    return outputs


def run_child(model_dir, dtype, steps, out_dir, max_tokens, vocab, extra_args=(), env=None, timeout=900):
    """Run ``bin/trace_run`` with the trace on its standard input; returns per-step outputs."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)] + list(extra_args)
    text = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout, env=env)
    assert p.returncode == 0, f"trace_run failed ({p.returncode}):\n{p.stdout[-2000:]}\n{p.stderr[-4000:]}"
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps]
    outputs = {}
    for s in steps:
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if any(e["want"] for e in s["entries"]):
            outputs[s["step"]] = np.fromfile(path, dtype="<f4").reshape(-1, vocab)
    return outputs
