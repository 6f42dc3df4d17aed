"""Generation through the entry points against the plain implementation: greedy tokens, long
decoding, the first tokens of a sequence, seeded sampling, a cache too small for everybody, and
the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import tracing
from tests.helpers import ROOT, TINY, make_model_dir, plain_logits, random_tokens, tolerance
from tests.plain import model as plain
from tests.plain import sampler as psampler

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen")
    return {name: make_model_dir(root, name) for name in TINY}


def _plain_greedy(folder, prompt, n):
    c, w = plain.read_config(folder), plain.read_weights(folder)
    toks, margins = list(prompt), []
    for _ in range(n):
        logits = plain.forward(c, w, toks)[-1]
        top = torch.topk(logits, 2).values
        margins.append(float(top[0] - top[1]))
        toks.append(int(torch.argmax(logits)))
    return toks[len(prompt):], margins


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_float32_equals_plain(folders, name):
    from glint_b200 import LLM
    vocab = TINY[name][0]["vocab_size"]
    lengths = [5, 23, 40] if name == "A" else [1, 9, 31]
    prompts = [random_tokens(n, vocab, 50 + i) for i, n in enumerate(lengths)]
    llm = LLM(folders[name], dtype="float32", cache_tokens=512, max_active=4, max_step_tokens=32)
    got = llm.generate(prompts, max_tokens=16, stop_at_eos=False)
    for p, g in zip(prompts, got):
        want, margins = _plain_greedy(folders[name], p, 16)
        for i, (a, b) in enumerate(zip(g, want)):
            if a != b:
                assert margins[i] < 1e-4, (name, len(p), i, g, want)     # a tie within float32 rounding
                break
    single = llm.generate(prompts[1], max_tokens=16, stop_at_eos=False)
    assert single == got[1]                                              # alone == in a batch
    assert llm.model_info()["architecture"] == "gemma2" and llm.model_info()["vocab_size"] == vocab
    assert all(s["live"] == 0 for s in llm.cache_stats().values())


def test_greedy_generation_bfloat16_follows_plain(folders):
    from glint_b200 import LLM
    vocab = TINY["B"][0]["vocab_size"]
    prompt = random_tokens(31, vocab, 77)
    llm = LLM(folders["B"], dtype="bfloat16", cache_tokens=256, max_active=2)
    got = llm.generate(prompt, max_tokens=12, stop_at_eos=False)
    want, margins = _plain_greedy(folders["B"], prompt, 12)
    for i, (a, b) in enumerate(zip(got, want)):
        if a != b:
            assert margins[i] < 0.1, (i, got, want, margins)   # the top two were within bfloat16 rounding
            break


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(folders, dtype):
    """From the very first token, one token per step for 300 steps, past several windows and pages."""
    from glint_b200.engine.loading import build_engine, load_model
    vocab = TINY["C"][0]["vocab_size"]
    toks = random_tokens(300, vocab, 5)
    steps = [{"step": i, "entries": [{"id": "r", "tokens": [t], "want": [0]}], "end": ["r"] if i == 299 else []}
             for i, t in enumerate(toks)]
    engine = build_engine(load_model(folders["C"], dtype), 320, num_slots=2)
    out = tracing.run_in_process(engine, steps)
    got = tracing.collect(steps, out, vocab)["r"]
    want = plain_logits(folders["C"], toks)
    diff = np.abs(got - want).max(axis=1)
    tol = tolerance(dtype, want)
    assert diff[:3].max() <= tol, diff[:3]                               # the first tokens of a sequence
    assert diff.max() <= tol, (int(np.argmax(diff > tol)), diff.max())


def test_temperature_sampling_is_seeded_and_follows_the_plain_sampler(folders):
    from glint_b200 import LLM
    vocab = TINY["B"][0]["vocab_size"]
    prompts = [random_tokens(n, vocab, 90 + i) for i, n in enumerate([1, 9, 31, 77])]
    llm = LLM(folders["B"], dtype="float32", cache_tokens=1024, max_active=4, max_step_tokens=24)
    a = llm.generate(prompts, max_tokens=24, temperature=0.8, seed=7, stop_at_eos=False)
    b = llm.generate(prompts, max_tokens=24, temperature=0.8, seed=7, stop_at_eos=False)
    c = llm.generate(prompts, max_tokens=24, temperature=0.8, seed=8, stop_at_eos=False)
    assert a == b and a != c and all(len(x) == 24 for x in a)
    # the same draws from the plain sampler on the plain logits, request 1 (seed 7 + 1)
    cfg, w = plain.read_config(folders["B"]), plain.read_weights(folders["B"])
    rng = psampler.Xorshift64(8)
    toks = list(prompts[1])
    agree = 0
    for i in range(24):
        logits = plain.forward(cfg, w, toks)[-1].numpy()
        t = psampler.sample(logits, toks, rng, temperature=0.8)
        if t != a[1][i]:
            break
        agree += 1
        toks.append(t)
    assert agree >= 20, (agree, a[1])      # a draw within rounding of a boundary may differ late


def test_all_sampling_options_with_and_without_lookahead(folders):
    """top-k, top-p, min-p and the repeat penalty through the entry point: the tokens do not depend on
    whether the next step is launched before the last tokens reach the host, and they are the plain
    sampler's on the plain logits (the penalty counts every token so far, the newest one included)."""
    from glint_b200 import LLM
    vocab = TINY["B"][0]["vocab_size"]
    prompts = [random_tokens(n, vocab, 50 + i) for i, n in enumerate([5, 40, 17])]
    opts = dict(temperature=0.9, top_k=12, top_p=0.92, min_p=0.01, repeat_penalty=1.3)
    outs = []
    for lookahead in (True, False):
        llm = LLM(folders["B"], dtype="float32", cache_tokens=1024, max_active=4, max_step_tokens=32, lookahead=lookahead)
        outs.append(llm.generate(prompts, max_tokens=20, seed=3, stop_at_eos=False, **opts))
    assert outs[0] == outs[1]
    cfg, w = plain.read_config(folders["B"]), plain.read_weights(folders["B"])
    rng = psampler.Xorshift64(3 + 2)                                       # request 2
    toks = list(prompts[2])
    agree = 0
    for i in range(20):
        logits = plain.forward(cfg, w, toks)[-1].numpy()
        t = psampler.sample(logits, toks, rng, **opts)
        if t != outs[0][2][i]:
            break
        agree += 1
        toks.append(t)
    assert agree >= 16, (agree, outs[0][2])


def test_sampling_over_a_wide_vocabulary_follows_the_plain_sampler(tmp_path):
    """A vocabulary of 20011 entries takes the sampling kernel that shares a row among the blocks of a
    cluster; with top-k the distribution is peaked enough for the plain sampler to agree token by token."""
    from glint_b200 import LLM
    from glint_b200.weights import write_random_model
    cfg = dict(TINY["A"][0], vocab_size=20011)
    folder = os.path.join(str(tmp_path), "wide_vocab")
    write_random_model(dict(cfg), folder, seed=4, std=0.05, norm_std=0.1)
    prompts = [random_tokens(n, cfg["vocab_size"], 70 + i) for i, n in enumerate([12, 3])]
    opts = dict(temperature=0.9, top_k=6, top_p=0.95, repeat_penalty=1.2)
    llm = LLM(folder, dtype="float32", cache_tokens=512, max_active=2)
    got = llm.generate(prompts, max_tokens=16, seed=9, stop_at_eos=False, **opts)
    assert got == llm.generate(prompts, max_tokens=16, seed=9, stop_at_eos=False, **opts)
    pcfg, w = plain.read_config(folder), plain.read_weights(folder)
    for r, prompt in enumerate(prompts):
        rng = psampler.Xorshift64(9 + r)
        toks = list(prompt)
        agree = 0
        for i in range(16):
            t = psampler.sample(plain.forward(pcfg, w, toks)[-1].numpy(), toks, rng, **opts)
            if t != got[r][i]:
                break
            agree += 1
            toks.append(t)
        assert agree >= 14, (r, agree, got[r])


def test_small_cache_preempts_and_still_gives_the_same_tokens(folders):
    from glint_b200 import LLM
    vocab = TINY["A"][0]["vocab_size"]
    prompts = [random_tokens(n, vocab, 30 + i) for i, n in enumerate([30, 28, 35, 20])]
    roomy = LLM(folders["A"], dtype="float32", cache_tokens=1024, max_active=4)
    want = roomy.generate(prompts, max_tokens=20, stop_at_eos=False)
    tight = LLM(folders["A"], dtype="float32", cache_tokens=96, max_active=4, max_step_tokens=48)
    got = tight.generate(prompts, max_tokens=20, stop_at_eos=False)
    assert got == want
    assert tight.scheduler.counters["preemptions"] >= 1 or any(s["reuses"] > 0 for s in tight.cache_stats().values())
    assert all(s["live"] == 0 for s in tight.cache_stats().values())
    with pytest.raises(ValueError, match="empty"):
        tight.generate([[]], max_tokens=3)
    with pytest.raises(ValueError, match="vocabulary"):
        tight.generate([vocab + 5], max_tokens=3)


def test_small_cache_with_sampling_and_repeat_penalty(folders):
    """Requests that lose their pages and start over keep their generator and their token counts: the
    sampled tokens are those of a roomy cache."""
    from glint_b200 import LLM
    vocab = TINY["A"][0]["vocab_size"]
    prompts = [random_tokens(n, vocab, 60 + i) for i, n in enumerate([30, 28, 35, 20])]
    opts = dict(max_tokens=20, stop_at_eos=False, temperature=0.8, top_k=8, repeat_penalty=1.4, seed=5)
    want = LLM(folders["A"], dtype="float32", cache_tokens=1024, max_active=4).generate(prompts, **opts)
    tight = LLM(folders["A"], dtype="float32", cache_tokens=96, max_active=4, max_step_tokens=48)
    assert tight.generate(prompts, **opts) == want
    assert tight.scheduler.counters["preemptions"] >= 1 or any(s["reuses"] > 0 for s in tight.cache_stats().values())


def test_eos_stops_and_is_delivered(folders, tmp_path):
    from glint_b200 import LLM
    vocab = TINY["A"][0]["vocab_size"]
    prompt = random_tokens(12, vocab, 3)
    llm = LLM(folders["A"], dtype="float32", cache_tokens=256, max_active=2)
    free = llm.generate(prompt, max_tokens=10, stop_at_eos=False)
    llm.eos_token_id = free[4]
    stopped = llm.generate(prompt, max_tokens=10)
    first = free.index(free[4])
    assert stopped == free[:first + 1]
    assert llm.last_requests[0].finish_reason == "stop"


def test_command_line(folders, tmp_path):
    env = dict(os.environ, PYTHONPATH=ROOT)
    run = lambda *args: subprocess.run([sys.executable, os.path.join(ROOT, "bin", "glint"), *args],
                                       capture_output=True, text=True, env=env, timeout=600)
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(TINY["A"][0]))
    out_dir = str(tmp_path / "made")
    p = run("init", "-c", str(cfg_path), "-o", out_dir, "--seed", "0", "--norm-std", "0.1")
    assert p.returncode == 0 and os.path.isfile(os.path.join(out_dir, "model.safetensors")), p.stderr
    p = run("inspect", "-f", out_dir, "--show-tensors")
    assert p.returncode == 0 and "model.embed_tokens.weight" in p.stdout and "head_count_kv: 2" in p.stdout
    p = run("generate", "-f", out_dir, "-t", "5,17,3", "-m", "6", "--dtype", "float32")
    assert p.returncode == 0, p.stderr
    ids = json.loads(p.stdout.strip().splitlines()[-1].split(":", 1)[1])
    want, _ = _plain_greedy(out_dir, [5, 17, 3], 6)
    assert ids == [5, 17, 3] + want
    p = run("run", "-f", out_dir, "-p", "5 17 3", "-m", "4", "--temperature", "0.7", "--seed", "1", "--dtype", "float32")
    assert p.returncode == 0 and "Output:" in p.stdout and "tok/s)" in p.stdout, p.stderr
    p = run("run", "-f", str(tmp_path / "nowhere"), "-p", "1", "-m", "1")
    assert p.returncode == 1 and "error:" in p.stderr
    p = run("bench", "-f", out_dir, "--mode", "all", "--prompt-len", "24", "--decode-tokens", "6", "--batch", "1,3",
            "--requests", "5", "--iters", "2", "--output", "json", "--dtype", "float32")
    assert p.returncode == 0, p.stderr
    rows = json.loads(p.stdout.strip().splitlines()[-1])["rows"]
    assert [r["mode"] for r in rows] == ["prefill", "decode", "decode", "serve"]
    assert all(r["tok_per_s"] > 0 for r in rows) and "frac_of_hbm_peak" in rows[1] and rows[3]["requests"] == 5


def test_slot_record_follows_the_plain_generator(folders):
    """The request's record in its slot on the device: after N sampled tokens the generator's state is
    the plain xorshift64's after N draws, the count is N and the position is the newest token's; a
    greedy request draws nothing; a request that loses its slot goes on from the state it had."""
    from glint_b200 import LLM
    from glint_b200.engine.scheduler import Request
    from glint_b200.sampling import SamplingParams
    vocab = TINY["A"][0]["vocab_size"]
    llm = LLM(folders["A"], dtype="float32", cache_tokens=512, max_active=3, max_step_tokens=16, lookahead=False)
    sch = llm.scheduler
    drawing = Request("d", random_tokens(21, vocab, 1), 40, SamplingParams(temperature=0.9, top_k=5, seed=11), None)
    greedy = Request("g", random_tokens(9, vocab, 2), 40, SamplingParams(), None)
    sch.add(drawing)
    sch.add(greedy)
    while len(drawing.output) < 13:
        sch.step()
    n = len(drawing.output)
    rec = llm.sampler.slot_record(drawing.slot)
    rng = psampler.Xorshift64(11)
    for _ in range(n):
        rng.next_u64()
    assert rec["rng_state"] == rng.state and rec["generated"] == n
    assert rec["position"] == len(drawing.prompt) + n - 1         # position of the newest token
    grec = llm.sampler.slot_record(greedy.slot)
    assert grec["rng_state"] == greedy.rng_state and grec["generated"] == len(greedy.output)   # drew nothing
    # preemption by hand: the state is read back, the slot freed, and the request goes on in another slot
    sch._preempt_or_finish()                                   # frees the request admitted last (the greedy one)
    assert greedy.slot is None and greedy in sch.waiting
    victim_state = drawing.rng_state
    sch.running.remove(drawing)
    drawing.rng_state = llm.sampler.generator_state(drawing.slot)
    assert drawing.rng_state == rng.state and drawing.rng_state != victim_state
    llm.engine.close(drawing.slot)
    drawing.slot, drawing.computed = None, 0
    sch.waiting.appendleft(drawing)
    before = list(drawing.output)
    sch.run()
    # the same request in one go draws the same tokens
    again = LLM(folders["A"], dtype="float32", cache_tokens=512, max_active=3, max_step_tokens=16, lookahead=False)
    want = again.generate(drawing.prompt, max_tokens=40, temperature=0.9, top_k=5, seed=11, stop_at_eos=False)
    assert drawing.output[:len(before)] == before and drawing.output == want


@pytest.mark.parametrize("temperature", [0.0, 0.7])
def test_eleven_requests_through_padded_graphs(folders, temperature):
    """Eleven requests decode in steps that replay the graph of twelve rows (one row of the engine's spare slot),
    with the next step launched ahead; output lengths differ, so the batch shrinks through 10, 9 (both padded to
    12) and 8 rows.  Greedy: the plain implementation's tokens.  Sampled: the tokens each request gets alone (its
    generator is its own)."""
    from glint_b200 import LLM
    from glint_b200.engine.scheduler import Request
    from glint_b200.sampling import SamplingParams
    vocab = TINY["A"][0]["vocab_size"]
    prompts = [random_tokens(6 + 2 * i, vocab, 300 + i) for i in range(11)]
    budgets = [14 - (i % 4) * 3 for i in range(11)]
    llm = LLM(folders["A"], dtype="float32", cache_tokens=2048, max_active=16, max_step_tokens=64)
    requests = [Request(("r", i), p, budgets[i], SamplingParams(temperature=temperature, seed=40 + i), None)
                for i, p in enumerate(prompts)]
    for r in requests:
        llm.scheduler.add(r)
    llm.scheduler.run()
    llm.model.rt.check_status()
    assert llm.engine.graph_counts["replayed"] > 0
    assert [len(r.output) for r in requests] == budgets
    alone = LLM(folders["A"], dtype="float32", cache_tokens=512, max_active=2, max_step_tokens=64)
    for i, r in enumerate(requests):
        if temperature == 0.0:
            want, margins = _plain_greedy(folders["A"], prompts[i], budgets[i])
            for k, (a, b) in enumerate(zip(r.output, want)):
                if a != b:
                    assert margins[k] < 1e-4, (i, k, r.output, want)
                    break
        elif i % 3 == 0:
            want = alone.generate(prompts[i], max_tokens=budgets[i], temperature=temperature, seed=40 + i,
                                  stop_at_eos=False)
            assert r.output == want, (i, r.output, want)
    assert all(s["live"] == 0 for s in llm.cache_stats().values())
