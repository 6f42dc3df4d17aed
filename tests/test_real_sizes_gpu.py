"""The kernels at the sizes of real models: hidden 2304, 8 heads of 256 in 4 groups, feed-forward 9216, and
hidden 4608, 32 heads of 128 in 16 groups, feed-forward 36864; vocabulary 256000, window 4096 (two layers,
random weights made on the device).

The tiny configurations of the other tests never reach the paths that these sizes take: whole-page TMA
boxes over four 64-column slices, the dual-tile product, split factors and clusters chosen for 148 SMs,
the argmax over several blocks.  Here the 32-bit engine is compared with the plain implementation (the same
weights on the CPU), the bfloat16 engine with the 32-bit engine (CUDA-core kernels, the same weights widened),
also on a request longer than the window, and with itself under other cuts, in a mixed batch and in a decode
step of 64 requests; and the entry point's tokens (CUDA graphs, the next step launched ahead) with a plain
step-by-step run.
"""
import json
import os

import numpy as np
import pytest
import torch

from tests.helpers import tolerance

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "num_hidden_layers": 2, "hidden_size": 2304,
    "num_attention_heads": 8, "num_key_value_heads": 4, "head_dim": 256, "intermediate_size": 9216,
    "vocab_size": 256000, "rope_theta": 10000.0, "sliding_window": 4096, "attn_logit_softcapping": 50.0,
    "final_logit_softcapping": 30.0, "query_pre_attn_scalar": 256, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 8192, "tie_word_embeddings": True, "hidden_activation": "gelu_pytorch_tanh",
}
TAIL = 6
SHAPES = {
    "2b": {},
    "9b": {"hidden_size": 3584, "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 256,
           "intermediate_size": 14336, "query_pre_attn_scalar": 256},
    "27b": {"hidden_size": 4608, "num_attention_heads": 32, "num_key_value_heads": 16, "head_dim": 128,
            "intermediate_size": 36864, "query_pre_attn_scalar": 144},
}


@pytest.fixture(scope="module", params=sorted(SHAPES))
def engines(request):
    from glint_b200.config import config_from_dict
    from glint_b200.engine.loading import build_engine
    from glint_b200.engine.model import CausalLM
    from glint_b200.runtime import Runtime
    from glint_b200.weights.loader import kept_dtype
    config = config_from_dict(dict(CONFIG, **SHAPES[request.param]))
    gen = torch.Generator(device="cuda:0")
    gen.manual_seed(11)
    made = {}
    out = {}
    for dtype in ("bfloat16", "float32"):
        rt = Runtime("cuda:0", dtype, "auto")
        model = CausalLM(config.model_spec(), rt)
        model.config = config
        tensors = {}
        for need in sorted(model.needs(), key=lambda n: n.name):
            if need.optional:
                continue
            if need.name not in made:                  # made once, as a bfloat16 file would hold them
                t = torch.empty(need.shape, dtype=torch.float32, device="cuda:0")
                t.normal_(0.0, 0.3 if need.kind == "vector" else 0.02, generator=gen)
                made[need.name] = t.to(torch.bfloat16)
            tensors[need.name] = made[need.name].to(kept_dtype(need.kind, "BF16", rt.dtype))
        model.bind(tensors)
        out[dtype] = build_engine(model, 6144 if dtype == "bfloat16" else 4608, num_slots=4)
    out["config"] = dict(CONFIG, **SHAPES[request.param])
    out["weights"] = made            # name -> bfloat16 tensor on the device, as a file would hold them
    yield out
    out.clear()
    made.clear()
    torch.cuda.empty_cache()


def _whole(engine, toks):
    from glint_b200.engine.step import StepEntry
    s = engine.open()
    out = engine.step([StepEntry(s, toks, list(range(len(toks) - TAIL, len(toks))))]).float().cpu().numpy()
    engine.close(s)
    return out


def _requests():
    rng = np.random.default_rng(4)
    return [[int(t) for t in rng.integers(0, CONFIG["vocab_size"], size=n)] for n in (300, 701, 4500)]


def test_32_bit_engine_against_the_plain_implementation_at_real_sizes(engines, tmp_path):
    """Head sizes 256 and 128, 2, 4 and 16 groups, vocabulary 256000: the 32-bit engine's logits at the last
    positions of a 300-token request against the plain implementation on the CPU with the same weights.

    Sums of 2,304 to 36,864 products in 32-bit differ with the order of summation by more than those of the
    tiny models (whose bound of 2e-5 stays the floor here).  The yardstick is therefore the plain
    implementation in 64-bit: the engine may lie as far from it as three times the distance of the plain
    implementation's own 32-bit run, which is what the order of summation alone costs at these sizes
    (a wrong page, head or position shows as 1e-2 and more)."""
    from tests.plain import model as plain
    toks = _requests()[0]
    with open(os.path.join(str(tmp_path), "config.json"), "w") as f:
        json.dump(engines["config"], f)
    c = plain.read_config(str(tmp_path))
    rows = range(len(toks) - TAIL, len(toks))
    w = {k: v.double().cpu() for k, v in engines["weights"].items()}
    truth = plain.forward(c, w, toks, positions=rows).numpy()
    w = {k: v.float() for k, v in w.items()}
    plain32 = plain.forward(c, w, toks, positions=rows).numpy()
    del w
    got = _whole(engines["float32"], toks)
    assert np.abs(truth).max() > 1.0
    own = float(np.abs(plain32 - truth).max())
    err = float(np.abs(got - truth).max())
    assert err <= max(tolerance("float32", truth), 3.0 * own), (err, own)
    assert float(np.abs(got - plain32).max()) <= max(tolerance("float32", truth), 4.0 * own)
    engines["float32"].rt.check_status()


@pytest.mark.parametrize("which", [1, 2])
def test_bfloat16_engine_against_the_32_bit_engine_at_real_sizes(engines, which):
    """A request of 701 tokens, and one of 4500 tokens, whose last positions lie past the window of 4096."""
    toks = _requests()[which]
    want = _whole(engines["float32"], toks)
    got = _whole(engines["bfloat16"], toks)
    assert np.abs(want).max() > 1.0
    assert np.abs(got - want).max() <= tolerance("bfloat16", want), np.abs(got - want).max() / np.abs(want).max()
    engines["bfloat16"].rt.check_status()
    engines["float32"].rt.check_status()


def test_cuts_and_batches_do_not_matter_at_real_sizes(engines):
    """Whole against portions of changing size with the last tokens decoded one by one, and against a
    mixed batch of all requests; one request is longer than the window."""
    from glint_b200.engine.step import StepEntry
    engine = engines["bfloat16"]
    reqs = _requests()
    ref = [_whole(engine, r) for r in reqs]
    scale = max(np.abs(r).max() for r in ref)
    rng = np.random.default_rng(9)
    # portions, then single tokens
    for i, r in enumerate(reqs):
        s, at, sizes, k = engine.open(), 0, [2, 300, 17, 1024], 0
        while at < len(r) - TAIL:
            n = min(sizes[k % 4], len(r) - TAIL - at)
            k += 1
            engine.step([StepEntry(s, r[at:at + n], [])])
            at += n
        got = np.concatenate([engine.step([StepEntry(s, r[t:t + 1], [0])]).float().cpu().numpy()
                              for t in range(len(r) - TAIL, len(r))])
        engine.close(s)
        assert np.abs(got - ref[i]).max() <= 0.01 * scale, (i, np.abs(got - ref[i]).max() / scale)
        assert (got.argmax(1) == ref[i].argmax(1)).all()
    # all requests together: portions of some beside single tokens of others
    slots, at, outs = [engine.open() for _ in reqs], [0] * len(reqs), [[] for _ in reqs]
    while any(at[i] < len(r) for i, r in enumerate(reqs)):
        entries, who = [], []
        for i, r in enumerate(reqs):
            left = len(r) - at[i]
            if left <= 0:
                continue
            n = 1 if left <= TAIL else min(int(rng.integers(1, 400)), left - TAIL)
            entries.append(StepEntry(slots[i], r[at[i]:at[i] + n], [0] if left <= TAIL else []))
            who.append((i, left <= TAIL))
            at[i] += n
        out = engine.step(entries)
        row = 0
        for i, wanted in who:
            if wanted:
                outs[i].append(out[row:row + 1].float().cpu().numpy())
                row += 1
    for s in slots:
        engine.close(s)
    for i in range(len(reqs)):
        got = np.concatenate(outs[i])
        assert np.abs(got - ref[i]).max() <= 0.01 * scale, (i, np.abs(got - ref[i]).max() / scale)
    engine.rt.check_status()


def test_decode_step_of_64_requests_against_each_request_alone(engines):
    """One decode step of 64 requests with contexts from a few tokens to past the window (the tiled products'
    64-token tiles, attention without a split of the keys): every request's logits are those it gets alone."""
    from glint_b200.engine.loading import build_engine
    from glint_b200.engine.step import StepEntry
    model = engines["bfloat16"].model
    rng = np.random.default_rng(21)
    lengths = [int(n) for n in rng.integers(3, 700, size=60)] + [4090, 4097, 4400, 5000]
    engine = build_engine(model, sum(lengths) + 64 * 32, num_slots=64)
    reqs = [[int(t) for t in rng.integers(0, CONFIG["vocab_size"], size=n)] for n in lengths]
    slots = [engine.open() for _ in reqs]
    for s, r in zip(slots, reqs):
        for at in range(0, len(r) - 1, 2048):
            engine.step([StepEntry(s, r[at:min(at + 2048, len(r) - 1)], [])])
    together = engine.step([StepEntry(s, r[-1:], [0]) for s, r in zip(slots, reqs)]).float().cpu().numpy()
    for s in slots:
        engine.close(s)
    scale = np.abs(together).max()
    worst = 0.0
    for i in list(range(0, 60, 7)) + [60, 61, 62, 63]:
        r = reqs[i]
        s = engine.open()
        for at in range(0, len(r) - 1, 2048):
            engine.step([StepEntry(s, r[at:min(at + 2048, len(r) - 1)], [])])
        alone = engine.step([StepEntry(s, r[-1:], [0])]).float().cpu().numpy()
        engine.close(s)
        worst = max(worst, float(np.abs(alone[0] - together[i]).max()))
    assert scale > 1.0 and worst <= 0.01 * scale, worst / scale
    engine.rt.check_status()


def test_entry_point_with_graphs_and_lookahead_at_real_sizes(engines):
    """``LLM.generate`` with CUDA graphs and the next step launched ahead, 8 prompts: at every step the chosen
    token's logit in a plain step-by-step run (no graphs, one request at a time) is the largest within the
    rounding of a logit; and a wrong token does not pass the same check."""
    from glint_b200 import LLM
    from glint_b200 import bench as B
    model = engines["bfloat16"].model
    llm = LLM(model=model, cache_tokens=8 * 1024, max_active=8, max_step_tokens=1024)
    rng = np.random.default_rng(33)
    prompts = [[int(t) for t in rng.integers(0, CONFIG["vocab_size"], size=n)] for n in (40, 333, 64, 700, 5, 129, 256, 90)]
    worst = B.check_generate(llm, prompts, new_tokens=12)
    assert worst <= 0.025
    assert llm.engine.graph_counts["replayed"] >= 8
    real = llm.generate

    def off_by_one(prompts, **kw):
        out = real(prompts, **kw)
        out[3][5] = (out[3][5] + 1) % CONFIG["vocab_size"]
        return out

    llm.generate = off_by_one
    with pytest.raises(AssertionError):
        B.check_generate(llm, prompts, new_tokens=12)
