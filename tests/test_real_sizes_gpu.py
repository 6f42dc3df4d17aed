"""The kernels at the sizes of real models: hidden 2304, 8 heads of 256 in 4 groups, feed-forward 9216, and
hidden 4608, 32 heads of 128 in 16 groups, feed-forward 36864; vocabulary 256000, window 4096 (two layers,
random weights made on the device).

The tiny configurations of the other tests never reach the paths that these sizes take: whole-page TMA
boxes over four 64-column slices, the dual-tile product, split factors and clusters chosen for 148 SMs,
the argmax over several blocks.  Here the bfloat16 engine is compared with the 32-bit engine (CUDA-core
kernels, the same weights widened) and with itself under other cuts and in a mixed batch.
"""
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
        out[dtype] = build_engine(model, 6144 if dtype == "bfloat16" else 1024, num_slots=4)
    made.clear()
    yield out
    out.clear()
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


def test_bfloat16_engine_against_the_32_bit_engine_at_real_sizes(engines):
    toks = _requests()[1]
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
