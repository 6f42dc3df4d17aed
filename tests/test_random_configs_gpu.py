"""Configurations drawn at random (head sizes in steps of 16 up to 256, one to three groups of one to
four heads, widths and vocabularies that are no power of two, windows, caps, tied or untied head):
the engine in 32-bit and in bfloat16 against the plain implementation, each request whole, in
portions, with its tail decoded and mixed with the others."""
import os
import random

import numpy as np
import pytest

from tests import tracing
from tests.helpers import plain_logits, random_tokens, tolerance

pytestmark = pytest.mark.gpu


def _draw(seed):
    rnd = random.Random(seed)
    hd = rnd.choice([16, 32, 48, 64, 80, 96, 128, 256])
    nkv = rnd.choice([1, 2, 3])
    nh = nkv * rnd.choice([1, 2, 4] if hd <= 128 else [1, 2])
    cfg = {"architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "num_hidden_layers": rnd.randint(1, 3),
           "hidden_size": 8 * rnd.randint(5, 40), "num_attention_heads": nh, "num_key_value_heads": nkv,
           "head_dim": hd, "intermediate_size": 8 * rnd.randint(6, 60), "vocab_size": rnd.randint(130, 1500),
           "rope_theta": rnd.choice([10000.0, 50000.0, 1e6]), "sliding_window": rnd.choice([8, 24, 40, 100]),
           "attn_logit_softcapping": rnd.choice([20.0, 50.0]), "final_logit_softcapping": rnd.choice([15.0, 30.0]),
           "query_pre_attn_scalar": rnd.choice([hd, 2 * hd, 144]), "rms_norm_eps": rnd.choice([1e-6, 1e-5]),
           "max_position_embeddings": 512, "tie_word_embeddings": rnd.random() < 0.7,
           "hidden_activation": "gelu_pytorch_tanh"}
    lens = [rnd.randint(1, 20), rnd.randint(20, 90), rnd.randint(90, 200), rnd.randint(2, 60)]
    return cfg, lens


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16])
def test_random_configuration_against_the_plain_implementation(tmp_path, seed):
    from glint_b200.engine.loading import build_engine, load_model
    from glint_b200.weights import write_random_model
    cfg, lens = _draw(seed)
    folder = os.path.join(str(tmp_path), "model")
    write_random_model(dict(cfg), folder, seed=seed, std=0.05, norm_std=0.15, untied_head=not cfg["tie_word_embeddings"])
    reqs = {f"r{i}": random_tokens(n, cfg["vocab_size"], 7 * seed + i) for i, n in enumerate(lens)}
    want = {rid: plain_logits(folder, toks) for rid, toks in reqs.items()}
    modes = {"whole": tracing.whole(reqs), "chunked": tracing.chunked(reqs), "mixed": tracing.mixed(reqs, seed=seed),
             "tail": tracing.tail_decode(reqs, 24)}
    for dtype in ("float32", "bfloat16"):
        for mode, steps in modes.items():
            engine = build_engine(load_model(folder, dtype), tracing.max_live_tokens(steps), num_slots=4)
            got = tracing.collect(steps, tracing.run_in_process(engine, steps), cfg["vocab_size"])
            engine.rt.check_status()
            for rid in reqs:
                diff = float(np.abs(got[rid] - want[rid]).max())
                assert diff <= tolerance(dtype, want[rid]), (cfg, dtype, mode, rid, diff)
