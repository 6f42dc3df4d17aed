"""The plain implementation checked against closed forms and the reference's own invariants
(no GPU): values from src/tensor/ops.rs:290-471, rotate-half equivalence
src/transformer/weights.rs:626-671, cap bound src/transformer/forward.rs:2489-2511."""
import math

import numpy as np
import pytest
import torch

from tests.helpers import TINY, make_model_dir, random_tokens
from tests.plain import model as plain
from tests.plain import sampler as psampler


def test_rms_norm_closed_form():
    x = torch.tensor([[1.0, 2.0, 3.0]])
    w = torch.tensor([0.0, 0.5, -0.5])
    r = 1.0 / math.sqrt((1 + 4 + 9) / 3 + 1e-6)
    want = torch.tensor([[1 * r * 1.0, 2 * r * 1.5, 3 * r * 0.5]])
    assert torch.allclose(plain.rms_norm(x, w, 1e-6), want, atol=1e-6)


def test_softcap_and_gelu_values():
    assert float(plain.softcap(torch.tensor(50.0), 50.0)) == pytest.approx(50 * math.tanh(1.0), rel=1e-6)
    assert float(plain.softcap(torch.tensor(3.0), None)) == 3.0
    assert float(plain.gelu_tanh(torch.tensor(1.0))) == pytest.approx(0.841192, abs=1e-5)
    assert float(plain.gelu_tanh(torch.tensor(0.0))) == 0.0


def test_rope_identity_at_position_zero_and_norm_kept():
    x = torch.randn(3, 2 * 16)
    assert torch.allclose(plain.rope_adjacent(x, [0, 0, 0], 16, 10000.0), x)
    y = plain.rope_adjacent(x, [5, 9, 100], 16, 10000.0)
    assert torch.allclose(y.reshape(3, 2, 16).norm(dim=-1), x.reshape(3, 2, 16).norm(dim=-1), atol=1e-5)


def test_permuted_adjacent_rope_equals_rotate_half():
    """The reference's row permutation + adjacent pairs against rotate-half on the file's order."""
    torch.manual_seed(0)
    nh, hd, H, T = 3, 8, 12, 5
    w = torch.randn(nh * hd, H)
    x = torch.randn(T, H)
    pos = [0, 1, 7, 30, 31]
    ours = plain.rope_adjacent(x @ plain.permute_qk_rows(w, nh, hd).T, pos, hd, 10000.0).reshape(T, nh, hd // 2, 2)
    q = (x @ w.T).reshape(T, nh, hd)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))
    ang = torch.tensor(pos).float()[:, None] * inv[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    lo, hi = q[..., :hd // 2], q[..., hd // 2:]
    assert torch.allclose(ours[..., 0], lo * cos - hi * sin, atol=1e-5)
    assert torch.allclose(ours[..., 1], lo * sin + hi * cos, atol=1e-5)


@pytest.mark.parametrize("name", ["A", "B"])
def test_logits_are_bounded_by_the_final_cap_and_causal(tmp_path, name):
    folder = make_model_dir(tmp_path, name)
    cfg = TINY[name][0]
    toks = random_tokens(30, cfg["vocab_size"], 3)
    full = plain.logits_of(folder, toks)
    assert full.shape == (30, cfg["vocab_size"]) and float(full.abs().max()) <= cfg["final_logit_softcapping"]
    part = plain.logits_of(folder, toks[:17])
    assert torch.allclose(full[:17], part, atol=1e-5)          # later tokens change nothing earlier


def test_window_hides_far_keys_on_even_layers_only(tmp_path):
    folder = make_model_dir(tmp_path, "B")                      # window 8
    c, w = plain.read_config(folder), plain.read_weights(folder)
    toks = random_tokens(24, c["vocab"], 4)
    other = list(toks)
    other[0] = (toks[0] + 1) % c["vocab"]                       # position 0 is outside every window at 23
    x_a = plain.embed(w["model.embed_tokens.weight"], toks, c["hidden"])
    x_b = plain.embed(w["model.embed_tokens.weight"], other, c["hidden"])
    lw = plain.layer_weights(w, 0)
    n = lambda x: plain.rms_norm(x, lw["in_norm"], c["eps"])
    even_a, even_b = plain.attention(n(x_a), lw, c, 0), plain.attention(n(x_b), lw, c, 0)
    odd_a, odd_b = plain.attention(n(x_a), lw, c, 1), plain.attention(n(x_b), lw, c, 1)
    assert torch.equal(even_a[8:], even_b[8:]) and not torch.equal(even_a[:8], even_b[:8])
    assert not torch.allclose(odd_a[23], odd_b[23])


def test_xorshift_matches_its_definition():
    r = psampler.Xorshift64(0)
    assert r.state == 1
    r = psampler.Xorshift64(42)
    s = 42
    s ^= (s << 13) & (2 ** 64 - 1); s ^= s >> 7; s ^= (s << 17) & (2 ** 64 - 1)
    assert r.next_u64() == s
    vals = [psampler.Xorshift64(7).next_f32() for _ in range(2)]
    assert vals[0] == vals[1] and 0.0 <= vals[0] < 1.0


def test_plain_sampler_stages():
    logits = [0.0, 5.0, 5.0, 1.0]
    assert psampler.argmax(logits) == 2                         # last of equal maxima
    rng = psampler.Xorshift64(1)
    assert psampler.sample(logits, [], rng, temperature=0.0) == 2
    counts = np.zeros(4)
    for _ in range(400):
        counts[psampler.sample([0.0, 1.0, 2.0, 3.0], [], rng, temperature=1.0, top_k=2)] += 1
    assert counts[0] == 0 and counts[1] == 0 and counts[3] > counts[2] > 0
    for _ in range(100):
        assert psampler.sample([0.0, 0.0, 10.0, 0.0], [], rng, temperature=1.0, top_p=0.5) == 2
        assert psampler.sample([0.0, 1.0, 9.0, 0.5], [], rng, temperature=1.0, min_p=0.1) == 2
    hot = psampler.sample([0.0, 3.0, 2.9, 0.0], [1, 1, 1], rng, temperature=0.01, repeat_penalty=2.0)
    assert hot == 2                                             # 3.0 / 2^3 falls below 2.9
