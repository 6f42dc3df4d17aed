"""Replay on the GPU against the plain implementation: each request whole, most of it in one
step and the last 32 tokens one by one, portions of changing size, and mixed batches with so
few pages that they are used again; in 32-bit and in bfloat16."""
import numpy as np
import pytest

from tests import tracing
from tests.helpers import TINY, make_model_dir, plain_logits, random_tokens, tolerance

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 23, 40, 61], "B": [1, 9, 31, 77], "C": [3, 50, 120, 97]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {name: make_model_dir(root, name) for name in TINY}


@pytest.fixture(scope="module")
def expected(folders):
    out = {}
    for name, folder in folders.items():
        vocab = TINY[name][0]["vocab_size"]
        reqs = {f"r{i}": random_tokens(n, vocab, 100 * ord(name) + i) for i, n in enumerate(LENGTHS[name])}
        out[name] = (reqs, {rid: plain_logits(folder, toks) for rid, toks in reqs.items()})
    return out


def _engine(folder, dtype, max_tokens, kernels="auto", attention="routed"):
    from glint_b200.engine.loading import build_engine, load_model
    engine = build_engine(load_model(folder, dtype, kernels=kernels), max_tokens, num_slots=4)
    engine.rt.single_token_attention(attention)
    return engine


def _check(name, dtype, steps, outputs, expected_logits):
    vocab = TINY[name][0]["vocab_size"]
    got = tracing.collect(steps, outputs, vocab)
    for rid, want in expected_logits.items():
        assert got[rid].shape == want.shape, (rid, got[rid].shape, want.shape)
        diff = np.abs(got[rid] - want)
        tol = tolerance(dtype, want)
        worst = np.unravel_index(np.argmax(diff), diff.shape)
        assert diff.max() <= tol, (
            f"{name}/{dtype}/{rid}: max |diff| {diff.max():.3e} (bound {tol:.3e}) at position {worst[0]}, token "
            f"{worst[1]}; first position over the bound: {int(np.argmax(diff.max(axis=1) > tol))}")


MODES = {
    "whole": lambda reqs: tracing.whole(reqs),
    "tail": lambda reqs: tracing.tail_decode(reqs, 32),
    "chunked": lambda reqs: tracing.chunked(reqs),
    "mixed": lambda reqs: tracing.mixed(reqs, seed=3),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("name", list(TINY))
def test_replay_in_process(folders, expected, name, mode, dtype):
    reqs, want = expected[name]
    steps = MODES[mode](reqs)
    engine = _engine(folders[name], dtype, tracing.max_live_tokens(steps))
    outputs = tracing.run_in_process(engine, steps)
    _check(name, dtype, steps, outputs, want)
    if mode == "mixed":
        assert any(s["reuses"] > 0 for s in engine.cache.stats().values()), "no page was used again"
    assert all(s["live"] == 0 for s in engine.cache.stats().values())


@pytest.mark.parametrize("mode", ["tail", "mixed"])
@pytest.mark.parametrize("name", list(TINY))
def test_replay_with_the_page_sharing_attention_kernel(folders, expected, name, mode):
    """Single tokens through the kernel that shares all pages of a launch evenly among its blocks (the runtime
    takes it only for larger launches than these): the last 32 tokens one by one, and mixed steps with pages
    that are used again."""
    reqs, want = expected[name]
    steps = MODES[mode](reqs)
    engine = _engine(folders[name], "bfloat16", tracing.max_live_tokens(steps), attention="stream")
    outputs = tracing.run_in_process(engine, steps)
    _check(name, "bfloat16", steps, outputs, want)
    assert all(s["live"] == 0 for s in engine.cache.stats().values())
    engine.rt.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_child_process(folders, expected, tmp_path, dtype):
    """The same through bin/trace_run as a child process (mixed trace of configuration B)."""
    reqs, want = expected["B"]
    steps = tracing.mixed(reqs, seed=7)
    outputs = tracing.run_child(folders["B"], dtype, steps, str(tmp_path / "out"),
                                tracing.max_live_tokens(steps), TINY["B"][0]["vocab_size"])
    _check("B", dtype, steps, outputs, want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_single_tokens_in_front_of_portions(folders, expected, name, dtype):
    """A step with decoding requests first and prompt portions behind them (a scheduler's order) sends
    the single tokens to the split attention kernel and the portions to the tiled one; the same step
    with the portions first takes the tiled kernel for all.  Both must give the plain logits."""
    from glint_b200.engine.step import StepEntry
    reqs, want = expected[name]
    ids = sorted(reqs)
    engine = _engine(folders[name], dtype, 512)
    for portions_first in (False, True):
        slots = {rid: engine.open() for rid in ids}
        singles, portions = ids[2:], ids[:2]                     # the two longest requests decode
        for rid in singles:                                       # all but their last token are in the cache
            engine.step([StepEntry(slots[rid], reqs[rid][:-1], [])])
        for rid in portions:                                      # the first two tokens of the portions too
            engine.step([StepEntry(slots[rid], reqs[rid][:2], [])]) if len(reqs[rid]) > 3 else None
        entries, order = [], []
        for rid in (portions + singles if portions_first else singles + portions):
            toks = reqs[rid]
            if rid in singles:
                entries.append(StepEntry(slots[rid], toks[-1:], [0]))
            else:
                at = 2 if len(toks) > 3 else 0
                entries.append(StepEntry(slots[rid], toks[at:], [len(toks) - at - 1]))
            order.append(rid)
        got = engine.step(entries).float().cpu().numpy()
        for row, rid in enumerate(order):
            diff = np.abs(got[row] - want[rid][-1]).max()
            assert diff <= tolerance(dtype, want[rid]), (name, dtype, portions_first, rid, diff)
        for s_ in slots.values():
            engine.close(s_)
        engine.rt.check_status()


@pytest.mark.parametrize("attention", ["routed", "stream"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_padded_to_a_graph_size(folders, dtype, attention):
    """Steps of 11 and then 9 single tokens replay the graph captured for 12 (the rows that fill the step
    up belong to the engine's spare slot): the logits are the plain ones at every step, a request that ends
    changes nothing for the others, and the spare slot's page is not counted among the caller's."""
    from glint_b200.engine.loading import build_engine, load_model
    from glint_b200.engine.step import StepEntry, padded_size
    assert [padded_size(n) for n in (1, 8, 9, 12, 13, 33, 64, 65)] == [1, 8, 12, 12, 16, 40, 64, 80]
    name = "C"
    vocab = TINY[name][0]["vocab_size"]
    reqs = [random_tokens(14 + 3 * i, vocab, 700 + i) for i in range(11)]
    want = [plain_logits(folders[name], r) for r in reqs]
    engine = build_engine(load_model(folders[name], dtype), 11 * 64, num_slots=11)
    engine.rt.single_token_attention(attention)
    slots = [engine.open() for _ in reqs]
    tail = 6
    for s, r in zip(slots, reqs):
        engine.step([StepEntry(s, r[:-tail], [])])
    live = list(range(11))
    for t in range(tail):
        if t == 4:                                              # two requests end: 9 rows, the same graph
            for i in (3, 7):
                engine.close(slots[i])
                live.remove(i)
        got = engine.step([StepEntry(slots[i], [reqs[i][len(reqs[i]) - tail + t]], [0]) for i in live])
        got = got.float().cpu().numpy()
        assert got.shape[0] == len(live)
        for row, i in enumerate(live):
            ref = want[i][len(reqs[i]) - tail + t]
            assert np.abs(got[row] - ref).max() <= tolerance(dtype, want[i]), (dtype, t, i)
    assert engine.graph_counts["replayed"] >= 4 and engine.graph_counts["captured"] == 1
    for i in live:
        engine.close(slots[i])
    assert all(s["live"] == 0 for s in engine.cache.stats().values())
    engine.cache.check_consistency()
    engine.rt.check_status()
