"""Weight files, loader errors and the random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from glint_b200.config import config_from_dict
from glint_b200.errors import WeightsError
from glint_b200.weights import (SafeTensorsFile, SafeTensorsModel, compare, model_needs, raise_if_mismatch,
                                random_tensors, write_random_model, write_safetensors)
from tests.helpers import TINY_A, TINY_A_INIT, TINY_B, TINY_C


def _raw(path, header, data=b""):
    raw = header if isinstance(header, bytes) else json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)) + raw + data)
    return str(path)


def test_write_then_read_matches_the_safetensors_library(tmp_path):
    from safetensors.torch import load_file
    folder = write_random_model(dict(TINY_A), str(tmp_path / "a"), **TINY_A_INIT)
    ours = SafeTensorsModel(folder)
    theirs = load_file(os.path.join(folder, "model.safetensors"))
    assert sorted(ours.names()) == sorted(theirs)
    for name, t in theirs.items():
        assert ours.dtype_name(name) == "BF16" and torch.equal(ours.tensor(name), t)
    assert "lm_head.weight" not in theirs                      # tied: no head tensor written
    cfg = json.load(open(os.path.join(folder, "config.json")))
    assert cfg["architectures"] == ["Gemma2ForCausalLM"] and cfg["hidden_size"] == 64


def test_random_mode_is_seeded_and_scaled(tmp_path):
    needs = model_needs(config_from_dict(dict(TINY_B)))
    a = random_tensors(needs, 1, 0.05, 0.2, torch.float32)
    b = random_tensors(needs, 1, 0.05, 0.2, torch.float32)
    c = random_tensors(needs, 2, 0.05, 0.2, torch.float32)
    assert all(torch.equal(a[k], b[k]) for k in a) and any(not torch.equal(a[k], c[k]) for k in a)
    emb = a["model.embed_tokens.weight"]
    assert emb.shape == (1000, 96) and abs(float(emb.std()) - 0.05) < 0.002
    norms = torch.cat([v for k, v in a.items() if "norm" in k])
    assert abs(float(norms.std()) - 0.2) < 0.02
    folder = write_random_model(dict(TINY_C), str(tmp_path / "c"), seed=5, untied_head=True)
    assert "lm_head.weight" in SafeTensorsModel(folder).names()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config = config_from_dict(dict(TINY_A))
    needs = model_needs(config)
    tensors = random_tensors(needs, 0)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(16, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    tensors["model.embed_tokens.weight"] = torch.zeros(512, 64, dtype=torch.int32)
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, tensors)
    files = SafeTensorsModel(str(tmp_path))
    available = {n: (files.shape(n), files.dtype_name(n)) for n in files.names()}
    with pytest.raises(WeightsError) as err:
        raise_if_mismatch("here", *compare(needs, available))
    e = err.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert len(e.wrong_shape) == 2
    text = str(e)
    assert "expected shape [32, 64], found [16, 64]" in text and "model.norm.weight" in text
    assert "q_norm" in text and "I32" in text
    # the optional head tensor is neither missing nor unexpected
    ok = random_tensors(needs, 0, include_optional=True)
    assert compare(needs, {k: (tuple(v.shape), "BF16") for k, v in ok.items()}) == ([], [], [])


HOSTILE = {
    "short file": lambda p: open(p, "wb").write(b"\x01\x02") and str(p),
    "header longer than file": lambda p: open(p, "wb").write(struct.pack("<Q", 1000) + b"{}") and str(p),
    "header over 100 MiB": lambda p: open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}") and str(p),
    "not json": lambda p: _raw(p, b"{nope"),
    "not an object": lambda p: _raw(p, b"[1,2]"),
    "entry not an object": lambda p: _raw(p, {"a": 3}),
    "unknown dtype": lambda p: _raw(p, {"a": {"dtype": "F8_E4M3", "shape": [1], "data_offsets": [0, 1]}}, b"\0"),
    "rank over 8": lambda p: _raw(p, {"a": {"dtype": "F32", "shape": [1] * 9, "data_offsets": [0, 4]}}, b"\0" * 4),
    "negative dim": lambda p: _raw(p, {"a": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 4]}}, b"\0" * 4),
    "shape overflow": lambda p: _raw(p, {"a": {"dtype": "F32", "shape": [1 << 40, 1 << 40], "data_offsets": [0, 4]}}, b"\0" * 4),
    "offsets past the data": lambda p: _raw(p, {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4),
    "begin after end": lambda p: _raw(p, {"a": {"dtype": "F32", "shape": [1], "data_offsets": [4, 0]}}, b"\0" * 4),
    "size mismatch": lambda p: _raw(p, {"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8),
    "overlap": lambda p: _raw(p, {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                                  "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12),
    "bad offsets type": lambda p: _raw(p, {"a": {"dtype": "F32", "shape": [1], "data_offsets": "0-4"}}, b"\0" * 4),
}


@pytest.mark.parametrize("case", list(HOSTILE))
def test_hostile_files_are_errors_not_crashes(tmp_path, case):
    path = HOSTILE[case](tmp_path / "model.safetensors")
    with pytest.raises(WeightsError):
        SafeTensorsFile(str(tmp_path / "model.safetensors"))


def test_shards_duplicates_and_path_escape(tmp_path):
    a = {"x": torch.ones(2, 2), "y": torch.zeros(3)}
    write_safetensors(str(tmp_path / "s1.safetensors"), {"x": a["x"]})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"y": a["y"]})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    m = SafeTensorsModel(str(tmp_path))
    assert torch.equal(m.tensor("x"), a["x"]) and torch.equal(m.tensor("y"), a["y"])
    write_safetensors(str(tmp_path / "s2.safetensors"), {"y": a["y"], "x": a["x"]})
    with pytest.raises(WeightsError, match="both"):
        SafeTensorsModel(str(tmp_path))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "../s1.safetensors"}}))
    with pytest.raises(WeightsError, match="leaves"):
        SafeTensorsModel(str(tmp_path))
    with pytest.raises(WeightsError, match="no .safetensors"):
        SafeTensorsModel(str(tmp_path / "empty_missing"))
