"""Configuration and registry (no GPU)."""
import json
import math

import pytest

from glint_b200.config import (Gemma2Config, config_from_dict, load_config, register_architecture,
                               registered_architectures)
from glint_b200.errors import ConfigError
from tests.helpers import TINY_A, TINY_B


def test_gemma2_keys_are_read():
    c = config_from_dict(dict(TINY_B))
    assert isinstance(c, Gemma2Config)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads) == (96, 5, 6, 1)
    assert (c.head_dim, c.intermediate_size, c.vocab_size, c.max_position_embeddings) == (32, 320, 1000, 256)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 100000.0 and c.sliding_window == 8
    assert c.attn_logit_softcapping == 20.0 and c.final_logit_softcapping == 15.0
    # query_pre_attn_scalar 16 -> multiplier 1/4 (reference: src/model/config.rs:291-294)
    assert c.score_multiplier() == pytest.approx(0.25)
    assert [c.layer_window(i) for i in range(4)] == [8, None, 8, None]


def test_defaults_follow_the_reference():
    d = {k: v for k, v in TINY_A.items() if k in ("architectures", "hidden_size", "num_hidden_layers",
                                                   "num_attention_heads", "vocab_size", "intermediate_size",
                                                   "max_position_embeddings")}
    c = config_from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads
    assert c.head_dim == 64 // 4
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0
    assert c.sliding_window is None and c.attn_logit_softcapping is None and c.final_logit_softcapping is None
    assert c.tie_word_embeddings is False
    assert c.score_multiplier() == pytest.approx(1 / math.sqrt(16))


def test_scalar_not_above_one_is_the_multiplier_itself():
    d = dict(TINY_A, query_pre_attn_scalar=0.5)
    assert config_from_dict(d).score_multiplier() == 0.5
    d = dict(TINY_A, query_pre_attn_scalar=1.0)
    assert config_from_dict(d).score_multiplier() == 1.0


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "vocab_size",
                                 "max_position_embeddings", "intermediate_size"])
def test_missing_required_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


def test_validation_errors():
    with pytest.raises(ConfigError, match="multiple"):
        config_from_dict(dict(TINY_A, num_attention_heads=4, num_key_value_heads=3))
    with pytest.raises(ConfigError, match="non-zero"):
        config_from_dict(dict(TINY_A, num_key_value_heads=0))
    with pytest.raises(ConfigError, match="rope_scaling"):
        config_from_dict(dict(TINY_A, rope_scaling={"rope_type": "yarn", "factor": 4.0}))
    with pytest.raises(ConfigError, match="hidden_activation"):
        config_from_dict(dict(TINY_A, hidden_activation="relu"))
    with pytest.raises(ConfigError, match="integer"):
        config_from_dict(dict(TINY_A, hidden_size="64"))
    d = dict(TINY_A)
    del d["head_dim"]
    with pytest.raises(ConfigError, match="divisible"):
        config_from_dict(dict(d, hidden_size=66))


def test_options():
    assert config_from_dict(dict(TINY_A, use_sliding_window=False)).sliding_window is None
    assert config_from_dict(dict(TINY_A, sliding_window=0)).sliding_window is None
    assert config_from_dict(dict(TINY_A, eos_token_id=[7, 9])).eos_token_id == 7
    assert config_from_dict(dict(TINY_A, rope_scaling={"type": "linear", "factor": 2.0})).rope_scaling_factor == 2.0
    assert config_from_dict(dict(TINY_A, rope_scaling={"rope_type": "default"})).rope_scaling_factor == 1.0


def test_round_trip_through_json(tmp_path):
    c = config_from_dict(dict(TINY_B, eos_token_id=1, bos_token_id=2, rope_scaling={"type": "linear", "factor": 2.0}))
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert load_config(str(tmp_path)) == c


def test_registry_picks_by_name_and_reports_unknown(tmp_path):
    assert "Gemma2ForCausalLM" in registered_architectures()
    d = dict(TINY_A)
    del d["architectures"]
    assert isinstance(config_from_dict(d), Gemma2Config)          # by model_type
    with pytest.raises(ConfigError, match="LlamaForCausalLM.*registered.*Gemma2ForCausalLM"):
        config_from_dict(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({"hidden_size": 4})
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="invalid JSON"):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError, match="not found"):
        load_config(str(tmp_path / "nowhere"))

    class Other:
        @classmethod
        def from_dict(cls, obj):
            return "other"
    register_architecture("OtherForCausalLM", Other)
    assert config_from_dict({"architectures": ["OtherForCausalLM"]}) == "other"


def test_model_spec_is_data():
    spec = config_from_dict(dict(TINY_B)).model_spec()
    assert len(spec.blocks) == 5 and [c.layer for c in spec.run_order] == [0, 1, 2, 3, 4]
    assert [b.mixer.params["window"] for b in spec.blocks] == [8, None, 8, None, 8]
    assert spec.blocks[0].mixer.kind == "attention" and spec.blocks[0].feed_forward.kind == "gated"
    assert spec.blocks[0].mixer.params["position"].kind == "rope"
    assert spec.embedding.params["scale"] == pytest.approx(math.sqrt(96.0))
    assert spec.head.params["softcap"] == 15.0
    assert spec.info["architecture"] == "gemma2" and spec.info["sliding_window"] == 8
