"""Typed configuration of Gemma 2, read from its own config.json keys.

Restates what the reference reads for this family in ``HfConfig::from_json``
(src/model/config.rs:180-341): required keys, defaults, validation and the
error for each.  Where the reference keeps ``Option`` fields for all families
this class has exactly the Gemma 2 keys.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict
from typing import Optional

from ..errors import ConfigError
from .spec import BlockSpec, LayerCall, ModelSpec, PartSpec

ARCHITECTURE = "Gemma2ForCausalLM"
MODEL_TYPE = "gemma2"

_ACTIVATIONS = {"gelu_pytorch_tanh": "gelu_tanh", "gelu_tanh": "gelu_tanh"}


def _require(obj, key, kind):
    if key not in obj or obj[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    return _typed(obj, key, kind)


def _typed(obj, key, kind):
    v = obj[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int) or v < 0:
            raise ConfigError(f"config.json: '{key}' must be a non-negative integer, found {v!r}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, found {v!r}")
        return float(v)
    if kind is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: '{key}' must be true or false, found {v!r}")
        return v
    raise AssertionError(kind)


def _optional(obj, key, kind, default=None):
    if key not in obj or obj[key] is None:
        return default
    return _typed(obj, key, kind)


@dataclass
class Gemma2Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling_factor: float = 1.0
    sliding_window: Optional[int] = None
    attn_logit_softcapping: Optional[float] = None
    final_logit_softcapping: Optional[float] = None
    query_pre_attn_scalar: Optional[float] = None
    hidden_activation: str = "gelu_pytorch_tanh"
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None

    # ---- reading ---------------------------------------------------------------------------

    @classmethod
    def from_dict(cls, obj):
        """Build from the parsed config.json.

        Required (src/model/config.rs:198-230): hidden_size, num_hidden_layers,
        num_attention_heads, vocab_size, max_position_embeddings; for this family also
        intermediate_size (the reference takes it from the gate tensor's rows,
        src/transformer/weights.rs:270-271; a folder written from a configuration and a
        seed has no tensor to take it from).  Defaults: kv heads = heads (:231), head_dim =
        hidden/heads (:131-134), eps 1e-5 (:307), rope_theta 10000
        (src/transformer/forward.rs:539), tie false (:334-337).
        """
        if not isinstance(obj, dict):
            raise ConfigError("config.json: top level value is not a JSON object")
        c = cls(
            hidden_size=_require(obj, "hidden_size", int),
            num_hidden_layers=_require(obj, "num_hidden_layers", int),
            num_attention_heads=_require(obj, "num_attention_heads", int),
            num_key_value_heads=0,
            head_dim=0,
            intermediate_size=_require(obj, "intermediate_size", int),
            vocab_size=_require(obj, "vocab_size", int),
            max_position_embeddings=_require(obj, "max_position_embeddings", int),
        )
        c.num_key_value_heads = _optional(obj, "num_key_value_heads", int, c.num_attention_heads)
        if c.num_attention_heads == 0 or c.num_key_value_heads == 0:
            raise ConfigError("config.json: num_attention_heads / num_key_value_heads must be non-zero")
        head_dim = _optional(obj, "head_dim", int)
        if head_dim is None:
            if c.hidden_size % c.num_attention_heads != 0:
                raise ConfigError(f"config.json: hidden_size {c.hidden_size} is not divisible by "
                                  f"num_attention_heads {c.num_attention_heads} and no head_dim is given")
            head_dim = c.hidden_size // c.num_attention_heads
        c.head_dim = head_dim
        c.rms_norm_eps = _optional(obj, "rms_norm_eps", float, 1e-5)
        c.rope_theta = _optional(obj, "rope_theta", float, 10000.0)
        c.attn_logit_softcapping = _optional(obj, "attn_logit_softcapping", float)
        c.final_logit_softcapping = _optional(obj, "final_logit_softcapping", float)
        c.query_pre_attn_scalar = _optional(obj, "query_pre_attn_scalar", float)
        c.tie_word_embeddings = _optional(obj, "tie_word_embeddings", bool, False)
        c.bos_token_id = _optional(obj, "bos_token_id", int)
        eos = obj.get("eos_token_id")
        if isinstance(eos, list):  # first of a list, src/model/config.rs:324-330
            eos = eos[0] if eos else None
            c.eos_token_id = None if eos is None else _typed({"eos_token_id": eos}, "eos_token_id", int)
        else:
            c.eos_token_id = _optional(obj, "eos_token_id", int)
        # use_sliding_window:false switches the window off (src/model/config.rs:261-264)
        window = _optional(obj, "sliding_window", int)
        if obj.get("use_sliding_window") is False or not window:
            window = None
        c.sliding_window = window
        # only linear RoPE scaling exists (src/model/config.rs:270-289)
        scaling = obj.get("rope_scaling")
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError("config.json: 'rope_scaling' must be an object")
            kind = scaling.get("rope_type", scaling.get("type", "linear"))
            factor = scaling.get("factor")
            if kind == "linear" and isinstance(factor, (int, float)) and not isinstance(factor, bool):
                c.rope_scaling_factor = float(factor)
            elif kind == "default":
                c.rope_scaling_factor = 1.0
            else:
                raise ConfigError(f"config.json: rope_scaling type '{kind}' — only linear scaling is implemented")
        act = obj.get("hidden_activation", obj.get("hidden_act", "gelu_pytorch_tanh"))
        if act not in _ACTIVATIONS:
            raise ConfigError(f"config.json: hidden_activation '{act}' is not supported "
                              f"(supported: {', '.join(sorted(_ACTIVATIONS))})")
        c.hidden_activation = act
        c.validate()
        return c

    def validate(self):
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(f"config.json: num_attention_heads {self.num_attention_heads} is not a "
                              f"multiple of num_key_value_heads {self.num_key_value_heads}")
        for key in ("hidden_size", "num_hidden_layers", "head_dim", "intermediate_size", "vocab_size",
                    "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"config.json: '{key}' must be positive")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary encoding")
        if not self.rms_norm_eps > 0:
            raise ConfigError("config.json: rms_norm_eps must be positive")
        for key in ("attn_logit_softcapping", "final_logit_softcapping"):
            v = getattr(self, key)
            if v is not None and not v > 0:
                raise ConfigError(f"config.json: '{key}' must be positive when given")

    def to_dict(self):
        """config.json content that ``from_dict`` reads back to an equal configuration."""
        d = asdict(self)
        factor = d.pop("rope_scaling_factor")
        if factor != 1.0:
            d["rope_scaling"] = {"rope_type": "linear", "factor": factor}
        d = {k: v for k, v in d.items() if v is not None}
        d["architectures"] = [ARCHITECTURE]
        d["model_type"] = MODEL_TYPE
        return d

    # ---- derived ---------------------------------------------------------------------------

    def score_multiplier(self):
        """1/sqrt(s) for s > 1, s itself otherwise, 1/sqrt(head_dim) when the key is absent
        (src/model/config.rs:291-294, src/transformer/forward.rs:583-585)."""
        s = self.query_pre_attn_scalar
        if s is None:
            return 1.0 / math.sqrt(self.head_dim)
        return 1.0 / math.sqrt(s) if s > 1.0 else s

    def layer_window(self, layer):
        """Even layers slide, odd layers see everything (src/transformer/forward.rs:574-582)."""
        return self.sliding_window if layer % 2 == 0 else None

    def model_info(self):
        """The keys of the reference's ``model_info()`` (src/python.rs:124-140)."""
        info = {
            "architecture": MODEL_TYPE,
            "context_length": self.max_position_embeddings,
            "embedding_length": self.hidden_size,
            "block_count": self.num_hidden_layers,
            "head_count": self.num_attention_heads,
            "head_count_kv": self.num_key_value_heads,
            "vocab_size": self.vocab_size,
            "head_dim": self.head_dim,
        }
        if self.sliding_window is not None:
            info["sliding_window"] = self.sliding_window
        return info

    # ---- the model as data ------------------------------------------------------------------

    def model_spec(self):
        """Gemma 2 as parts: embedding times sqrt(hidden); per layer a (1+w) RMSNorm before and
        after attention and before and after the GeGLU feed-forward; final norm; tied head with
        a soft cap.  Tensor names are the HF ones the reference loads
        (src/transformer/weights.rs:179-313)."""
        norm = lambda name: PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps,
                                                  "unit_offset": True}, {"weight": name})
        blocks = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            rope = PartSpec("rope", {"head_dim": self.head_dim, "rotary_dim": self.head_dim,
                                     "theta": self.rope_theta, "factor": self.rope_scaling_factor})
            mixer = PartSpec("attention", {
                "hidden_size": self.hidden_size, "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
                "score_multiplier": self.score_multiplier(), "softcap": self.attn_logit_softcapping,
                "window": self.layer_window(i), "position": rope,
            }, {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
                "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight"})
            ffn = PartSpec("gated", {
                "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
                "activation": _ACTIVATIONS[self.hidden_activation],
            }, {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                "down": p + "mlp.down_proj.weight"})
            blocks.append(BlockSpec(
                mixer=mixer, feed_forward=ffn,
                pre_mixer_norm=norm(p + "input_layernorm.weight"),
                post_mixer_norm=norm(p + "post_attention_layernorm.weight"),
                pre_ffn_norm=norm(p + "pre_feedforward_layernorm.weight"),
                post_ffn_norm=norm(p + "post_feedforward_layernorm.weight")))
        spec = ModelSpec(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab_size, hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                             "scale": math.sqrt(float(self.hidden_size))},
                               {"table": "model.embed_tokens.weight"}),
            blocks=blocks,
            run_order=[LayerCall(i) for i in range(self.num_hidden_layers)],
            final_norm=norm("model.norm.weight"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                      "softcap": self.final_logit_softcapping,
                                      "tie": self.tie_word_embeddings},
                          {"weight": "lm_head.weight", "tied_to": "model.embed_tokens.weight"}),
            bos_token_id=self.bos_token_id, eos_token_id=self.eos_token_id,
            info=self.model_info())
        spec.validate()
        return spec
