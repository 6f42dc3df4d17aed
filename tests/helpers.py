"""Shared by the tests: the tiny configurations, model folders in temporary places, tolerances."""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two tiny Gemma 2 configurations that differ in every size and option.
TINY_A = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 512, "rope_theta": 10000.0,
    "sliding_window": 16, "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0,
    "query_pre_attn_scalar": 16, "rms_norm_eps": 1e-6, "max_position_embeddings": 128,
    "tie_word_embeddings": True, "hidden_activation": "gelu_pytorch_tanh",
}
TINY_A_INIT = {"seed": 0, "std": 0.02, "norm_std": 0.1}

TINY_B = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 5, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 320, "vocab_size": 1000, "rope_theta": 100000.0,
    "sliding_window": 8, "attn_logit_softcapping": 20.0, "final_logit_softcapping": 15.0,
    "query_pre_attn_scalar": 16, "rms_norm_eps": 1e-5, "max_position_embeddings": 256,
    "tie_word_embeddings": True, "hidden_activation": "gelu_pytorch_tanh",
}
TINY_B_INIT = {"seed": 1, "std": 0.05, "norm_std": 0.2}

# A third shape for longer sequences: odd sizes, head_dim 48, 3 query heads per kv head.
TINY_C = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 3, "hidden_size": 80, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 48, "intermediate_size": 176, "vocab_size": 777, "rope_theta": 50000.0,
    "sliding_window": 40, "attn_logit_softcapping": 30.0, "final_logit_softcapping": 25.0,
    "query_pre_attn_scalar": 48, "rms_norm_eps": 1e-6, "max_position_embeddings": 1024,
    "tie_word_embeddings": False, "hidden_activation": "gelu_pytorch_tanh",
}
TINY_C_INIT = {"seed": 5, "std": 0.06, "norm_std": 0.15}

TINY = {"A": (TINY_A, TINY_A_INIT), "B": (TINY_B, TINY_B_INIT), "C": (TINY_C, TINY_C_INIT)}

# Largest |difference| of logits against the plain implementation that a test accepts.
# float32: both sides compute in 32-bit and only the order of summation differs; measured 3e-6 at
# most on these models.  bfloat16: activations are rounded to 8 bits of mantissa between
# products; measured 0.5 to 0.9 % of the largest |logit|; the bound is relative to that size.
TOL = {"float32": 2e-5, "bfloat16": 0.025}


def tolerance(dtype, reference):
    """Absolute bound for ``dtype`` given the reference logits it is compared with."""
    if dtype == "float32":
        return TOL["float32"]
    return TOL["bfloat16"] * float(np.abs(reference).max())


def make_model_dir(tmp_path, name, untied_head=None):
    from glint_b200.weights import write_random_model
    cfg, init = TINY[name]
    out = os.path.join(str(tmp_path), f"tiny_{name}")
    if untied_head is None:
        untied_head = not cfg["tie_word_embeddings"]
    write_random_model(dict(cfg), out, untied_head=untied_head, **init)
    return out


def random_tokens(n, vocab, seed):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=n)]


def plain_logits(model_dir, tokens):
    from tests.plain import model as plain
    return plain.logits_of(model_dir, tokens).numpy()
