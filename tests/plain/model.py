"""Plain, slow Gemma 2 forward pass: the yardstick every engine test compares with.

It rests on the formulas of HamadAndrabi/glint's CPU forward pass, restated
here by reading its Rust sources: the reference is a Rust crate, no Rust
toolchain exists in this environment, so it was never compiled or run and no
output of it could be recorded under ``tests/golden``.  Each function cites
the reference file and lines it restates.

Whole sequences, no cache, one function per part.  It shares no code with the
``glint_b200`` package: it reads ``config.json`` with ``json``, the weights
with the ``safetensors`` library, and computes with torch on the CPU in the
dtype given (float32 as the reference does, or float64 for error budgets).
"""
from __future__ import annotations

import json
import math
import os

import torch


# ----------------------------------------------------------------------------
# files
# ----------------------------------------------------------------------------

def read_config(model_dir):
    """config.json keys as the reference reads them (src/model/config.rs:180-341).

    Defaults: num_key_value_heads = heads (:231); rms_norm_eps 1e-5 (:307);
    rope_theta 10000 at use (src/transformer/forward.rs:539); head_dim =
    hidden/heads unless given (:131-134); the caps disable when absent;
    ``query_pre_attn_scalar`` s becomes the multiplier 1/sqrt(s) when s > 1,
    else s itself (:291-294); absent, the multiplier is 1/sqrt(head_dim)
    (src/transformer/forward.rs:583-585).
    """
    with open(os.path.join(model_dir, "config.json")) as f:
        raw = json.load(f)
    c = {}
    c["hidden"] = int(raw["hidden_size"])
    c["layers"] = int(raw["num_hidden_layers"])
    c["heads"] = int(raw["num_attention_heads"])
    c["kv_heads"] = int(raw.get("num_key_value_heads", c["heads"]))
    c["head_dim"] = int(raw.get("head_dim", c["hidden"] // c["heads"]))
    c["vocab"] = int(raw["vocab_size"])
    c["eps"] = float(raw.get("rms_norm_eps", 1e-5))
    c["theta"] = float(raw.get("rope_theta", 10000.0))
    window = raw.get("sliding_window")
    if raw.get("use_sliding_window") is False or not window:
        window = None
    c["window"] = window
    c["attn_cap"] = raw.get("attn_logit_softcapping")
    c["final_cap"] = raw.get("final_logit_softcapping")
    s = raw.get("query_pre_attn_scalar")
    if s is None:
        c["scale"] = 1.0 / math.sqrt(c["head_dim"])
    else:
        s = float(s)
        c["scale"] = 1.0 / math.sqrt(s) if s > 1.0 else s
    rs = raw.get("rope_scaling")
    c["rope_factor"] = float(rs["factor"]) if rs and rs.get("rope_type", rs.get("type", "linear")) == "linear" else 1.0
    c["tie"] = bool(raw.get("tie_word_embeddings", False))
    return c


def read_weights(model_dir, dtype=torch.float32):
    """All tensors of model.safetensors widened to ``dtype``.

    The reference widens every stored weight exactly to f32 before use
    (src/tensor/quantized.rs:1021-1044, src/tensor/dequantize.rs:65-74).
    """
    from safetensors.torch import load_file

    tensors = load_file(os.path.join(model_dir, "model.safetensors"))
    return {k: v.to(dtype) for k, v in tensors.items()}


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------

def embed(table, tokens, hidden):
    """Row lookup times sqrt(hidden) in 32-bit (src/transformer/forward.rs:73-83)."""
    scale = torch.tensor(math.sqrt(float(hidden)), dtype=torch.float32).to(table.dtype)
    return table[torch.as_tensor(tokens, dtype=torch.long)] * scale


def rms_norm(x, w, eps):
    """x * 1/sqrt(mean(x^2) + eps) * (1 + w)  (src/tensor/ops.rs:134-152)."""
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    r = 1.0 / torch.sqrt(mean_sq + eps)
    return x * r * (1.0 + w)


def permute_qk_rows(w, n_heads, head_dim):
    """new[2j+a] = old[a*half + j] inside each head (src/transformer/weights.rs:504-530)."""
    half = head_dim // 2
    out = w.clone()
    for h in range(n_heads):
        base = h * head_dim
        for j in range(half):
            for a in range(2):
                out[base + 2 * j + a] = w[base + a * half + j]
    return out


def rope_adjacent(x, positions, head_dim, theta, factor=1.0):
    """Adjacent pairs (2j, 2j+1) rotate by pos/factor * theta^(-2j/head_dim)
    (src/tensor/ops.rs:212-245).  ``x`` is [T, n*head_dim], permuted rows."""
    T = x.shape[0]
    xs = x.reshape(T, -1, head_dim // 2, 2)
    i = torch.arange(0, head_dim, 2, dtype=torch.float32)
    freq = (1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), i / head_dim)).to(x.dtype)
    pos = (torch.as_tensor(positions, dtype=torch.float32) / factor).to(x.dtype)
    ang = pos[:, None] * freq[None, :]
    cos = torch.cos(ang)[:, None, :]
    sin = torch.sin(ang)[:, None, :]
    x0, x1 = xs[..., 0], xs[..., 1]
    out = torch.stack((x0 * cos - x1 * sin, x0 * sin + x1 * cos), dim=-1)
    return out.reshape(T, -1)


def softcap(x, cap):
    """cap * tanh(x / cap) (src/tensor/ops.rs:98-103, src/tensor/flash.rs:82-85)."""
    if cap is None:
        return x
    return cap * torch.tanh(x / cap)


def attention(n, lw, c, layer_idx):
    """Causal attention of a whole sequence starting at position 0.

    q/k/v products without bias (src/transformer/forward.rs:546-557), RoPE on q
    and k (:569-570), group h -> h // (heads/kv_heads) (:255), scores times the
    multiplier then the cap (src/tensor/flash.rs:76-87), softmax and weighted
    sum of values (src/transformer/forward.rs:203-225), keys of position p from
    max(0, p-W+1) on even layers and from 0 on odd ones (:574-582).
    """
    T = n.shape[0]
    nh, nkv, hd = c["heads"], c["kv_heads"], c["head_dim"]
    wq = permute_qk_rows(lw["q"], nh, hd)
    wk = permute_qk_rows(lw["k"], nkv, hd)
    q = n @ wq.T
    k = n @ wk.T
    v = n @ lw["v"].T
    pos = list(range(T))
    q = rope_adjacent(q, pos, hd, c["theta"], c["rope_factor"]).reshape(T, nh, hd)
    k = rope_adjacent(k, pos, hd, c["theta"], c["rope_factor"]).reshape(T, nkv, hd)
    v = v.reshape(T, nkv, hd)
    sliding = c["window"] is not None and layer_idx % 2 == 0
    out = torch.zeros(T, nh, hd, dtype=n.dtype)
    group = nh // nkv
    for p in range(T):
        start = max(0, p - c["window"] + 1) if sliding else 0
        for h in range(nh):
            g = h // group
            s = (k[start:p + 1, g] @ q[p, h]) * c["scale"]
            s = softcap(s, c["attn_cap"])
            w = torch.softmax(s, dim=0)
            out[p, h] = w @ v[start:p + 1, g]
    return out.reshape(T, nh * hd) @ lw["o"].T


def gelu_tanh(x):
    """0.5 x (1 + tanh(0.7978846 (x + 0.044715 x^3))) (src/tensor/ops.rs:169-178)."""
    return 0.5 * x * (1.0 + torch.tanh(0.7978846 * (x + 0.044715 * x * x * x)))


def feed_forward(f, lw):
    """down(gelu(gate f) * (up f)) (src/transformer/forward.rs:273-318)."""
    return (gelu_tanh(f @ lw["gate"].T) * (f @ lw["up"].T)) @ lw["down"].T


def layer_weights(w, i):
    p = f"model.layers.{i}."
    return {
        "in_norm": w[p + "input_layernorm.weight"],
        "post_attn_norm": w[p + "post_attention_layernorm.weight"],
        "pre_ffn_norm": w[p + "pre_feedforward_layernorm.weight"],
        "post_ffn_norm": w[p + "post_feedforward_layernorm.weight"],
        "q": w[p + "self_attn.q_proj.weight"],
        "k": w[p + "self_attn.k_proj.weight"],
        "v": w[p + "self_attn.v_proj.weight"],
        "o": w[p + "self_attn.o_proj.weight"],
        "gate": w[p + "mlp.gate_proj.weight"],
        "up": w[p + "mlp.up_proj.weight"],
        "down": w[p + "mlp.down_proj.weight"],
    }


def block(x, lw, c, layer_idx):
    """norm, attention, norm, add; norm, feed-forward, norm, add
    (src/transformer/forward.rs:103-122 and :473-503)."""
    a = x + rms_norm(attention(rms_norm(x, lw["in_norm"], c["eps"]), lw, c, layer_idx),
                     lw["post_attn_norm"], c["eps"])
    d = rms_norm(feed_forward(rms_norm(a, lw["pre_ffn_norm"], c["eps"]), lw),
                 lw["post_ffn_norm"], c["eps"])
    return a + d


def forward(c, w, tokens, positions=None):
    """Logits [T, vocab] of one whole sequence from position 0, or only the rows at ``positions``.

    Final norm, the tied (or separate) output matrix and the final cap
    (src/transformer/forward.rs:516-520, src/transformer/weights.rs:315-319); the reference also
    computes the head for the positions it keeps only (:1045-1064).
    """
    x = embed(w["model.embed_tokens.weight"], tokens, c["hidden"])
    for i in range(c["layers"]):
        x = block(x, layer_weights(w, i), c, i)
    if positions is not None:
        x = x[torch.as_tensor(list(positions), dtype=torch.long)]
    y = rms_norm(x, w["model.norm.weight"], c["eps"])
    head = w["model.embed_tokens.weight"] if (c["tie"] or "lm_head.weight" not in w) else w["lm_head.weight"]
    return softcap(y @ head.T, c["final_cap"])


def logits_of(model_dir, tokens, dtype=torch.float32):
    """Convenience: read a model folder and run one sequence."""
    c = read_config(model_dir)
    w = read_weights(model_dir, dtype)
    return forward(c, w, tokens).to(torch.float32)
