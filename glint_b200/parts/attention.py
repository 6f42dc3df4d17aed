"""Grouped-query attention over the paged cache.

q, k, v products without bias (src/transformer/forward.rs:546-557; the three matrices are
stacked into one at load, which is exact), position encoding of q and k, cache write
(:569-572), scores * multiplier then cap * tanh(score / cap) (src/tensor/flash.rs:76-87),
softmax and weighted values in 32-bit (:65-123), keys of a token at position p from
max(0, p - window + 1) to p, or from 0 without a window
(src/transformer/forward.rs:574-582), output product (:675).
"""
from __future__ import annotations

import torch

from ..cache import PagedKVNeed
from .base import Part, TensorNeed, run_lowered
from .registry import build_part, register_part


class Attention(Part):
    def __init__(self, rt, params, tensors):
        super().__init__(rt, params, tensors)
        p = params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.multiplier = float(p["score_multiplier"])
        self.softcap = p.get("softcap") or 0.0
        self.window = p.get("window") or None
        self.position = build_part("position", p["position"], rt)
        self.w_qkv = None
        self.w_o = None

    @property
    def q_size(self):
        return self.num_heads * self.head_dim

    @property
    def kv_size(self):
        return self.num_kv_heads * self.head_dim

    def cache_need(self):
        return PagedKVNeed(self.num_kv_heads, self.head_dim, self.window)

    def needs(self):
        n = self.names
        return [TensorNeed(n["q"], (self.q_size, self.hidden_size)),
                TensorNeed(n["k"], (self.kv_size, self.hidden_size)),
                TensorNeed(n["v"], (self.kv_size, self.hidden_size)),
                TensorNeed(n["o"], (self.hidden_size, self.q_size))]

    def bind(self, tensors):
        n = self.names
        self.w_qkv = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        self.w_o = tensors[n["o"]]

    def lower(self, prog, normed, view, state=None):
        """q/k/v product with the position encoding and the cache write, attention over the pages of
        ``view``, output product.  Returns the value float32 [tokens, hidden].  A position encoding
        that offers no ``lower`` runs through its ``encode_and_store`` between the native operations."""
        nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        q = prog.value("mixer.q", self.q_size)
        if hasattr(self.position, "lower"):
            self.position.lower(prog, normed, self.w_qkv, q, view, nh, nkv, hd)
        else:
            qkv = prog.value("mixer.qkv", self.w_qkv.shape[0], torch.float32)
            prog.linear(normed, self.w_qkv, qkv)
            position = self.position
            prog.host(lambda ctx: position.encode_and_store(qkv.rows(ctx.num_tokens), ctx, q.rows(ctx.num_tokens), view,
                                                            nh, nkv, hd))
        out = prog.value("mixer.out", self.q_size)
        prog.attention(q, view, out, nh, nkv, hd, self.multiplier, self.softcap, self.window)
        y = prog.value("mixer.y", self.w_o.shape[0], torch.float32)
        prog.linear(out, self.w_o, y)
        return y

    def forward(self, normed, ctx, view, state=None):
        return run_lowered(self.rt, ctx, normed.shape[0], lambda prog: self.lower(prog, prog.bind(normed), view, state))

    def parameter_bytes(self):
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_o.element_size()

    def flops(self, tokens):
        return 2 * tokens * (self.w_qkv.numel() + self.w_o.numel())

    def keys_read(self, start, n):
        """Keys that ``n`` tokens at positions ``start``.. read in all: position p reads p + 1 of them,
        or the last ``window``."""
        total = n * start + n * (n + 1) // 2
        if self.window is not None:
            over = max(0, start + n - self.window)          # positions whose p + 1 exceeds the window
            first = max(start, self.window)                 # the first such position
            k = start + n - first                           # how many there are
            if over > 0 and k > 0:
                total -= k * (first + 1 - self.window) + k * (k - 1) // 2
        return total

    def attention_flops(self, start, n):
        return 4 * self.num_heads * self.head_dim * self.keys_read(start, n)

    def cache_read_bytes(self, position, element_size):
        return self.keys_read(position, 1) * 2 * self.num_kv_heads * self.head_dim * element_size


register_part("mixer", "attention", Attention)
