"""Token embedding and the output head."""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorNeed
from .linear import linear
from .registry import register_part


class ScaledEmbedding(Part):
    """x = table[token] * scale in 32-bit (src/transformer/forward.rs:73-83)."""

    def __init__(self, rt, params, tensors):
        super().__init__(rt, params, tensors)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.scale = float(params.get("scale", 1.0))
        self.table = None

    def needs(self):
        return [TensorNeed(self.names["table"], (self.vocab_size, self.hidden_size), "matrix")]

    def bind(self, tensors):
        self.table = tensors[self.names["table"]]

    def lower(self, prog):
        """The residual stream of the step's tokens, float32 [tokens, hidden]."""
        out = prog.value("embedding.x", self.hidden_size, torch.float32)
        prog.embed(self.table, out, self.scale, self.vocab_size)
        return out

    def forward(self, token_ids, ctx):
        out = torch.empty((token_ids.shape[0], self.hidden_size), dtype=torch.float32, device=token_ids.device)
        ops.embed_scale(self.table, token_ids, out, self.scale, self.rt.status)
        return out

    def parameter_bytes(self):
        return 0  # a few rows per step


class LMHead(Part):
    """logits = W y, then cap * tanh(logits / cap) (src/transformer/forward.rs:516-520).  W is the
    embedding table when ``tie`` is set or the file has no head tensor
    (src/transformer/weights.rs:315-319)."""

    def __init__(self, rt, params, tensors):
        super().__init__(rt, params, tensors)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.softcap = params.get("softcap") or 0.0
        self.tie = bool(params.get("tie", False))
        self.weight = None

    def needs(self):
        shape = (self.vocab_size, self.hidden_size)
        return [TensorNeed(self.names["weight"], shape, "matrix", optional=True),
                TensorNeed(self.names["tied_to"], shape, "matrix")]

    def bind(self, tensors):
        own = tensors.get(self.names["weight"])
        self.weight = tensors[self.names["tied_to"]] if (self.tie or own is None) else own

    def lower(self, prog, rows, out):
        """Logits of the normalized ``rows`` (the step's wanted rows) into ``out`` [rows, vocab] float32."""
        prog.linear(rows, self.weight, out, cap=self.softcap, logit_rows=True)
        return out

    def forward(self, normed_rows, ctx):
        return linear(self.rt, normed_rows, self.weight, cap=self.softcap)

    def parameter_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def flops(self, rows):
        return 2 * rows * self.weight.numel()


register_part("embedding", "embedding", ScaledEmbedding)
register_part("head", "lm_head", LMHead)
