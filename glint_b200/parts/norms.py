"""Root-mean-square norm: x * rsqrt(mean(x^2) + eps) * (offset + w).

``unit_offset`` True is the Gemma form with (1 + w) (src/tensor/ops.rs:134-152); False is the
plain form (src/tensor/ops.rs:109-128).  Statistics and the product are 32-bit.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorNeed
from .registry import register_part


class RMSNorm(Part):
    def __init__(self, rt, params, tensors):
        super().__init__(rt, params, tensors)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.offset = 1.0 if params.get("unit_offset", False) else 0.0
        self.weight = None

    def needs(self):
        return [TensorNeed(self.names["weight"], (self.size,), "vector")]

    def bind(self, tensors):
        self.weight = tensors[self.names["weight"]]

    def triple(self):
        return (self.weight, self.eps, self.offset)

    def lower(self, prog, x, out, logit_rows=False):
        """out = norm(x) as an operation of ``prog``; with ``logit_rows`` of the step's wanted rows only."""
        prog.rmsnorm(x, self.weight, self.eps, self.offset, out, logit_rows)
        return out

    def forward(self, x, out=None, row_index=None):
        rows = x.shape[0] if row_index is None else row_index.shape[0]
        if out is None:
            out = torch.empty((rows, self.size), dtype=self.rt.dtype, device=x.device)
        ops.rmsnorm(x, self.weight, out, self.eps, self.offset, row_index)
        return out

    def parameter_bytes(self):
        return self.size * 4


register_part("norm", "rmsnorm", RMSNorm)
