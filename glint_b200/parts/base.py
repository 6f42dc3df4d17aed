"""What every part is: a class built from its sizes and constants, that names the tensors it
needs and later receives them.  No part knows which model it is in.

Interfaces (``ctx`` is the step's ``StepContext``; activations are [tokens, size]):

* norm:          ``forward(x_f32, out=None, row_index=None) -> normalized (activation dtype)``;
                 ``triple()`` -> (weight, eps, offset) for fused add+norm kernels, or ``None``
* position:      ``encode_and_store(qkv_f32, ctx, q_out, view, nh, nkv, hd)``
* mixer:         ``cache_need() -> a cache declaration or None``;
                 ``forward(normed, ctx, view, state) -> float32 [tokens, hidden]``
* feed-forward:  ``forward(normed, ctx) -> float32 [tokens, hidden]``
* embedding:     ``forward(token_ids, ctx) -> float32 [tokens, hidden]``
* head:          ``forward(normed_rows, ctx) -> float32 logits [rows, vocab]``

``forward`` runs at once on tensors.  A part may also offer ``lower(prog, ...)``, which describes the same
work as operations of a ``glint_b200.native.Program`` on its ``Value`` objects; a model whose parts all
offer it runs a whole step with one call into the native executor, and a part without it runs through
``forward`` between two native stretches.  The package's parts implement ``forward`` by lowering
themselves into a short program and running it (``run_lowered``): one description of the work serves both.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class TensorNeed:
    """One tensor of the weight file: ``kind`` is 'matrix' (kept in the engine's dtype),
    'vector' (kept in 32-bit: norms) or 'int' (kept as int32)."""
    name: str
    shape: tuple
    kind: str = "matrix"
    optional: bool = False


class Part:
    """Base of all parts.  ``spec.tensors`` maps the part's roles to file names."""

    def __init__(self, rt, params, tensors):
        self.rt = rt
        self.params = dict(params)
        self.names = dict(tensors)

    def needs(self):
        return []

    def bind(self, tensors):
        """Receive the loaded tensors (by file name) once, on the device."""

    # ---- accounting (rooflines): each part answers for itself, so that a measurement needs no
    # knowledge of the architecture ----------------------------------------------------------------

    def parameter_bytes(self):
        """Bytes of weights this part reads in one step."""
        return 0

    def flops(self, tokens):
        """Floating-point operations of this part's matrix products for ``tokens`` tokens."""
        return 0

    def attention_flops(self, start, n):
        """Mixers: operations of scores and weighted values for ``n`` tokens at positions from ``start``."""
        return 0

    def cache_read_bytes(self, position, element_size):
        """Mixers: bytes of cache a single token at ``position`` has to read."""
        return 0


def run_lowered(rt, ctx, rows, lower):
    """Run ``lower(prog) -> Value`` at once for the step ``ctx``: a short program for ``rows`` tokens, run on
    the current stream; returns the first ``rows`` rows of the value it produced."""
    from ..native import Program
    prog = Program(rt, rows, ctx.groups)
    out = lower(prog)
    prog.run(ctx)
    return out.rows(rows)
