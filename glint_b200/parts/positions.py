"""Rotary position encoding, applied where keys enter the cache.

Pair (j, j + rot/2) of a head turns by (pos / factor) * theta^(-2j/head_dim), all in 32-bit
(src/tensor/ops.rs:212-245).  The reference permutes the q/k rows at load and turns adjacent
pairs; that is the same rotation of the same pairs (src/transformer/weights.rs:473-530, test
:626-671), and q.k does not change under a permutation common to both, so the file's row
order is kept here.  Keys are cached after the rotation (src/transformer/forward.rs:569-572).
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .base import Part
from .registry import register_part


class Rotary(Part):
    def __init__(self, rt, params, tensors):
        super().__init__(rt, params, tensors)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim)) & ~1
        self.theta = float(params["theta"])
        self.factor = float(params.get("factor", 1.0))
        # freq_j = 1 / theta^(2j / head_dim) in 32-bit, as the reference computes it
        i = np.arange(0, self.rotary_dim, 2, dtype=np.float32)
        inv = np.float32(1.0) / np.power(np.float32(self.theta), i / np.float32(self.head_dim), dtype=np.float32)
        self.inv_freq = torch.from_numpy(inv.astype(np.float32)).to(rt.device)

    def lower(self, prog, x, w_qkv, q_out, view, nh, nkv, hd):
        """The q/k/v product of ``x``, the rotation of q and k, q into ``q_out``, k and v into the pages of
        ``view`` (only q when the view does not write), as one operation: the runtime takes one kernel
        where there is one for these sizes (the weight-streaming product for a few single tokens, the tiled
        product for heads in steps of 256, both with the rotation and the cache write in their epilogue) and
        else the product followed by the rotation kernel."""
        from ..native import TrigTable
        key = ("rope_table", self.theta, self.factor, self.rotary_dim, self.head_dim)
        trig = self.rt.shared.get(key)                # the step's table of angles, shared by all layers with these parameters
        if trig is None:
            trig = self.rt.shared[key] = TrigTable(self.rt, self.rotary_dim // 2)
        trig.reserve(prog.capacity)
        tmp = prog.value("mixer.qkv", w_qkv.shape[0], torch.float32)
        prog.qkv_rope(x, w_qkv, q_out, tmp, view, nh, nkv, hd, self.inv_freq, self.factor, self.rotary_dim, trig)

    def encode_and_store(self, qkv, ctx, q_out, view, nh, nkv, hd):
        """Rotate q and k of a finished product ``qkv``; q goes to ``q_out``; k and v go into the pages of
        ``view`` (only q when the view does not write)."""
        writes = view.writes
        ops.rope_kv_write(qkv, ctx.positions, ctx.token_seq, ctx.block_table(view.group), self.inv_freq,
                          self.factor, self.rotary_dim, q_out, view.k if writes else None,
                          view.v if writes else None, nh, nkv, hd, view.page_size, view.num_pages,
                          self.rt.status)


register_part("position", "rope", Rotary)
