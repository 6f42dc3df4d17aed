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

    def encode_and_store(self, qkv, ctx, q_out, view, nh, nkv, hd):
        """Rotate q and k of ``qkv``; q goes to ``q_out``; k and v go into the pages of ``view``
        (only q when the view does not write)."""
        writes = view.writes
        ops.rope_kv_write(qkv, ctx.positions, ctx.token_seq, ctx.block_table(view.group), self.inv_freq,
                          self.factor, self.rotary_dim, q_out, view.k if writes else None,
                          view.v if writes else None, nh, nkv, hd, view.page_size, view.num_pages,
                          self.rt.status)

    def angles(self, ctx):
        """(cos, sin) of every token's angles, float32 [tokens, rotary_dim / 2, 2]; computed by the first
        layer of a step that asks and shared through ``ctx.memo`` by all layers with these parameters."""
        key = ("rope_table", self.theta, self.factor, self.rotary_dim, self.head_dim)
        table = ctx.memo.get(key)
        if table is None:
            table = torch.empty((ctx.num_tokens, self.rotary_dim // 2, 2), dtype=torch.float32, device=self.rt.device)
            ops.rope_table(ctx.positions, self.inv_freq, self.factor, table)
            ctx.memo[key] = table
        return table

    def project_encode_store(self, x, w_qkv, ctx, q_out, view, nh, nkv, hd):
        """The q/k/v product, the rotation and the cache write as one kernel, where there is one for
        these sizes in bfloat16 (the weight-streaming kernel for a few single tokens, the tiled kernel
        for heads in steps of 256); returns False when the caller has to run the product and
        ``encode_and_store`` itself."""
        rt = self.rt
        if not (rt.tensor_cores and w_qkv.dtype == torch.bfloat16 and x.dtype == torch.bfloat16):
            return False
        from .. import ops_tensor
        writes = view.writes
        k, v = (view.k, view.v) if writes else (None, None)
        table = ctx.block_table(view.group)
        if ops_tensor.qkv_rope_supported(x.shape[0], x.shape[1], hd, self.rotary_dim):
            ops_tensor.qkv_rope(x, w_qkv, ctx.positions, ctx.token_seq, table, self.inv_freq, self.factor, q_out,
                                k, v, nh, nkv, hd, view.page_size, view.num_pages, rt.status)
            return True
        if ops_tensor.qkv_rope_tiled_supported(x.shape[0], x.shape[1], hd, self.rotary_dim,
                                               nh + 2 * nkv if writes else nh):
            ops_tensor.qkv_rope_tiled(x, w_qkv, self.angles(ctx), ctx.positions, ctx.token_seq, table, q_out, k, v,
                                      nh, nkv, hd, view.page_size, view.num_pages, rt.status)
            return True
        return False


register_part("position", "rope", Rotary)
