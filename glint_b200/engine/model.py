"""A causal language model put together from a ``ModelSpec``.

The forward pass is the reference's order of work (src/transformer/forward.rs:450-522):
embedding, the layers of the run order, final norm and output head at the wanted rows only
(the reference computes the head for every prompt position and keeps the last, :1045-1064,
:715-718).  Which layer runs when, and whose cache it reads, is the spec's ``run_order``.
"""
from __future__ import annotations

from ..parts import build_block, build_part


class CausalLM:
    def __init__(self, spec, rt):
        spec.validate()
        self.spec = spec
        self.rt = rt
        self.embedding = build_part("embedding", spec.embedding, rt)
        self.blocks = [build_block(b, rt) for b in spec.blocks]
        self.final_norm = build_part("norm", spec.final_norm, rt)
        self.head = build_part("head", spec.head, rt)
        self.run_order = list(spec.run_order)

    # ---- weights ------------------------------------------------------------------------------

    def parts(self):
        out = [self.embedding]
        for b in self.blocks:
            out.extend(b.parts())
        if self.final_norm is not None:
            out.append(self.final_norm)
        out.append(self.head)
        return out

    def needs(self):
        """Every tensor the model reads from the weight file, once per name."""
        seen = {}
        for part in self.parts():
            for need in part.needs():
                old = seen.get(need.name)
                if old is None:
                    seen[need.name] = need
                elif tuple(old.shape) != tuple(need.shape):
                    raise ValueError(f"tensor '{need.name}' is wanted with shapes {old.shape} and {need.shape}")
                elif old.optional and not need.optional:
                    seen[need.name] = need
        return list(seen.values())

    def bind(self, tensors):
        for part in self.parts():
            part.bind(tensors)

    def parameter_bytes(self):
        """Bytes of weights one step reads: every block as often as the run order names it."""
        total = self.head.parameter_bytes()
        if self.final_norm is not None:
            total += self.final_norm.parameter_bytes()
        for call in self.run_order:
            total += sum(p.parameter_bytes() for p in self.blocks[call.layer].parts())
        return total

    def flops(self, portions, logit_rows=1):
        """Floating-point operations of one step that runs ``portions`` = [(start, n)] (``n`` tokens of
        a request that has ``start`` tokens cached) and computes ``logit_rows`` rows of logits: the
        parts' matrix products and their mixers' work over the cache."""
        tokens = sum(n for _, n in portions)
        total = self.head.flops(logit_rows)
        for call in self.run_order:
            for p in self.blocks[call.layer].parts():
                total += p.flops(tokens)
                total += sum(p.attention_flops(start, n) for start, n in portions)
        return total

    def decode_read_bytes(self, positions, element_size):
        """Bytes a step of one token per request has to read: every weight once, and what each
        request's mixers read of the cache (the tokens stand at ``positions``)."""
        total = self.parameter_bytes()
        for call in self.run_order:
            for p in self.blocks[call.layer].parts():
                total += sum(p.cache_read_bytes(pos, element_size) for pos in positions)
        return total

    # ---- cache --------------------------------------------------------------------------------

    def cache_needs(self):
        """Per run-order entry: the mixer's declaration, and the entry whose cache it reads."""
        needs = [self.blocks[c.layer].cache_need() for c in self.run_order]
        return needs, [c.cache_of for c in self.run_order]

    # ---- forward ------------------------------------------------------------------------------

    def forward(self, ctx, cache):
        """Run the step's tokens; return float32 logits [len(ctx.logit_rows), vocab], or ``None``
        when no row is wanted."""
        x = self.embedding.forward(ctx.token_ids, ctx)
        normed = None
        n = len(self.run_order)
        for i, call in enumerate(self.run_order):
            block = self.blocks[call.layer]
            last = i + 1 == n
            next_norm = None if last else self.blocks[self.run_order[i + 1].layer].entry_norm()
            normed = block.forward(x, normed, ctx, cache.views[i], cache.states[i], next_norm,
                                   want_next=next_norm is not None)
        if ctx.num_logit_rows == 0:
            return None
        if self.final_norm is not None:
            rows = self.final_norm.forward(x, row_index=ctx.logit_rows)
        else:
            rows = x.index_select(0, ctx.logit_rows.long()).to(self.rt.dtype)
        return self.head.forward(rows, ctx)
