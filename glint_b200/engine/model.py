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
        self._programs = {}           # per cache manager: (program, logits tensor, the cache)

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

    def lower(self, prog, cache, logit_capacity):
        """The whole forward pass as operations of ``prog``: embedding, the layers of the run order with
        the cache views and state tensors of ``cache``, final norm and output head at the wanted rows.
        A part or a block kind that offers no ``lower`` runs through its ``forward`` between the native
        operations.  Returns the logits as a [logit_capacity, vocab] float32 tensor."""
        import torch
        from ..native import Value
        rt = self.rt
        H = self.spec.hidden_size
        if hasattr(self.embedding, "lower"):
            x = self.embedding.lower(prog)
        else:
            x = prog.value("embedding.x", H, torch.float32)
            emb = self.embedding
            prog.host(lambda ctx: x.rows(ctx.num_tokens).copy_(emb.forward(ctx.token_ids, ctx)))
        normed = None
        n = len(self.run_order)
        for i, call in enumerate(self.run_order):
            block = self.blocks[call.layer]
            next_norm = None if i + 1 == n else self.blocks[self.run_order[i + 1].layer].entry_norm()
            view, state = cache.views[i], cache.states[i]
            if hasattr(block, "lower"):
                normed = block.lower(prog, x, normed, view, state, next_norm, next_norm is not None)
            else:
                normed = self._host_block(prog, block, x, normed, view, state, next_norm)
        rows = Value(rt.buffer("head.rows", (logit_capacity, H)))
        if self.final_norm is not None and hasattr(self.final_norm, "lower"):
            self.final_norm.lower(prog, x, rows, logit_rows=True)
        else:
            norm = self.final_norm

            def gather(ctx):
                r = rows.rows(ctx.num_logit_rows)
                if norm is not None:
                    norm.forward(x.rows(ctx.num_tokens), out=r, row_index=ctx.logit_rows)
                else:
                    r.copy_(x.rows(ctx.num_tokens).index_select(0, ctx.logit_rows.long()))
            prog.host(gather)
        logits = Value(rt.buffer("head.logits", (logit_capacity, self.spec.vocab_size), torch.float32))
        if hasattr(self.head, "lower"):
            self.head.lower(prog, rows, logits)
        else:
            head = self.head
            prog.host(lambda ctx: logits.rows(ctx.num_logit_rows).copy_(head.forward(rows.rows(ctx.num_logit_rows), ctx)))
        return logits.tensor

    @staticmethod
    def _host_block(prog, block, x, normed, view, state, next_norm):
        """A block kind without ``lower``: its ``forward`` between the native operations."""
        want_next = next_norm is not None
        out = prog.value("block.normed", x.width) if want_next else None
        given = normed

        def run(ctx):
            T = ctx.num_tokens
            got = block.forward(x.rows(T), None if given is None else given.rows(T), ctx, view, state, next_norm, want_next)
            if want_next:
                out.rows(T).copy_(got)
        prog.host(run)
        return out

    def program(self, cache, tokens, logit_rows):
        """The lowered program for ``cache`` with room for a step of ``tokens`` tokens and ``logit_rows``
        wanted rows: (program, logits tensor, whether it was built anew, in which case launches captured
        earlier point into memory that is no longer used)."""
        from ..native import Program
        entry = self._programs.get(id(cache))
        fresh = False
        if entry is None or entry[0].capacity < tokens or entry[1].shape[0] < logit_rows:
            capacity = max(tokens, 2 * entry[0].capacity if entry is not None and entry[0].capacity < tokens else 0,
                           entry[0].capacity if entry is not None else 0, 64)
            rows_cap = max(logit_rows, entry[1].shape[0] if entry is not None else 0, min(64, capacity))
            prog = Program(self.rt, capacity, cache.groups)
            logits = self.lower(prog, cache, rows_cap)
            entry = self._programs[id(cache)] = (prog, logits, cache)
            fresh = True
        return entry[0], entry[1], fresh

    def forward(self, ctx, cache):
        """Run the step's tokens; return float32 logits [len(ctx.logit_rows), vocab], or ``None``
        when no row is wanted."""
        prog, logits, _ = self.program(cache, ctx.num_tokens, ctx.num_logit_rows)
        prog.run(ctx)
        if ctx.num_logit_rows == 0:
            return None
        return logits[:ctx.num_logit_rows]
