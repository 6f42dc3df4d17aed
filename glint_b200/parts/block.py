"""One layer: mixer and feed-forward, each between optional norms, around a 32-bit residual.

    x = x + post_mixer_norm(mixer(pre_mixer_norm(x)))
    x = x + post_ffn_norm(feed_forward(pre_ffn_norm(x)))

which is the reference's layer with its four Gemma 2 norms
(src/transformer/forward.rs:103-122, :473-503); a norm that is absent is the identity, which
gives the usual pre-norm layer.  The residual sum is float32 in every dtype.  The add, the norm
after a part and the norm before the next part run as one kernel when the norms offer their
(weight, eps, offset) triple; ``next_norm`` is the norm that the following layer would apply
first, so that its result can leave this layer already computed.
"""
from __future__ import annotations

import torch

from .registry import build_part, register_part


def _triple(norm):
    return None if norm is None else norm.triple()


def _fusable(*norms):
    return all(n is None or hasattr(n, "triple") for n in norms)


def lower_norm(prog, norm, x, role):
    """``norm(x)`` in the activation dtype as a value of ``role``: the norm's own operation, or, for a norm
    that is not lowered (or no norm at all: a cast), its ``forward`` between the native operations."""
    out = prog.value(role, x.width)
    if norm is not None and hasattr(norm, "lower"):
        return norm.lower(prog, x, out)
    if norm is None:
        prog.host(lambda ctx: out.rows(ctx.num_tokens).copy_(x.rows(ctx.num_tokens)))
    else:
        prog.host(lambda ctx: norm.forward(x.rows(ctx.num_tokens), out=out.rows(ctx.num_tokens)))
    return out


def lower_mixer(prog, mixer, normed, view, state, hidden):
    """The mixer's result as a value float32 [tokens, hidden]: its own operations, or its ``forward``."""
    if hasattr(mixer, "lower"):
        return mixer.lower(prog, normed, view, state)
    y = prog.value("mixer.y", hidden, torch.float32)
    prog.host(lambda ctx: y.rows(ctx.num_tokens).copy_(mixer.forward(normed.rows(ctx.num_tokens), ctx, view, state)))
    return y


def lower_feed_forward(prog, ffn, normed, hidden):
    if hasattr(ffn, "lower"):
        return ffn.lower(prog, normed)
    y = prog.value("ffn.y", hidden, torch.float32)
    prog.host(lambda ctx: y.rows(ctx.num_tokens).copy_(ffn.forward(normed.rows(ctx.num_tokens), ctx)))
    return y


class Block:
    """The ``"sandwich"`` arrangement.  What the model asks of any block kind: ``parts()``,
    ``cache_need()``, ``entry_norm()`` (the norm it applies to the residual first, or ``None``; the
    block before it may hand its result in as ``normed``) and ``forward``; optionally ``lower``."""

    def __init__(self, rt, spec):
        self.rt = rt
        self.spec = spec
        self.mixer = build_part("mixer", spec.mixer, rt)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, rt)
        self.pre_mixer_norm = build_part("norm", spec.pre_mixer_norm, rt)
        self.post_mixer_norm = build_part("norm", spec.post_mixer_norm, rt)
        self.pre_ffn_norm = build_part("norm", spec.pre_ffn_norm, rt)
        self.post_ffn_norm = build_part("norm", spec.post_ffn_norm, rt)

    def parts(self):
        return [p for p in (self.mixer, getattr(self.mixer, "position", None), self.feed_forward,
                            self.pre_mixer_norm, self.post_mixer_norm, self.pre_ffn_norm, self.post_ffn_norm)
                if p is not None]

    def cache_need(self):
        """What the layer keeps per request between steps: its mixer's declaration."""
        return self.mixer.cache_need()

    def entry_norm(self):
        return self.pre_mixer_norm

    def _add_then_norm(self, prog, x, y, post_norm, next_norm, want_next):
        """x += post_norm(y); returns the value next_norm(x) in the activation dtype when wanted."""
        if _fusable(post_norm, next_norm):
            out = prog.value("block.normed", x.width) if want_next else None
            prog.add_rmsnorm(x, y, _triple(post_norm), out, _triple(next_norm) if want_next else None)
            return out
        if post_norm is not None:
            normed_y = prog.value("block.post", x.width, torch.float32)
            prog.host(lambda ctx: normed_y.rows(ctx.num_tokens).copy_(post_norm.forward(y.rows(ctx.num_tokens))))
            y = normed_y
        prog.add_rmsnorm(x, y, None, None, None)
        return lower_norm(prog, next_norm, x, "block.normed") if want_next else None

    def lower(self, prog, x, normed, view, state, next_norm=None, want_next=False):
        """The layer as operations of ``prog``: updates the residual value ``x`` in place.  ``normed`` is the
        value ``pre_mixer_norm(x)`` if the caller has it already.  Returns the value ``next_norm(x)`` when
        ``want_next``."""
        if normed is None:
            normed = lower_norm(prog, self.pre_mixer_norm, x, "block.normed")
        y = lower_mixer(prog, self.mixer, normed, view, state, x.width)
        n2 = self._add_then_norm(prog, x, y, self.post_mixer_norm, self.pre_ffn_norm, True)
        d = lower_feed_forward(prog, self.feed_forward, n2, x.width)
        return self._add_then_norm(prog, x, d, self.post_ffn_norm, next_norm, want_next)

    def forward(self, x, normed, ctx, view, state, next_norm=None, want_next=False):
        """Update the residual tensor ``x`` in place, at once.  Returns ``next_norm(x)`` when ``want_next``."""
        def lower(prog):
            given = None if normed is None else prog.bind(normed)
            return self.lower(prog, prog.bind(x), given, view, state, next_norm, want_next)
        from ..native import Program
        prog = Program(self.rt, x.shape[0], ctx.groups)
        out = lower(prog)
        prog.run(ctx)
        return None if out is None else out.rows(x.shape[0])


register_part("block", "sandwich", Block)
