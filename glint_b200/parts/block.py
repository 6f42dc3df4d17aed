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

from .. import ops
from .registry import build_part, register_part


def _triple(norm):
    return None if norm is None else norm.triple()


def _fusable(*norms):
    return all(n is None or hasattr(n, "triple") for n in norms)


class Block:
    """The ``"sandwich"`` arrangement.  What the model asks of any block kind: ``parts()``,
    ``cache_need()``, ``entry_norm()`` (the norm it applies to the residual first, or ``None``; the
    block before it may hand its result in as ``normed``) and ``forward``."""

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

    def _enter(self, x, norm):
        if norm is not None:
            return norm.forward(x)
        return x if x.dtype == self.rt.dtype else x.to(self.rt.dtype)

    def _add_then_norm(self, x, y, post_norm, next_norm, want_next):
        """x += post_norm(y); returns next_norm(x) in the activation dtype when wanted."""
        out = self.rt.buffer("block.normed", tuple(x.shape)) if want_next else None
        if _fusable(post_norm, next_norm):
            ops.add_rmsnorm(x, y, _triple(post_norm), out, _triple(next_norm) if want_next else None)
            return out
        if post_norm is not None:
            y = post_norm.forward(y, out=torch.empty_like(y))
        ops.add_rmsnorm(x, y, None, None, None)
        return self._enter(x, next_norm) if want_next else None

    def forward(self, x, normed, ctx, view, state, next_norm=None, want_next=False):
        """Update the residual ``x`` in place.  ``normed`` is ``pre_mixer_norm(x)`` if the caller
        has it already.  Returns ``next_norm(x)`` when ``want_next``."""
        if normed is None:
            normed = self._enter(x, self.pre_mixer_norm)
        y = self.mixer.forward(normed, ctx, view, state)
        n2 = self._add_then_norm(x, y, self.post_mixer_norm, self.pre_ffn_norm, True)
        d = self.feed_forward.forward(n2, ctx)
        return self._add_then_norm(x, d, self.post_ffn_norm, next_norm, want_next)


register_part("block", "sandwich", Block)
