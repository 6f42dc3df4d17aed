"""Model description as data: which parts, with which sizes, in which order.

An architecture turns its typed configuration into a ``ModelSpec``.  The spec
names parts by ``kind`` (looked up in ``glint_b200.parts`` registries) and
gives each its sizes and constants as ``params``; nothing below this file
knows which architecture it serves.  The reference has one forward pass with
``is_gemma`` switches instead (src/transformer/forward.rs:64-83).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class PartSpec:
    """One part: ``kind`` selects the class, ``params`` are its constructor arguments,
    ``tensors`` maps the part's own tensor roles to names in the weight file."""
    kind: str
    params: dict = field(default_factory=dict)
    tensors: dict = field(default_factory=dict)


@dataclass
class BlockSpec:
    """One layer: a mixer, a feed-forward and up to four norms, arranged by the block class that
    ``kind`` names in the ``"block"`` registry.

    The package's kind ``"sandwich"`` computes ``x = x + post_mixer_norm(mixer(pre_mixer_norm(x)))``
    and then the same shape for the feed-forward; a norm that is ``None`` is the identity.  Another
    arrangement (a parallel residual, a shared norm) is another kind, which reads the same fields
    and its own ``params``.
    """
    mixer: PartSpec
    feed_forward: PartSpec
    pre_mixer_norm: Optional[PartSpec] = None
    post_mixer_norm: Optional[PartSpec] = None
    pre_ffn_norm: Optional[PartSpec] = None
    post_ffn_norm: Optional[PartSpec] = None
    kind: str = "sandwich"
    params: dict = field(default_factory=dict)


@dataclass
class LayerCall:
    """One entry of the run order: run block ``layer``.

    ``cache_of`` is ``None`` when the call keeps a cache of its own, or the index of an
    earlier entry of the run order whose cache this call reads without writing.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    blocks: list
    run_order: list
    final_norm: Optional[PartSpec]
    head: PartSpec
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    info: dict = field(default_factory=dict)

    def validate(self):
        n = len(self.blocks)
        for i, call in enumerate(self.run_order):
            if not 0 <= call.layer < n:
                raise ValueError(f"run order entry {i} names layer {call.layer}, model has {n}")
            if call.cache_of is not None and not 0 <= call.cache_of < i:
                raise ValueError(f"run order entry {i} reads the cache of entry {call.cache_of}, "
                                 f"which does not come before it")
