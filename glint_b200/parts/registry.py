"""Registries from a part's ``kind`` to its class, one per category.

A new mixer, feed-forward, norm, position encoding or arrangement of a layer (``"block"``) is added
by registering a class under a new kind; an architecture's ``model_spec()`` then names that kind.
Nothing else changes.
"""
from __future__ import annotations

from ..errors import ConfigError

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "embedding", "head", "block")
_REGISTRY = {c: {} for c in CATEGORIES}


def register_part(category, kind, cls):
    if category not in _REGISTRY:
        raise ConfigError(f"unknown part category '{category}' (known: {', '.join(CATEGORIES)})")
    _REGISTRY[category][kind] = cls
    return cls


def part_class(category, kind):
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        raise ConfigError(f"no {category} of kind '{kind}' is registered "
                          f"(registered: {', '.join(sorted(_REGISTRY.get(category, {})))})") from None


def build_part(category, spec, rt):
    if spec is None:
        return None
    return part_class(category, spec.kind)(rt, spec.params, spec.tensors)


def build_block(spec, rt):
    """A layer from its ``BlockSpec``: the class registered for ``spec.kind`` gets the runtime and the
    whole spec (its parts' specs and its own ``params``)."""
    return part_class("block", spec.kind)(rt, spec)
