"""One registry from an architecture's name to its configuration class.

The reference keeps an allow-list of family strings and one forward pass with
switches (src/model/config.rs:149-157, :205-216).  Here a name maps to a class
with ``from_dict(config.json) -> config`` and ``config.model_spec() -> ModelSpec``;
everything after that is built from the spec alone.  The name is
``architectures[0]`` of config.json, else ``model_type``.
"""
from __future__ import annotations

import json
import os

from ..errors import ConfigError

_ARCHITECTURES = {}
_MODEL_TYPES = {}


def register_architecture(name, config_class, model_type=None):
    """Register ``config_class`` under ``name`` (and under ``model_type`` for files that lack
    ``architectures``).  Registering a name again replaces the earlier entry."""
    _ARCHITECTURES[name] = config_class
    if model_type is not None:
        _MODEL_TYPES[model_type.lower()] = name


def registered_architectures():
    return sorted(_ARCHITECTURES)


def architecture_name(obj):
    if not isinstance(obj, dict):
        raise ConfigError("config.json: top level value is not a JSON object")
    archs = obj.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    model_type = obj.get("model_type")
    if isinstance(model_type, str):
        name = _MODEL_TYPES.get(model_type.lower())
        if name is None:
            raise ConfigError(f"config.json: model_type '{model_type}' is not supported "
                              f"(registered: {', '.join(registered_architectures())})")
        return name
    raise ConfigError("config.json: required key 'architectures' (or 'model_type') is missing")


def config_from_dict(obj):
    name = architecture_name(obj)
    cls = _ARCHITECTURES.get(name)
    if cls is None:
        raise ConfigError(f"config.json: architecture '{name}' is not supported "
                          f"(registered: {', '.join(registered_architectures())})")
    return cls.from_dict(obj)


def read_config_json(model_dir):
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: file not found")
    try:
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)
    except (json.JSONDecodeError, UnicodeDecodeError) as e:
        raise ConfigError(f"{path}: invalid JSON: {e}") from None


def load_config(model_dir):
    """config.json of a model folder -> typed configuration of its architecture."""
    return config_from_dict(read_config_json(model_dir))
