"""Typed configurations and the architecture registry."""
from .spec import PartSpec, BlockSpec, LayerCall, ModelSpec
from .registry import (register_architecture, registered_architectures, architecture_name,
                       config_from_dict, read_config_json, load_config)
from .gemma2 import Gemma2Config, ARCHITECTURE as _GEMMA2, MODEL_TYPE as _GEMMA2_TYPE

register_architecture(_GEMMA2, Gemma2Config, _GEMMA2_TYPE)

__all__ = ["PartSpec", "BlockSpec", "LayerCall", "ModelSpec", "register_architecture",
           "registered_architectures", "architecture_name", "config_from_dict", "read_config_json",
           "load_config", "Gemma2Config"]
