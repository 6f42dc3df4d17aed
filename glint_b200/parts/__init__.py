"""The parts a model is put together from, each registered under its kind."""
from .base import Part, TensorNeed
from .registry import register_part, part_class, build_part, build_block, CATEGORIES
from .linear import linear
from . import norms, positions, embedding, attention, feed_forward  # registration
from .norms import RMSNorm
from .positions import Rotary
from .embedding import ScaledEmbedding, LMHead
from .attention import Attention
from .feed_forward import GatedFeedForward
from .block import Block

__all__ = ["Part", "TensorNeed", "register_part", "part_class", "build_part", "build_block", "CATEGORIES", "linear",
           "RMSNorm", "Rotary", "ScaledEmbedding", "LMHead", "Attention", "GatedFeedForward", "Block"]
