"""Weight files, the loader and the random-weights mode."""
from .safetensors_io import SafeTensorsFile, SafeTensorsModel, write_safetensors
from .loader import load_weights, compare, raise_if_mismatch
from .random_init import write_random_model, fill_random, random_tensors, model_needs

__all__ = ["SafeTensorsFile", "SafeTensorsModel", "write_safetensors", "load_weights", "compare",
           "raise_if_mismatch", "write_random_model", "fill_random", "random_tensors", "model_needs"]
