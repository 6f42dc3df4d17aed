"""From a model folder (or a configuration and a seed) to a model with weights on the device.

The reference's path is ``Model::load`` -> ``HfModelDir::open`` -> ``HfConfig::from_json`` ->
``TransformerWeights::from_safetensors`` (src/api/mod.rs:130-156,
src/model/safetensors.rs:710-749, src/transformer/weights.rs:157-328); here the model class
is chosen by config.json through the architecture registry.
"""
from __future__ import annotations

from ..config import config_from_dict, load_config
from ..runtime import Runtime
from ..weights import fill_random, load_weights
from .model import CausalLM
from .step import Engine


def load_model(model_dir, dtype="bfloat16", device="cuda:0", kernels="auto"):
    config = load_config(model_dir)
    rt = Runtime(device, dtype, kernels)
    model = CausalLM(config.model_spec(), rt)
    model.config = config
    return load_weights(model, model_dir)


def random_model(config, seed=0, std=0.02, norm_std=0.1, dtype="bfloat16", device="cuda:0", kernels="auto"):
    """A model of ``config`` (typed, or a config.json dict) with random weights made on the device."""
    if isinstance(config, dict):
        config = config_from_dict(config)
    rt = Runtime(device, dtype, kernels)
    model = CausalLM(config.model_spec(), rt)
    model.config = config
    return fill_random(model, seed, std, norm_std)


def pages_for_tokens(tokens, page_size):
    return max(1, (int(tokens) + page_size - 1) // page_size)


def build_engine(model, max_tokens, num_slots=64, page_size=16, use_graphs=True):
    """An engine whose every cache group can hold ``max_tokens`` tokens in all."""
    return Engine(model, pages_for_tokens(max_tokens, page_size), num_slots, page_size, use_graphs)
