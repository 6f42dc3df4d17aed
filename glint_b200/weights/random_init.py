"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration
and a seed, or the same kind of weights straight into a model on the device.

The reference has only test fixtures for this (arithmetic ramps,
src/transformer/forward.rs:1604-1685; an LCG in [-0.5, 0.5), src/model/safetensors.rs:882-892).
Matrices are N(0, std), vectors (norm weights) N(0, norm_std); values are drawn in float32
from one seeded generator in sorted-name order and stored in ``store_dtype`` (bfloat16 by
default, so that the 32-bit and the bfloat16 engine read identical weights).
"""
from __future__ import annotations

import json
import os

import torch

from ..config import config_from_dict
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


class MetaRuntime:
    """Stands in for the runtime where parts are built only to be asked what they need."""

    def __init__(self, dtype=torch.float32):
        self.device = torch.device("cpu")
        self.dtype = dtype
        self.status = None
        self.kernels = "plain"
        self.tensor_cores = False


def model_needs(config):
    from ..engine.model import CausalLM
    return CausalLM(config.model_spec(), MetaRuntime()).needs()


def random_tensors(needs, seed, std=0.02, norm_std=0.1, dtype=torch.bfloat16, device="cpu",
                   include_optional=False):
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out = {}
    for need in sorted(needs, key=lambda n: n.name):
        if need.optional and not include_optional:
            continue
        if need.kind == "int":
            out[need.name] = torch.zeros(need.shape, dtype=torch.int32, device=device)
            continue
        sigma = norm_std if need.kind == "vector" else std
        t = torch.empty(need.shape, dtype=torch.float32, device=device)
        t.normal_(0.0, sigma, generator=gen)
        out[need.name] = t.to(dtype)
    return out


def write_random_model(config, out_dir, seed=0, std=0.02, norm_std=0.1, store_dtype="bfloat16",
                       untied_head=False):
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors``.  ``config`` is a typed
    configuration or the dict of a config.json.  ``untied_head`` also writes the optional head
    tensor (for Gemma 2: ``lm_head.weight``)."""
    if isinstance(config, dict):
        config = config_from_dict(config)
    os.makedirs(out_dir, exist_ok=True)
    tensors = random_tensors(model_needs(config), seed, std, norm_std, _STORE[store_dtype],
                             include_optional=untied_head)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      {"format": "pt", "seed": seed, "std": std, "norm_std": norm_std})
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=1)
    return out_dir


def fill_random(model, seed=0, std=0.02, norm_std=0.1):
    """Give ``model`` random weights generated on its device (no folder): for benchmarks of
    shapes too large to be worth writing out.  Values differ from ``write_random_model``'s."""
    from .loader import kept_dtype
    dtype, device = model.rt.dtype, model.rt.device
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    tensors = {}
    for need in sorted(model.needs(), key=lambda n: n.name):
        if need.optional:
            continue
        kept = kept_dtype(need.kind, "BF16", dtype)
        if need.kind == "int":
            tensors[need.name] = torch.zeros(need.shape, dtype=kept, device=device)
            continue
        t = torch.empty(need.shape, dtype=kept, device=device)
        t.normal_(0.0, norm_std if need.kind == "vector" else std, generator=gen)
        if need.kind == "vector":   # the values a bfloat16 file would hold
            t = t.to(torch.bfloat16).to(torch.float32)
        tensors[need.name] = t
    model.bind(tensors)
    return model
