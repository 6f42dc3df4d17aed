"""Weights from a model folder into a model, by tensor name.

The model says which tensors it needs (name, shape, kind); the file says which it has.  All
differences are reported in ONE ``WeightsError`` that lists missing tensors, unexpected
tensors and wrong shapes together (the reference stops at the first: ``TensorNotFound``,
"expected shape [r, c], found [...]", src/transformer/weights.rs:387-443).

Kept dtypes: matrices in the engine's dtype (bfloat16, or float32 for the true 32-bit path;
bfloat16 and float16 widen to float32 exactly, as the reference widens every stored weight,
src/tensor/quantized.rs:1021-1044); vectors (norm weights) in 32-bit, as the reference keeps
its norms (src/model/safetensors.rs:588-601); integer tables as int32.  A matrix stored in
32-bit is rounded to bfloat16 only when the engine itself runs in bfloat16, because the
tensor-core products take bfloat16 operands; every other 32-bit tensor stays 32-bit.
"""
from __future__ import annotations

import torch

from ..errors import WeightsError
from .safetensors_io import SafeTensorsModel

_FLOAT_STORED = ("F32", "BF16", "F16")
_INT_STORED = ("I32", "I64")


def compare(needs, available):
    """``available``: name -> (shape, stored dtype name).  Returns (missing, unexpected, wrong)."""
    wanted = {n.name: n for n in needs}
    missing = sorted(n.name for n in needs if not n.optional and n.name not in available)
    unexpected = sorted(name for name in available if name not in wanted)
    wrong = []
    for name, need in sorted(wanted.items()):
        if name not in available:
            continue
        shape, stored = available[name]
        if tuple(shape) != tuple(need.shape):
            wrong.append(f"{name}: expected shape {list(need.shape)}, found {list(shape)}")
        elif need.kind == "int" and stored not in _INT_STORED:
            wrong.append(f"{name}: expected an integer table, found dtype {stored}")
        elif need.kind != "int" and stored not in _FLOAT_STORED:
            wrong.append(f"{name}: expected a float tensor, found dtype {stored}")
    return missing, unexpected, wrong


def raise_if_mismatch(where, missing, unexpected, wrong):
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where}: the weights do not fit the model"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shapes or dtypes ({len(wrong)}): " + "; ".join(wrong))
    raise WeightsError("\n".join(lines), missing, unexpected, wrong)


def kept_dtype(kind, stored, engine_dtype):
    if kind == "int":
        return torch.int32
    if kind == "vector":
        return torch.float32
    return engine_dtype


def load_weights(model, model_dir):
    """Read every tensor ``model`` needs from ``model_dir``, move it to the model's device in
    its kept dtype and hand the set to ``model.bind``."""
    files = SafeTensorsModel(model_dir)
    try:
        needs = model.needs()
        available = {name: (files.shape(name), files.dtype_name(name)) for name in files.names()}
        raise_if_mismatch(model_dir, *compare(needs, available))
        device, dtype = model.rt.device, model.rt.dtype
        tensors = {}
        for need in needs:
            if need.name not in available:
                continue
            host = files.tensor(need.name)
            tensors[need.name] = host.to(device=device, dtype=kept_dtype(need.kind, available[need.name][1], dtype))
        model.bind(tensors)
    finally:
        files.close()
    return model
