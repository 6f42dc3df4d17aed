"""y = x W^T for a weight kept [out, in] as in the file (src/transformer/forward.rs:546-557)."""
from __future__ import annotations

import torch

from .. import ops


def linear(rt, a, w, cap=0.0, out=None):
    """float32 [M, N] = a [M, K] @ w [N, K]^T, with an optional soft cap on the result.

    float32 weights take the CUDA-core product (true 32-bit).  bfloat16 weights take a tensor-core
    kernel unless the runtime asks for plain kernels; which one is the native runtime's choice
    (``glint_op_linear`` in csrc/runtime.cu), the same that a lowered program makes.
    """
    if out is None:
        out = torch.empty((a.shape[0], w.shape[0]), dtype=torch.float32, device=a.device)
    ops.op_linear(rt, a, w, out, cap)
    return out
