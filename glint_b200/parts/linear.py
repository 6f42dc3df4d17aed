"""y = x W^T for a weight kept [out, in] as in the file (src/transformer/forward.rs:546-557)."""
from __future__ import annotations

import torch

from .. import ops


def linear(rt, a, w, cap=0.0, out=None):
    """float32 [M, N] = a [M, K] @ w [N, K]^T, with an optional soft cap on the result.

    float32 weights take the CUDA-core product (true 32-bit).  bfloat16 weights take the
    tcgen05 tensor-core kernel unless the runtime asks for plain kernels.
    """
    M = a.shape[0]
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    if rt.tensor_cores and w.dtype == torch.bfloat16:
        from .. import ops_tensor
        if ops_tensor.gemm_supported(M, N, w.shape[1]):
            ops_tensor.gemm(a, w, out, cap, rt.status)
            return out
    ops.gemm_plain(a, w, out, cap)
    return out
