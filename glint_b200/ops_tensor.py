"""Python face of the tensor-core kernels (bfloat16 only)."""
from __future__ import annotations


def gemm_supported(M, N, K):
    return False


def attention_supported(nh, nkv, hd, page_size):
    return False
