"""Python face of the tensor-core kernels (bfloat16 only): tcgen05 matrix products."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import ops
from .errors import KernelError

_P, _I, _F, _L = c_void_p, c_int, c_float, c_longlong

_SIGNATURES = {
    "glint_gemm_tcgen05": [_P, _P, _P, _I, _I, _I, _I, _L, _F, _I, _I, _I, _P, _P, _P, _I, _P],
}

_lib = None
_scratch = {}


def lib():
    global _lib
    if _lib is None:
        _lib = ops._Lib("tensor", _SIGNATURES)
        _lib.lib.glint_gemm_workspace_bytes.restype = c_longlong
        _lib.lib.glint_gemm_counter_count.restype = c_int
    return _lib


def scratch(device):
    """Split-K workspace and zeroed tile counters of a device (allocated once)."""
    key = str(device)
    if key not in _scratch:
        l = lib()
        ws = torch.empty(l.lib.glint_gemm_workspace_bytes() // 4, dtype=torch.float32, device=device)
        counters = torch.zeros(l.lib.glint_gemm_counter_count(), dtype=torch.int32, device=device)
        _scratch[key] = (ws, counters)
    return _scratch[key]


def gemm_supported(M, N, K):
    return M > 0 and N > 0 and K > 0 and K % 8 == 0


def gemm(a, w, out, cap=0.0, status=None, force_splits=0):
    """out[M, N] = a[M, K] @ w[N, K]^T with bfloat16 operands, float32 accumulation; ``out`` is
    float32 or bfloat16; ``cap`` > 0 applies the soft cap."""
    M, K = a.shape
    N = w.shape[0]
    ops.require(a, torch.bfloat16, "a"); ops.require(w, torch.bfloat16, "w"); ops.require(out, None, "out")
    if w.shape[1] != K or tuple(out.shape) != (M, N) or out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError(f"gemm shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    ws, counters = scratch(a.device)
    st = status if status is not None else counters[-1:]
    ops.check(lib().glint_gemm_tcgen05(ops.ptr(a), ops.ptr(w), ops.ptr(out), int(out.dtype == torch.bfloat16), M, N,
                                       K, N, cap or 0.0, 0, 0, 0, ops.ptr(ws), ops.ptr(counters), ops.ptr(st),
                                       force_splits, ops.stream()), "gemm_tcgen05")


def gemm_gated(a, w_gate_up, out, activation, status=None, force_splits=0):
    """out[M, I] (bfloat16) = act(a @ w[:I]^T) * (a @ w[I:]^T) for w_gate_up [2I, K], in one kernel."""
    M, K = a.shape
    I = w_gate_up.shape[0] // 2
    ops.require(a, torch.bfloat16, "a"); ops.require(w_gate_up, torch.bfloat16, "w"); ops.require(out, torch.bfloat16, "out")
    if w_gate_up.shape[1] != K or tuple(out.shape) != (M, I):
        raise KernelError(f"gated gemm shapes do not fit: a {tuple(a.shape)}, w {tuple(w_gate_up.shape)}, "
                          f"out {tuple(out.shape)}")
    ws, counters = scratch(a.device)
    st = status if status is not None else counters[-1:]
    ops.check(lib().glint_gemm_tcgen05(ops.ptr(a), ops.ptr(w_gate_up), ops.ptr(out), 1, M, I, K, 2 * I, 0.0, 1, I,
                                       ops.ACTIVATIONS[activation], ops.ptr(ws), ops.ptr(counters), ops.ptr(st),
                                       force_splits, ops.stream()), "gemm_tcgen05 (gated)")


def attention_supported(nh, nkv, hd, page_size):
    return False
