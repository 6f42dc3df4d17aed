"""Python face of the CUDA kernels: torch tensors in, a launch on the current stream out.

There is no CPU fallback and no library stand-in: if the extension cannot be built or
loaded, or a tensor is not on a CUDA device, the call raises ``KernelError``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .csrc import build
from .errors import KernelError

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

ACTIVATIONS = {"gelu_tanh": 0, "silu": 1}

launch_count = 0  # kernels launched through this module since import (graph replays add their own)


def launches():
    """Kernels of this package launched so far in this process: through this module's calls, through the
    native runtime's routed operations and programs, and by replayed graphs."""
    lib = core().lib
    lib.glint_native_launches.restype = c_longlong
    return launch_count + int(lib.glint_native_launches())


def dtype_code(dtype):
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 storage, not {dtype}") from None


class _Lib:
    """A loaded kernel library with typed entry points."""

    def __init__(self, name, signatures):
        self.lib = build.load_library(name)
        self.err = None
        for fn, argtypes in signatures.items():
            f = getattr(self.lib, fn)
            f.argtypes = argtypes
            f.restype = c_int
            setattr(self, fn, f)


_P, _I, _F, _L = c_void_p, c_int, c_float, c_longlong

_CORE_SIGNATURES = {
    "glint_embed_scale": [_P, _I, _P, _P, _I, _I, _F, _I, _P, _P],
    "glint_rmsnorm": [_P, _P, _P, _P, _I, _I, _I, _F, _F, _P],
    "glint_add_rmsnorm": [_P, _P, _P, _F, _F, _P, _I, _P, _F, _F, _I, _I, _P],
    "glint_rope_table": [_P, _P, _F, _P, _I, _I, _P],
    "glint_rope_kv_write": [_P, _P, _P, _P, _I, _P, _F, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "glint_gated_act": [_P, _P, _I, _I, _I, _I, _P],
    "glint_softcap": [_P, _L, _F, _P],
    "glint_place_tokens": [_P, _P, _P, _P, _I, _P],
    "glint_gemm_plain": [_P, _P, _I, _P, _I, _I, _I, _F, _P],
    "glint_attention_plain": [_P, _P, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _F, _I, _P, _P],
    "glint_argmax": [_P, _L, _I, _I, _P, _P],
    "glint_argmax_wide": [_P, _L, _I, _I, _P, _P, _P, _P],
    "glint_apply_penalty": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P],
    "glint_sample": [_P, _L, _P, _I, _I, _P, _P, _P, _P, _P, _P, _P],
    "glint_sample_rows": [_P, _L, _P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P],
    "glint_sample_prepare": [_P, _P, _P, _P, _I, _I, _P, _I, _P],
}

_core = None


def core():
    global _core
    if _core is None:
        _core = _Lib("core", _CORE_SIGNATURES)
        _core.lib.glint_error_string.argtypes = [c_int]
        _core.lib.glint_error_string.restype = ctypes.c_char_p
    return _core


def error_string(code):
    return core().lib.glint_error_string(code).decode()


def check(code, what):
    global launch_count
    if code != 0:
        raise KernelError(f"{what}: {error_string(code)} (code {code})")
    launch_count += 1


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def stream():
    """Handle of the current stream of the current device.  Called once per launch: the two C entry
    points cost a fraction of a microsecond, ``torch.cuda.current_stream()`` builds a Python object
    each time (a third of the host time of a step that is not replayed from a graph)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def fallbacks():
    """Operations that a tensor-core runtime ran on CUDA cores so far because of their sizes."""
    lib = core().lib
    lib.glint_native_fallbacks.restype = c_longlong
    return int(lib.glint_native_fallbacks())


def ptr(t):
    return 0 if t is None else t.data_ptr()


def require(t, dtype, name):
    if t is None:
        return
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: the kernels have no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


# -------------------------------------------------------------------------------------------------


def embed_scale(table, ids, out, scale, status):
    """out[t] = table[ids[t]] * scale; out is float32 [T, H]."""
    T, H = out.shape
    require(table, None, "table"); require(ids, torch.int32, "ids"); require(out, torch.float32, "out")
    check(core().glint_embed_scale(ptr(table), dtype_code(table.dtype), ptr(ids), ptr(out), T, H, scale,
                                   table.shape[0], ptr(status), stream()), "embed_scale")


def rmsnorm(x, weight, out, eps, offset, row_index=None):
    """out[r] = x[row_index[r] or r] * rsqrt(mean(x^2)+eps) * (offset + weight)."""
    rows, H = out.shape
    require(x, torch.float32, "x"); require(weight, torch.float32, "weight"); require(out, None, "out")
    require(row_index, torch.int32, "row_index")
    check(core().glint_rmsnorm(ptr(x), ptr(row_index), ptr(weight), ptr(out), dtype_code(out.dtype), rows, H,
                               eps, offset, stream()), "rmsnorm")


def add_rmsnorm(x, y, norm_a, out, norm_b):
    """x += norm_a(y); out = norm_b(x).  ``norm_a``/``norm_b`` are (weight, eps, offset) or None
    (identity); ``out`` may be None."""
    rows, H = x.shape
    require(x, torch.float32, "x"); require(y, torch.float32, "y"); require(out, None, "out")
    wa, ea, oa = norm_a if norm_a is not None else (None, 0.0, 0.0)
    wb, eb, ob = norm_b if norm_b is not None else (None, 0.0, 0.0)
    require(wa, torch.float32, "norm_a weight"); require(wb, torch.float32, "norm_b weight")
    code = dtype_code(out.dtype) if out is not None else F32
    check(core().glint_add_rmsnorm(ptr(x), ptr(y), ptr(wa), ea, oa, ptr(out), code, ptr(wb), eb, ob, rows, H,
                                   stream()), "add_rmsnorm")


def rope_kv_write(qkv, positions, token_slot, block_table, inv_freq, factor, rot, q_out, k_pool, v_pool,
                  nh, nkv, hd, page_size, num_pages, status):
    """Rotate q and k of ``qkv`` [T, (nh+2nkv)*hd] float32, write q to ``q_out`` and k, v into the
    pages named by ``block_table``.  ``k_pool`` None: rotate q only."""
    T = qkv.shape[0]
    require(qkv, torch.float32, "qkv"); require(positions, torch.int32, "positions")
    require(token_slot, torch.int32, "token_slot"); require(block_table, torch.int32, "block_table")
    require(inv_freq, torch.float32, "inv_freq"); require(q_out, None, "q_out")
    require(k_pool, q_out.dtype, "k_pool"); require(v_pool, q_out.dtype, "v_pool")
    check(core().glint_rope_kv_write(ptr(qkv), ptr(positions), ptr(token_slot), ptr(block_table),
                                     block_table.shape[1], ptr(inv_freq), factor, rot, ptr(q_out), ptr(k_pool),
                                     ptr(v_pool), dtype_code(q_out.dtype), T, nh, nkv, hd, page_size, num_pages,
                                     ptr(status), stream()), "rope_kv_write")


def rope_table(positions, inv_freq, factor, out):
    """out[t, j] = (cos, sin) of (positions[t] / factor) * inv_freq[j]; out float32 [T, half, 2]."""
    T, half = out.shape[0], inv_freq.numel()
    require(positions, torch.int32, "positions"); require(inv_freq, torch.float32, "inv_freq")
    require(out, torch.float32, "out")
    if tuple(out.shape) != (positions.shape[0], half, 2):
        raise KernelError(f"rope_table: out {tuple(out.shape)} does not fit {positions.shape[0]} tokens x {half} pairs")
    check(core().glint_rope_table(ptr(positions), ptr(inv_freq), factor, ptr(out), T, half, stream()), "rope_table")


def gated_act(gu, out, activation):
    """out[t, i] = act(gu[t, i]) * gu[t, I + i]; gu float32 [T, 2I]."""
    T, I = out.shape
    require(gu, torch.float32, "gu"); require(out, None, "out")
    check(core().glint_gated_act(ptr(gu), ptr(out), dtype_code(out.dtype), T, I, ACTIVATIONS[activation],
                                 stream()), "gated_act")


def place_tokens(ids, dst_rows, src, src_idx):
    """ids[dst_rows[i]] = src[src_idx[i]] (all int32 on the device)."""
    check(core().glint_place_tokens(ptr(ids), ptr(dst_rows), ptr(src), ptr(src_idx), dst_rows.shape[0], stream()),
          "place_tokens")


def softcap_(x, cap):
    require(x, torch.float32, "x")
    check(core().glint_softcap(ptr(x), x.numel(), cap, stream()), "softcap")


def gemm_plain(a, w, out, cap=0.0):
    """out[M, N] (float32) = a[M, K] @ w[N, K]^T on CUDA cores, optional soft cap."""
    M, K = a.shape
    N = w.shape[0]
    require(a, w.dtype, "a"); require(w, None, "w"); require(out, torch.float32, "out")
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    check(core().glint_gemm_plain(ptr(a), ptr(w), dtype_code(w.dtype), ptr(out), M, N, K, cap or 0.0, stream()),
          "gemm_plain")


def attention_plain(q, k_pool, v_pool, positions, token_slot, block_table, out, nh, nkv, hd, page_size,
                    num_pages, multiplier, cap, window, status):
    T = q.shape[0]
    require(q, None, "q"); require(k_pool, q.dtype, "k_pool"); require(v_pool, q.dtype, "v_pool")
    require(out, q.dtype, "out"); require(positions, torch.int32, "positions")
    require(token_slot, torch.int32, "token_slot"); require(block_table, torch.int32, "block_table")
    check(core().glint_attention_plain(ptr(q), ptr(k_pool), ptr(v_pool), dtype_code(q.dtype), ptr(positions),
                                       ptr(token_slot), ptr(block_table), block_table.shape[1], ptr(out), T, nh,
                                       nkv, hd, page_size, num_pages, multiplier, cap or 0.0, window or 0,
                                       ptr(status), stream()), "attention_plain")


_argmax_scratch = {}


def argmax(logits, out):
    """out[r] = index of the largest logit of row r (the last one among equals).  Wide rows are
    shared by several blocks that meet in a per-row atomic (scratch kept per device, left zeroed)."""
    rows, V = logits.shape
    require(logits, torch.float32, "logits"); require(out, torch.int32, "out")
    keys = counters = None
    if V >= 32768:
        entry = _argmax_scratch.get(str(logits.device))
        if entry is None or entry[0].numel() < rows:
            n = max(rows, 1024)
            entry = (torch.zeros(n, dtype=torch.int64, device=logits.device),
                     torch.zeros(n, dtype=torch.int32, device=logits.device))
            _argmax_scratch[str(logits.device)] = entry
        keys, counters = entry
    check(core().glint_argmax_wide(ptr(logits), logits.stride(0), rows, V, ptr(out), ptr(keys), ptr(counters),
                                   stream()), "argmax")


def apply_penalty(logits, work, offsets, tokens, counts, penalty):
    rows, V = logits.shape
    check(core().glint_apply_penalty(ptr(logits), logits.stride(0), rows, V, ptr(work), ptr(offsets), ptr(tokens),
                                     ptr(counts), ptr(penalty), stream()), "apply_penalty")


def sample(src, work, temperature, top_k, top_p, min_p, uniform, out):
    rows, V = src.shape
    require(src, torch.float32, "logits"); require(work, torch.float32, "work")
    require(temperature, torch.float32, "temperature"); require(top_k, torch.int32, "top_k")
    require(top_p, torch.float32, "top_p"); require(min_p, torch.float32, "min_p")
    require(uniform, torch.float32, "uniform"); require(out, torch.int32, "out")
    check(core().glint_sample(ptr(src), src.stride(0), ptr(work), rows, V, ptr(temperature), ptr(top_k),
                              ptr(top_p), ptr(min_p), ptr(uniform), ptr(out), stream()), "sample")


def sampler_record_words():
    """32-bit words of the sampler's per-request record (see ``sample_prepare``)."""
    lib = core().lib
    lib.glint_sampler_record_words.restype = c_int
    return int(lib.glint_sampler_record_words())


def sample_prepare(records, row_slots, positions, logit_rows, row_opts):
    """For the rows of a step that are about to be sampled: copy each row's options from its request
    slot's record (``records`` int32 [slots, words]: temperature, top-p, min-p, penalty as float bits,
    top-k, not-greedy, generator state low and high, position, count) into ``row_opts`` (float32
    [7, stride]: temperature, uniform draw, top-p, min-p, penalty, not-greedy, top-k as int bits),
    advance the generators of the rows that draw, and bring position and count up to date."""
    rows = row_slots.shape[0]
    require(records, torch.int32, "records"); require(row_slots, torch.int32, "row_slots")
    require(positions, torch.int32, "positions"); require(logit_rows, torch.int32, "logit_rows")
    require(row_opts, torch.float32, "row_opts")
    if records.dim() != 2 or row_opts.dim() != 2 or row_opts.shape[0] != 7 or logit_rows.shape[0] != rows:
        raise KernelError("sample_prepare: records [slots, words], row_opts [7, stride] and one logit row per row")
    check(core().glint_sample_prepare(ptr(records), ptr(row_slots), ptr(positions), ptr(logit_rows), rows,
                                      records.shape[0], ptr(row_opts), row_opts.shape[1], stream()), "sample_prepare")


def sample_rows(logits, work, temperature, top_k, top_p, min_p, uniform, out, penalties=None):
    """The whole choice for every row of ``logits`` [rows, V]: repeat penalty (``penalties`` = (offsets
    [rows + 1], tokens, counts, penalty [rows]), a token once per row, or None), temperature, top-k,
    min-p, softmax, top-p, draw with ``uniform``.  Rows of 16 K entries and more are shared by the blocks
    of a cluster; ``work`` [rows, V] is scratch for narrower rows."""
    rows, V = logits.shape
    require(logits, torch.float32, "logits"); require(work, torch.float32, "work")
    require(temperature, torch.float32, "temperature"); require(top_k, torch.int32, "top_k")
    require(top_p, torch.float32, "top_p"); require(min_p, torch.float32, "min_p")
    require(uniform, torch.float32, "uniform"); require(out, torch.int32, "out")
    offsets = tokens = counts = penalty = None
    if penalties is not None:
        offsets, tokens, counts, penalty = penalties
        require(offsets, torch.int32, "offsets"); require(tokens, torch.int32, "tokens")
        require(counts, torch.int32, "counts"); require(penalty, torch.float32, "penalty")
        if offsets.numel() != rows + 1 or penalty.numel() != rows or tokens.numel() != counts.numel():
            raise KernelError("sample_rows: the penalty lists do not fit the rows")
    if work.shape[0] < rows or work.shape[1] != V:
        raise KernelError(f"sample_rows: work {tuple(work.shape)} does not fit {rows} rows of {V}")
    check(core().glint_sample_rows(ptr(logits), logits.stride(0), ptr(work), rows, V, ptr(temperature), ptr(top_k),
                                   ptr(top_p), ptr(min_p), ptr(uniform), ptr(offsets), ptr(tokens), ptr(counts),
                                   ptr(penalty), ptr(out), stream()), "sample_rows")


# ---- routed operations: the native runtime chooses the kernel (csrc/runtime.h) -------------------------------


def _routed():
    lib = core().lib
    if not getattr(lib, "_glint_routed", False):
        lib.glint_op_linear.argtypes = [_P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P, _P]
        lib.glint_op_linear.restype = c_int
        lib._glint_routed = True
    return lib


def op_linear(rt, a, w, out, cap=0.0, gated=None, tmp=None):
    """out [M, N] = a [M, K] w[N, K]^T with the kernel the runtime chooses for these sizes (CUDA cores for
    float32, the weight-streaming or the tiled tensor-core product for bfloat16); ``gated`` (an activation
    name): w is [2N, K] and out = act(a w[:N]^T) * (a w[N:]^T) in the activation dtype."""
    M, K = a.shape
    N = w.shape[0] // 2 if gated else w.shape[0]
    require(a, w.dtype, "a"); require(w, None, "w"); require(out, None, "out"); require(tmp, torch.float32, "tmp")
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"linear shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    rc = _routed().glint_op_linear(ctypes.addressof(rt.native), ptr(a), ptr(w), ptr(out), int(out.dtype == torch.bfloat16),
                                   M, N, K, cap or 0.0, 1 if gated else 0, ACTIVATIONS[gated] if gated else 0, ptr(tmp),
                                   stream())
    if rc != 0:
        raise KernelError(f"linear: {error_string(rc)} (code {rc})")
