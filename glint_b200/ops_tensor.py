"""Python face of the tensor-core kernels (bfloat16 only), one function per kernel: the tcgen05 and the
weight-streaming products, their variants with the rotary epilogue, and the attention kernels.  Which of
them a model's operation takes is decided by the native runtime (csrc/runtime.cu); these functions are
for kernel tests and measurements."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import ops
from .errors import KernelError

_P, _I, _F, _L = c_void_p, c_int, c_float, c_longlong

_SIGNATURES = {
    "glint_gemm_tcgen05": [_P, _P, _P, _I, _I, _I, _I, _L, _F, _I, _I, _I, _P, _P, _P, _I, _P],
    "glint_gemm_skinny": [_P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _I, _P],
    "glint_gemm_tcgen05_rope": [_P, _P, _I, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "glint_gemm_skinny_rope": [_P, _P, _I, _I, _P, _P, _P, _I, _P, _F, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    "glint_attention_decode": [_P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _F, _I, _I, _P, _P],
    "glint_attention_decode_supported": [_I, _I, _I, _I],
    "glint_attention_decode_stream_workspace": [_I, _I, _I, _I],
    "glint_attention_decode_stream_plan": [_P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P],
    "glint_attention_decode_stream": [_P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _F, _I, _I, _P, _P,
                                      _P, _I, _P, _P],
    "glint_attention_prefill": [_P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _F, _F, _I, _P, _P],
    "glint_attention_tcgen05": [_P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _I, _P, _P],
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
    entry = _scratch.get(device)
    if entry is None:
        l = lib()
        ws = torch.empty(l.lib.glint_gemm_workspace_bytes() // 4, dtype=torch.float32, device=device)
        counters = torch.zeros(l.lib.glint_gemm_counter_count(), dtype=torch.int32, device=device)
        entry = _scratch[device] = (ws, counters)
    return entry


_route_rt = None


def route_linear(M, N, K):
    """The runtime's choice for a bfloat16 product of these sizes: 1 the weight-streaming kernel, 2 the
    tiled tcgen05 kernel (0: neither takes them)."""
    global _route_rt
    from . import native
    if _route_rt is None:
        _route_rt = native.RuntimeStruct()
        _route_rt.tensor_cores, _route_rt.dtype = 1, ops.BF16
    return native.lib().glint_route_linear(ctypes.addressof(_route_rt), M, N, K)


def skinny_supported(M, N, K):
    return 1 <= M <= 16 and N >= 1 and K >= 64 and K % 64 == 0


def takes_skinny(M, N, K, force_splits, path):
    """``path`` ("skinny", "tcgen05") names the kernel; without it the runtime's choice."""
    if path == "tcgen05" or force_splits:
        return False
    if path == "skinny":
        if not skinny_supported(M, N, K):
            raise KernelError(f"the weight-streaming product takes up to 16 tokens and K in steps of 64, not M={M} K={K}")
        return True
    return route_linear(M, N, K) == 1


def gemm(a, w, out, cap=0.0, status=None, force_splits=0, path=None):
    """out[M, N] = a[M, K] @ w[N, K]^T with bfloat16 operands, float32 accumulation; ``out`` is
    float32 or bfloat16; ``cap`` > 0 applies the soft cap."""
    M, K = a.shape
    N = w.shape[0]
    ops.require(a, torch.bfloat16, "a"); ops.require(w, torch.bfloat16, "w"); ops.require(out, None, "out")
    if w.shape[1] != K or tuple(out.shape) != (M, N) or out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError(f"gemm shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if takes_skinny(M, N, K, force_splits, path):
        ops.check(lib().glint_gemm_skinny(ops.ptr(a), ops.ptr(w), ops.ptr(out), int(out.dtype == torch.bfloat16), M, N,
                                          K, cap or 0.0, 0, 0, 0, ops.stream()), "gemm_skinny")
        return
    ws, counters = scratch(a.device)
    st = status if status is not None else counters[-1:]
    ops.check(lib().glint_gemm_tcgen05(ops.ptr(a), ops.ptr(w), ops.ptr(out), int(out.dtype == torch.bfloat16), M, N,
                                       K, N, cap or 0.0, 0, 0, 0, ops.ptr(ws), ops.ptr(counters), ops.ptr(st),
                                       force_splits, ops.stream()), "gemm_tcgen05")


def qkv_rope(a, w_qkv, positions, token_slot, block_table, inv_freq, factor, q_out, k_pool, v_pool, nh, nkv, hd,
             page_size, num_pages, status):
    """q, k, v = a @ w_qkv^T for up to 16 tokens with the rotary encoding and the cache write in the
    product's epilogue: rotated q goes to ``q_out`` [M, nh * hd], rotated k and v into the pages named
    by ``block_table`` at each token's position (``k_pool`` None: q only)."""
    M, K = a.shape
    ops.require(a, torch.bfloat16, "a"); ops.require(w_qkv, torch.bfloat16, "w_qkv")
    ops.require(q_out, torch.bfloat16, "q_out"); ops.require(k_pool, torch.bfloat16, "k_pool")
    ops.require(v_pool, torch.bfloat16, "v_pool"); ops.require(inv_freq, torch.float32, "inv_freq")
    ops.require(positions, torch.int32, "positions"); ops.require(token_slot, torch.int32, "token_slot")
    ops.require(block_table, torch.int32, "block_table")
    if w_qkv.shape != ((nh + 2 * nkv) * hd, K) or tuple(q_out.shape) != (M, nh * hd) or inv_freq.numel() != hd // 2:
        raise KernelError(f"qkv_rope shapes do not fit: a {tuple(a.shape)}, w {tuple(w_qkv.shape)}, "
                          f"q_out {tuple(q_out.shape)}, heads {nh}/{nkv} x {hd}")
    ops.check(lib().glint_gemm_skinny_rope(ops.ptr(a), ops.ptr(w_qkv), M, K, ops.ptr(positions), ops.ptr(token_slot),
                                           ops.ptr(block_table), block_table.shape[1], ops.ptr(inv_freq), factor,
                                           ops.ptr(q_out), ops.ptr(k_pool), ops.ptr(v_pool), nh, nkv, hd, page_size,
                                           num_pages, ops.ptr(status), ops.stream()), "gemm_skinny_rope")


def qkv_rope_tiled_supported(M, K, hd, rotary_dim, heads, min_blocks=None):
    """The tiled q/k/v product with the rotary epilogue: head sizes in steps of 256 (a thread holds
    features j and j + hd/2 of a head), whole-head rotation, K in steps of 8, and, as its grid is heads x
    token tiles with K unsplit, enough tokens for ``min_blocks`` blocks (default: half of the SMs)."""
    if not (M >= 1 and K % 8 == 0 and hd >= 256 and hd % 256 == 0 and rotary_dim == hd):
        return False
    mb = sm_count() // 2 if min_blocks is None else min_blocks
    head_tiles = heads * (hd // 256)
    return head_tiles * -(-M // 128) >= mb          # the kernel takes tiles of 256 tokens if they suffice, else of 128


def qkv_rope_tiled(a, w_qkv, trig, positions, token_seq, block_table, q_out, k_pool, v_pool, nh, nkv, hd, page_size,
                   num_pages, status, min_blocks=None):
    """As ``qkv_rope`` for any number of tokens on the tiled kernel; ``trig`` [M, hd/2, 2] float32 holds
    (cos, sin) of every token's angles (``ops.rope_table``)."""
    M, K = a.shape
    ops.require(a, torch.bfloat16, "a"); ops.require(w_qkv, torch.bfloat16, "w_qkv")
    ops.require(q_out, torch.bfloat16, "q_out"); ops.require(k_pool, torch.bfloat16, "k_pool")
    ops.require(v_pool, torch.bfloat16, "v_pool"); ops.require(trig, torch.float32, "trig")
    ops.require(positions, torch.int32, "positions"); ops.require(token_seq, torch.int32, "token_seq")
    ops.require(block_table, torch.int32, "block_table")
    if (w_qkv.shape != ((nh + 2 * nkv) * hd, K) or tuple(q_out.shape) != (M, nh * hd)
            or tuple(trig.shape) != (M, hd // 2, 2)):
        raise KernelError(f"qkv_rope_tiled shapes do not fit: a {tuple(a.shape)}, w {tuple(w_qkv.shape)}, "
                          f"q_out {tuple(q_out.shape)}, trig {tuple(trig.shape)}, heads {nh}/{nkv} x {hd}")
    ops.check(lib().glint_gemm_tcgen05_rope(ops.ptr(a), ops.ptr(w_qkv), M, K, ops.ptr(trig), ops.ptr(positions),
                                            ops.ptr(token_seq), ops.ptr(block_table), block_table.shape[1],
                                            ops.ptr(q_out), ops.ptr(k_pool), ops.ptr(v_pool), nh, nkv, hd, page_size,
                                            num_pages, sm_count() // 2 if min_blocks is None else min_blocks,
                                            ops.ptr(status), ops.stream()), "gemm_tcgen05_rope")


def gemm_gated(a, w_gate_up, out, activation, status=None, force_splits=0, path=None):
    """out[M, I] (bfloat16) = act(a @ w[:I]^T) * (a @ w[I:]^T) for w_gate_up [2I, K], in one kernel."""
    M, K = a.shape
    I = w_gate_up.shape[0] // 2
    ops.require(a, torch.bfloat16, "a"); ops.require(w_gate_up, torch.bfloat16, "w"); ops.require(out, torch.bfloat16, "out")
    if w_gate_up.shape[1] != K or tuple(out.shape) != (M, I):
        raise KernelError(f"gated gemm shapes do not fit: a {tuple(a.shape)}, w {tuple(w_gate_up.shape)}, "
                          f"out {tuple(out.shape)}")
    if takes_skinny(M, I, K, force_splits, path):
        ops.check(lib().glint_gemm_skinny(ops.ptr(a), ops.ptr(w_gate_up), ops.ptr(out), 1, M, I, K, 0.0, 1, I,
                                          ops.ACTIVATIONS[activation], ops.stream()), "gemm_skinny (gated)")
        return
    ws, counters = scratch(a.device)
    st = status if status is not None else counters[-1:]
    ops.check(lib().glint_gemm_tcgen05(ops.ptr(a), ops.ptr(w_gate_up), ops.ptr(out), 1, M, I, K, 2 * I, 0.0, 1, I,
                                       ops.ACTIVATIONS[activation], ops.ptr(ws), ops.ptr(counters), ops.ptr(st),
                                       force_splits, ops.stream()), "gemm_tcgen05 (gated)")


def decode_supported(nh, nkv, hd, page_size):
    """Sizes the single-token attention kernels take (three stages of a page of keys and values have to fit a
    block's shared memory: pages of up to 64 tokens at head size 256)."""
    if nkv <= 0:
        return False
    return bool(lib().glint_attention_decode_supported(nh, nkv, hd, page_size))


def prefill_supported(nh, nkv, hd):
    return nkv > 0 and nh % nkv == 0 and nh // nkv <= 64 and hd % 16 == 0 and 16 <= hd <= 256


_sm_count = {}


def sm_count(device=None):
    """Streaming multiprocessors of the device (asked once)."""
    device = torch.cuda.current_device() if device is None else device
    n = _sm_count.get(device)
    if n is None:
        n = _sm_count[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def decode_splits(tokens, nkv, max_context, sms=None, uneven=0):
    """How many blocks share the keys of one token in the split attention kernel (the runtime's choice).
    ``uneven``: the contexts add up to about (tokens x max_context) >> uneven."""
    from . import native
    return native.lib().glint_decode_splits(tokens, nkv, max_context, uneven, sms or sm_count())


def decode_streams(tokens, nh, nkv, max_context, sms=None, uneven=0):
    """True when single tokens of these counts take the kernel that shares all pages of the launch evenly among
    its blocks (the runtime's choice), False when every (token, kv head) gets a cluster of ``decode_splits`` blocks."""
    from . import native
    return bool(native.lib().glint_decode_streams(tokens, nh, nkv, max_context, uneven, sms or sm_count()))


def attention_decode(q, k_pool, v_pool, positions, token_seq, block_table, out, nh, nkv, hd, page_size, num_pages,
                     multiplier, cap, window, status, splits, tokens=None):
    """Every token attends alone (split over its keys): right for any batch, meant for single tokens.
    ``tokens``: only the first so many rows of ``q``."""
    T = q.shape[0] if tokens is None else tokens
    ops.require(q, torch.bfloat16, "q"); ops.require(k_pool, torch.bfloat16, "k_pool")
    ops.require(v_pool, torch.bfloat16, "v_pool"); ops.require(out, torch.bfloat16, "out")
    ops.check(lib().glint_attention_decode(ops.ptr(q), ops.ptr(k_pool), ops.ptr(v_pool), ops.ptr(positions),
                                           ops.ptr(token_seq), ops.ptr(block_table), block_table.shape[1],
                                           ops.ptr(out), T, nh, nkv, hd, page_size, num_pages, multiplier,
                                           cap or 0.0, window or 0, splits, ops.ptr(status), ops.stream()),
              "attention_decode")


def stream_workspace_floats(blocks, nh, nkv, hd):
    """Floats of workspace a launch of ``attention_decode_stream`` over ``blocks`` blocks needs."""
    fn = lib().lib.glint_attention_decode_stream_workspace
    fn.restype = c_longlong
    return int(fn(blocks, nh, nkv, hd))


def attention_decode_stream_plan(positions, token_seq, tokens, window, page_size, hd, nkv, blocks, min_pages=8,
                                 pair_cost=-1):
    """Plans a launch of ``attention_decode_stream``: (starts [blocks, 2, 4] int32, header [2] int32 = units per
    block and units in all, blocks).  A unit is a page; every (token, kv head) pair counts ``pair_cost`` more
    (default: what the runtime takes for pages of this size)."""
    starts = torch.empty(blocks, 2, 4, dtype=torch.int32, device=positions.device)
    header = torch.zeros(2, dtype=torch.int32, device=positions.device)
    ops.check(lib().glint_attention_decode_stream_plan(ops.ptr(positions), ops.ptr(token_seq), tokens, window or 0,
                                                       page_size, hd, nkv, blocks, min_pages, pair_cost,
                                                       ops.ptr(starts), ops.ptr(header), ops.stream()),
              "attention_decode_stream_plan")
    return starts, header, blocks


def attention_decode_stream(q, k_pool, v_pool, positions, token_seq, block_table, out, nh, nkv, hd, page_size,
                            num_pages, multiplier, cap, window, status, plan, partials, arrive, tokens=None):
    """``attention_decode`` with the pages of the whole launch shared evenly among the blocks (``plan`` from
    ``attention_decode_stream_plan`` with the same positions, window, page size and kv heads): ``partials``
    float32 [``stream_workspace_floats``], ``arrive`` int32 [tokens * nkv], zero before the first launch."""
    T = q.shape[0] if tokens is None else tokens
    starts, header, blocks = plan
    ops.require(q, torch.bfloat16, "q"); ops.require(k_pool, torch.bfloat16, "k_pool")
    ops.require(v_pool, torch.bfloat16, "v_pool"); ops.require(out, torch.bfloat16, "out")
    if partials.numel() < stream_workspace_floats(blocks, nh, nkv, hd) or arrive.numel() < T * nkv:
        raise KernelError("attention_decode_stream: the workspace is too small for this launch")
    ops.check(lib().glint_attention_decode_stream(ops.ptr(q), ops.ptr(k_pool), ops.ptr(v_pool), ops.ptr(positions),
                                                  ops.ptr(token_seq), ops.ptr(block_table), block_table.shape[1],
                                                  ops.ptr(out), T, nh, nkv, hd, page_size, num_pages, multiplier,
                                                  cap or 0.0, window or 0, blocks, ops.ptr(starts),
                                                  ops.ptr(partials), ops.ptr(arrive), 0, ops.ptr(status), ops.stream()),
              "attention_decode_stream")


def attention_prefill(q, k_pool, v_pool, cu_seqlens, seq_start, block_table, out, n_seqs, max_q_len, nh, nkv, hd,
                      page_size, num_pages, multiplier, cap, window, status):
    """Flash attention of prompt portions (any mix of lengths, single tokens included)."""
    ops.require(q, torch.bfloat16, "q"); ops.require(k_pool, torch.bfloat16, "k_pool")
    ops.require(v_pool, torch.bfloat16, "v_pool"); ops.require(out, torch.bfloat16, "out")
    ops.check(lib().glint_attention_prefill(ops.ptr(q), ops.ptr(k_pool), ops.ptr(v_pool), ops.ptr(cu_seqlens),
                                            ops.ptr(seq_start), ops.ptr(block_table), block_table.shape[1],
                                            ops.ptr(out), n_seqs, max_q_len, nh, nkv, hd, page_size, num_pages,
                                            multiplier, cap or 0.0, window or 0, ops.ptr(status), ops.stream()),
              "attention_prefill")


def tcgen05_attention_supported(nh, nkv, hd, page_size):
    return (nkv > 0 and nh % nkv == 0 and nh // nkv <= 128 and hd % 16 == 0 and 16 <= hd <= 256
            and page_size in (16, 32, 64))


def attention_tcgen05(q, k_pool, v_pool, cu_seqlens, seq_start, block_table, out, n_seqs, max_q_len, nh, nkv, hd,
                      page_size, num_pages, multiplier, cap, window, status):
    """Flash attention of prompt portions on tcgen05 tensor cores (any mix of lengths)."""
    ops.require(q, torch.bfloat16, "q"); ops.require(k_pool, torch.bfloat16, "k_pool")
    ops.require(v_pool, torch.bfloat16, "v_pool"); ops.require(out, torch.bfloat16, "out")
    ops.check(lib().glint_attention_tcgen05(ops.ptr(q), ops.ptr(k_pool), ops.ptr(v_pool), ops.ptr(cu_seqlens),
                                            ops.ptr(seq_start), ops.ptr(block_table), block_table.shape[1],
                                            ops.ptr(out), q.shape[0], n_seqs, max_q_len, nh, nkv, hd, page_size,
                                            num_pages, multiplier, cap or 0.0, window or 0, ops.ptr(status),
                                            ops.stream()), "attention_tcgen05")
