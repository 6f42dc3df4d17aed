"""Python face of the native step runtime (``csrc/runtime.h``): the structures it shares with the
C++ side, and ``Program``, through which parts are lowered into operations that one native call runs.

A part describes its work by calling the methods of a ``Program`` (``linear``, ``qkv_rope``,
``attention``, ``rmsnorm`` ...) on ``Value`` objects, the tensors between kernels.  The same code
serves both ways of running: a model is lowered once into one long program that every step runs with
one call into the C++ executor (the stretch between two ``host`` operations, which are Python
callables for parts that are not lowered), and a part's own ``forward`` lowers just itself into a
short program and runs it at once.  Which kernel an operation takes is decided in C++ for both.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_void_p

import torch

from . import ops
from .errors import KernelError

MAX_GROUPS = 8

OP_EMBED, OP_RMSNORM, OP_ADD_RMSNORM, OP_LINEAR, OP_QKV_ROPE, OP_ROPE_STORE, OP_ATTENTION, OP_HOST = range(1, 9)


class StepStruct(Structure):
    _fields_ = [("id", c_longlong),
                ("num_tokens", c_int), ("num_seqs", c_int), ("max_seq_len", c_int), ("max_context", c_int),
                ("leading_single", c_int), ("leading_single_context", c_int), ("num_logit_rows", c_int),
                ("num_groups", c_int), ("uneven", c_int),
                ("token_ids", c_void_p), ("positions", c_void_p), ("token_seq", c_void_p), ("seq_slot", c_void_p),
                ("seq_start", c_void_p), ("cu_seqlens", c_void_p), ("logit_rows", c_void_p),
                ("block_table", c_void_p * MAX_GROUPS), ("max_pages", c_int * MAX_GROUPS)]


class TensorEntries(Structure):
    _fields_ = [(name, c_void_p) for name in ("gemm_tcgen05", "gemm_skinny", "gemm_tcgen05_rope", "gemm_skinny_rope",
                                              "attention_decode", "attention_decode_stream_plan",
                                              "attention_decode_stream", "attention_prefill", "attention_tcgen05")]


ATTN_PLANS = 8


class AttnScratchStruct(Structure):
    """``GlintAttnScratch`` of csrc/runtime.h."""
    _fields_ = [("mode", c_int), ("early_off", c_int), ("blocks", c_int), ("starts", c_void_p),
                ("headers", c_void_p), ("partials", c_void_p), ("partial_floats", c_longlong), ("arrive", c_void_p), ("arrive_ints", c_int), ("next", c_int),
                ("plan_step", c_longlong * ATTN_PLANS), ("plan_tokens", c_int * ATTN_PLANS),
                ("plan_window", c_int * ATTN_PLANS), ("plan_page", c_int * ATTN_PLANS), ("plan_nkv", c_int * ATTN_PLANS),
                ("plan_hd", c_int * ATTN_PLANS)]


class RuntimeStruct(Structure):
    _fields_ = [("tensor_cores", c_int), ("dtype", c_int), ("sms", c_int), ("status", c_void_p),
                ("workspace", c_void_p), ("counters", c_void_p), ("attn", POINTER(AttnScratchStruct)),
                ("tensor", TensorEntries)]


class ViewStruct(Structure):
    _fields_ = [("k", c_void_p), ("v", c_void_p), ("page_size", c_int), ("num_pages", c_int), ("group", c_int),
                ("writes", c_int)]


class TrigStruct(Structure):
    _fields_ = [("table", c_void_p), ("filled_step", c_longlong)]


class OpStruct(Structure):
    _fields_ = [("kind", c_int), ("rows", c_int), ("p", c_void_p * 10), ("i", c_longlong * 10), ("f", c_float * 6)]


_bound = False


def lib():
    """The core library with the runtime's entry points typed."""
    global _bound
    core = ops.core().lib
    if not _bound:
        core.glint_program_create.restype = c_void_p
        core.glint_program_create.argtypes = [c_void_p]
        core.glint_program_destroy.restype = None
        core.glint_program_destroy.argtypes = [c_void_p]
        core.glint_program_add.restype = c_int
        core.glint_program_add.argtypes = [c_void_p, POINTER(OpStruct)]
        core.glint_program_run.restype = c_int
        core.glint_program_run.argtypes = [c_void_p, POINTER(StepStruct), c_int, c_int, POINTER(c_int), c_void_p]
        core.glint_route_linear.restype = c_int
        core.glint_route_linear.argtypes = [c_void_p, c_int, c_int, c_int]
        core.glint_decode_splits.restype = c_int
        core.glint_decode_splits.argtypes = [c_int, c_int, c_int, c_int, c_int]
        core.glint_decode_streams.restype = c_int
        core.glint_decode_streams.argtypes = [c_int, c_int, c_int, c_int, c_int, c_int]
        _bound = True
    return core


def make_runtime_struct(rt):
    """The C++ side's view of a ``Runtime``: dtype, kernel choice, SM count, status word, and, for the
    tensor-core kernels, the split-K scratch and the entry points of their library."""
    s = RuntimeStruct()
    s.tensor_cores = 1 if rt.tensor_cores else 0
    s.dtype = ops.dtype_code(rt.dtype)
    s.sms = torch.cuda.get_device_properties(rt.device).multi_processor_count
    s.status = rt.status.data_ptr()
    if rt.tensor_cores:
        from . import ops_tensor
        tl = ops_tensor.lib().lib
        ws, counters = ops_tensor.scratch(rt.device)
        s.workspace, s.counters = ws.data_ptr(), counters.data_ptr()
        for name, _ in TensorEntries._fields_:
            setattr(s.tensor, name, ctypes.cast(getattr(tl, "glint_" + name), c_void_p).value)
        # scratch of the single-token attention that shares a launch's pages evenly: two blocks per SM, partial
        # results of up to 8 query heads of 256 per kv head, counters for 1024 tokens x 64 kv heads
        a = AttnScratchStruct()
        a.blocks = 2 * s.sms
        a.partial_floats = ops_tensor.stream_workspace_floats(a.blocks, 8, 1, 256)
        a.arrive_ints = 65536
        tensors = (torch.empty(ATTN_PLANS * a.blocks * 8, dtype=torch.int32, device=rt.device),
                   torch.zeros(ATTN_PLANS * 2, dtype=torch.int32, device=rt.device),
                   torch.empty(a.partial_floats, dtype=torch.float32, device=rt.device),
                   torch.zeros(a.arrive_ints, dtype=torch.int32, device=rt.device))
        a.starts, a.headers, a.partials, a.arrive = (t.data_ptr() for t in tensors)
        for i in range(ATTN_PLANS):
            a.plan_step[i] = -1
        rt.attn_scratch = (a, tensors)             # owned by the runtime: the structure below only points at them
        s.attn = ctypes.pointer(a)
    return s


def fill_step(step, ctx, step_id):
    """Copy a ``StepContext`` into the structure the executor reads."""
    step.id = step_id
    step.num_tokens, step.num_seqs = ctx.num_tokens, ctx.num_seqs
    step.max_seq_len, step.max_context = ctx.max_seq_len, ctx.max_context
    step.leading_single, step.leading_single_context = ctx.leading_single, ctx.leading_single_context
    step.num_logit_rows = ctx.num_logit_rows
    step.uneven = ctx.uneven
    tables = ctx.block_tables
    if len(tables) > MAX_GROUPS:
        raise KernelError(f"a step carries block tables of {len(tables)} cache groups; the runtime takes {MAX_GROUPS}")
    step.num_groups = len(tables)
    step.token_ids, step.positions, step.token_seq = ctx.token_ids.data_ptr(), ctx.positions.data_ptr(), ctx.token_seq.data_ptr()
    step.seq_slot, step.seq_start, step.cu_seqlens = ctx.seq_slot.data_ptr(), ctx.seq_start.data_ptr(), ctx.cu_seqlens.data_ptr()
    step.logit_rows = ctx.logit_rows.data_ptr()
    for g, t in enumerate(tables):
        step.block_table[g] = t.data_ptr()
        step.max_pages[g] = t.shape[1]
    return step


class Value:
    """A tensor between two operations: ``tensor`` is [capacity rows, width]; operations run on its first
    rows (the step's tokens, or its wanted logit rows)."""
    __slots__ = ("tensor", "width")

    def __init__(self, tensor):
        self.tensor = tensor
        self.width = tensor.shape[1]

    @property
    def dtype(self):
        return self.tensor.dtype

    @property
    def ptr(self):
        return self.tensor.data_ptr()

    def rows(self, n):
        return self.tensor[:n]


_step_ids = 0


def next_step_id():
    global _step_ids
    _step_ids += 1
    return _step_ids


class Program:
    """A list of operations over fixed device memory, run for a step's tokens by the C++ executor.

    ``capacity`` is the most tokens a step may bring (values are allocated for it); ``groups`` is the cache
    manager's list of paged groups, in the order of the step's block tables.  ``host(fn)`` puts a Python
    callable ``fn(ctx)`` between two native stretches.
    """

    def __init__(self, rt, capacity, groups=()):
        self.rt = rt
        self.capacity = int(capacity)
        self.groups = list(groups)
        self._lib = lib()
        self.handle = self._lib.glint_program_create(ctypes.addressof(rt.native))
        self.segments = []            # ("native", first, last) or ("host", fn)
        self._open = None             # first operation of the native stretch being built
        self.size = 0
        self._keep = []               # structures the operations point to
        self._views = {}
        self._step = StepStruct()
        self._failed = c_int(0)

    def __del__(self):
        try:
            if self.handle:
                self._lib.glint_program_destroy(self.handle)
                self.handle = None
        except Exception:
            pass

    # ---- values ---------------------------------------------------------------------------------------

    def value(self, role, width, dtype=None):
        """The value of ``role``: one allocation per role and dtype serves every layer (see ``Runtime.buffer``)."""
        return Value(self.rt.buffer(role, (self.capacity, int(width)), dtype))

    def bind(self, tensor):
        """An existing [rows, width] tensor as a value."""
        if tensor.dim() != 2 or not tensor.is_contiguous() or not tensor.is_cuda:
            raise KernelError("a value is a contiguous [rows, width] tensor on the device")
        return Value(tensor)

    def view_struct(self, view):
        s = self._views.get(id(view))
        if s is None:
            s = ViewStruct()
            s.k, s.v = view.k.data_ptr(), view.v.data_ptr()
            s.page_size, s.num_pages = view.page_size, view.num_pages
            s.group = next(i for i, g in enumerate(self.groups) if g is view.group)
            s.writes = 1 if view.writes else 0
            self._views[id(view)] = s
            self._keep.append((s, view))
        return ctypes.addressof(s)

    # ---- operations -----------------------------------------------------------------------------------

    def _add(self, kind, rows=0, p=(), i=(), f=()):
        op = OpStruct()
        op.kind, op.rows = kind, rows
        for k, v in enumerate(p):
            op.p[k] = v or None
        for k, v in enumerate(i):
            op.i[k] = int(v)
        for k, v in enumerate(f):
            op.f[k] = float(v)
        at = self._lib.glint_program_add(self.handle, ctypes.byref(op))
        if at < 0:
            raise KernelError(f"the runtime refused an operation of kind {kind}")
        self.size = at + 1
        if kind != OP_HOST and self._open is None:
            self._open = at
        return at

    def _close(self):
        if self._open is not None:
            self.segments.append(("native", self._open, self.size))
            self._open = None

    def host(self, fn):
        """``fn(ctx)`` runs here, in Python, between the native operations before and after it."""
        self._close()
        self._add(OP_HOST)
        self.segments.append(("host", fn))

    def embed(self, table, out, scale, vocab):
        self._add(OP_EMBED, 0, (table.data_ptr(), out.ptr), (ops.dtype_code(table.dtype), out.width, vocab), (scale,))

    def rmsnorm(self, x, weight, eps, offset, out, logit_rows=False):
        """out = norm(x); with ``logit_rows`` only the step's wanted rows of x, gathered."""
        self._add(OP_RMSNORM, 1 if logit_rows else 0, (x.ptr, weight.data_ptr(), out.ptr),
                  (ops.dtype_code(out.dtype), x.width), (eps, offset))

    def add_rmsnorm(self, x, y, norm_a, out, norm_b):
        """x += norm_a(y); out = norm_b(x).  Norms are (weight, eps, offset) or None; ``out`` may be None."""
        wa, ea, oa = norm_a if norm_a is not None else (None, 0.0, 0.0)
        wb, eb, ob = norm_b if norm_b is not None else (None, 0.0, 0.0)
        self._add(OP_ADD_RMSNORM, 0,
                  (x.ptr, y.ptr, wa.data_ptr() if wa is not None else 0, out.ptr if out is not None else 0,
                   wb.data_ptr() if wb is not None else 0),
                  (ops.dtype_code(out.dtype) if out is not None else ops.F32, x.width), (ea, oa, eb, ob))

    def linear(self, a, w, out, cap=0.0, gated=None, tmp=None, logit_rows=False):
        """out = a w^T (float32), or with ``gated`` (an activation name) act(a w[:N]^T) * (a w[N:]^T) in the
        activation dtype; ``tmp`` [rows, 2N] float32 serves a gated product that no kernel fuses."""
        N = w.shape[0] // 2 if gated else w.shape[0]
        if w.shape[1] != a.width or out.width != N:
            raise KernelError(f"linear: a [*, {a.width}], w {tuple(w.shape)}, out [*, {out.width}] do not fit")
        self._add(OP_LINEAR, 1 if logit_rows else 0, (a.ptr, w.data_ptr(), out.ptr, tmp.ptr if tmp is not None else 0),
                  (1 if out.dtype == torch.bfloat16 else 0, N, w.shape[1], 1 if gated else 0,
                   ops.ACTIVATIONS[gated] if gated else 0), (cap or 0.0,))

    def qkv_rope(self, x, w_qkv, q_out, tmp, view, nh, nkv, hd, inv_freq, factor, rotary_dim, trig):
        self._keep.append(trig)
        self._add(OP_QKV_ROPE, 0, (x.ptr, w_qkv.data_ptr(), q_out.ptr, tmp.ptr if tmp is not None else 0,
                                   self.view_struct(view), inv_freq.data_ptr(),
                                   ctypes.addressof(trig.struct) if trig is not None else 0),
                  (nh, nkv, hd, w_qkv.shape[1], rotary_dim), (factor,))

    def rope_store(self, qkv, q_out, view, nh, nkv, hd, inv_freq, factor, rotary_dim):
        self._add(OP_ROPE_STORE, 0, (qkv.ptr, q_out.ptr, self.view_struct(view), inv_freq.data_ptr()),
                  (nh, nkv, hd, rotary_dim), (factor,))

    def attention(self, q, view, out, nh, nkv, hd, multiplier, cap, window):
        self._add(OP_ATTENTION, 0, (q.ptr, self.view_struct(view), out.ptr), (nh, nkv, hd, window or 0),
                  (multiplier, cap or 0.0))

    # ---- running --------------------------------------------------------------------------------------

    def run(self, ctx):
        """Run every operation for the step ``ctx`` on the current stream."""
        self._close()
        if ctx.num_tokens > self.capacity:
            raise KernelError(f"a step of {ctx.num_tokens} tokens exceeds the program's capacity of {self.capacity}")
        step = fill_step(self._step, ctx, next_step_id())
        stream = ops.stream()
        for seg in self.segments:
            if seg[0] == "host":
                seg[1](ctx)
                continue
            rc = self._lib.glint_program_run(self.handle, ctypes.byref(step), seg[1], seg[2], ctypes.byref(self._failed),
                                             stream)
            if rc != 0:
                raise KernelError(f"operation {self._failed.value} of the program: {ops.error_string(rc)} (code {rc})")


class TrigTable:
    """The table of rotation angles that layers with the same rotary parameters share: filled by the first
    operation of a step that wants it (``GlintTrigTable`` in csrc/runtime.h)."""

    def __init__(self, rt, half):
        self.rt, self.half = rt, half
        self.struct = TrigStruct()
        self.tensor = None
        self.reserve(256)

    def reserve(self, tokens):
        if self.tensor is None or self.tensor.shape[0] < tokens:
            self.tensor = torch.empty((tokens, self.half, 2), dtype=torch.float32, device=self.rt.device)
            self.struct.table = self.tensor.data_ptr()
            self.struct.filled_step = -1
