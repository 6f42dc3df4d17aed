"""The device, the dtype and the kernel choice that all parts of one model share."""
from __future__ import annotations

import torch

from . import ops
from .errors import KernelError

DTYPES = {"float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
          "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}

_STATUS_TEXT = {1: "a token id lies outside the embedding table",
                2: "a token's position has no page in its block table (cache write)",
                3: "a key's position has no page in its block table (attention read)",
                4: "a bounded device-side wait ran out"}


def parse_dtype(dtype):
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise KernelError(f"the engine runs in float32 or bfloat16, not {dtype}")
        return dtype
    try:
        return DTYPES[str(dtype).lower()]
    except KeyError:
        raise KernelError(f"unknown dtype '{dtype}' (known: float32, bfloat16)") from None


class Runtime:
    """``dtype`` float32 means the true 32-bit path: CUDA-core products, no tensor cores.
    ``kernels`` is 'auto' (tensor-core kernels where they exist, for bfloat16) or 'plain'."""

    def __init__(self, device="cuda:0", dtype=torch.bfloat16, kernels="auto"):
        self.device = torch.device(device)
        self.dtype = parse_dtype(dtype)
        if kernels not in ("auto", "plain"):
            raise KernelError(f"kernels must be 'auto' or 'plain', not '{kernels}'")
        self.kernels = kernels
        if self.device.type != "cuda":
            raise KernelError(f"the engine needs a CUDA device, not '{self.device}': there is no CPU path")
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is available: the engine has no CPU path")
        ops.core()  # build or load the kernels now, loudly
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.shared = {}          # what several parts of a model share (a table of rotation angles), by key
        from . import native
        self.native = native.make_runtime_struct(self)     # the C++ side's view of this runtime
        self._backing = {}        # (role, dtype) -> flat tensor
        self._views = {}          # (role, shape, dtype) -> view of the backing tensor
        self._retired = []        # outgrown backing tensors: captured launches may still point into them

    @property
    def tensor_cores(self):
        return self.dtype == torch.bfloat16 and self.kernels == "auto"

    def single_token_attention(self, which):
        """Which of the two single-token attention kernels steps take from now on: "routed" (the runtime's
        choice, the default), "stream" (the kernel that shares all pages of a launch evenly among its blocks,
        wherever it takes the sizes) or "cluster" (a cluster of blocks per token and kv head, always).  For
        tests and measurements; graphs captured before the call keep what they captured."""
        modes = {"routed": 0, "stream": 1, "cluster": 2}
        if which not in modes:
            raise KernelError(f"single_token_attention: {which!r} is none of {sorted(modes)}")
        scratch = getattr(self, "attn_scratch", None)
        if scratch is not None:
            scratch[0].mode = modes[which]

    def empty(self, shape, dtype=None):
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    def buffer(self, role, shape, dtype=None):
        """A tensor of this shape for a value that lives from one kernel to the next within a step.  One
        allocation per role serves every layer and every step: the kernels of a step run in order on
        one stream, so whatever read the role's previous value was issued before the kernel that
        writes the next one.  Two values that are alive at the same time need different roles; a part
        that cannot promise that allocates with ``empty``.  (A step of a few hundred tokens is bound by
        the host, and seven allocations per layer were a sixth of its time.)"""
        dtype = dtype or self.dtype
        key = (role, shape, dtype)
        view = self._views.get(key)
        if view is None:
            n = 1
            for d in shape:
                n *= int(d)
            base = self._backing.get((role, dtype))
            if base is None or base.numel() < n:
                grown = 2 * base.numel() if base is not None else 1      # what was outgrown stays allocated: keep it a fraction
                if base is not None:
                    self._retired.append(base)
                    self._views = {k: v for k, v in self._views.items() if k[0] != role or k[2] != dtype}
                base = torch.empty(max(n, grown), dtype=dtype, device=self.device)
                self._backing[(role, dtype)] = base
            if len(self._views) > 512:
                self._views.clear()
            view = base[:n].view(shape)
            self._views[key] = view
        return view

    def check_status(self):
        """Read the device status word (synchronizes); raise if a kernel reported a fault."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise KernelError(f"a kernel reported: {_STATUS_TEXT.get(code, f'status {code}')}")
