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

    @property
    def tensor_cores(self):
        return self.dtype == torch.bfloat16 and self.kernels == "auto"

    def empty(self, shape, dtype=None):
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    def check_status(self):
        """Read the device status word (synchronizes); raise if a kernel reported a fault."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise KernelError(f"a kernel reported: {_STATUS_TEXT.get(code, f'status {code}')}")
