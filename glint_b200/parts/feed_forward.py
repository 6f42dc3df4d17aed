"""Dense gated feed-forward: down(act(gate x) * (up x)) without biases.

``activation`` 'gelu_tanh' is Gemma's GeGLU (src/transformer/forward.rs:273-318 with
src/tensor/ops.rs:169-178); 'silu' is the SwiGLU of the reference's other families
(src/tensor/ops.rs:157-164).  Gate and up are stacked into one matrix at load (exact).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorNeed, run_lowered
from .registry import register_part


class GatedFeedForward(Part):
    def __init__(self, rt, params, tensors):
        super().__init__(rt, params, tensors)
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self.activation = params.get("activation", "gelu_tanh")
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation '{self.activation}' is not one of {sorted(ops.ACTIVATIONS)}")
        self.w_gate_up = None
        self.w_down = None

    def needs(self):
        n = self.names
        return [TensorNeed(n["gate"], (self.intermediate_size, self.hidden_size)),
                TensorNeed(n["up"], (self.intermediate_size, self.hidden_size)),
                TensorNeed(n["down"], (self.hidden_size, self.intermediate_size))]

    def bind(self, tensors):
        n = self.names
        self.w_gate_up = torch.cat([tensors[n["gate"]], tensors[n["up"]]], dim=0).contiguous()
        self.w_down = tensors[n["down"]]

    def lower(self, prog, normed):
        """Two operations: the gated product (one kernel with the activation in its epilogue where the
        runtime has one, else the product and the activation), and the down product.  Returns the value
        float32 [tokens, hidden]."""
        act = prog.value("ffn.act", self.intermediate_size)
        # the two-kernel path keeps gate and up in 32-bit between the kernels
        fused = self.rt.tensor_cores and self.w_gate_up.dtype == torch.bfloat16 and self.hidden_size % 8 == 0
        tmp = None if fused else prog.value("ffn.gate_up", 2 * self.intermediate_size, torch.float32)
        prog.linear(normed, self.w_gate_up, act, gated=self.activation, tmp=tmp)
        y = prog.value("ffn.y", self.hidden_size, torch.float32)
        prog.linear(act, self.w_down, y)
        return y

    def forward(self, normed, ctx):
        return run_lowered(self.rt, ctx, normed.shape[0], lambda prog: self.lower(prog, prog.bind(normed)))

    def parameter_bytes(self):
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def flops(self, tokens):
        return 2 * tokens * (self.w_gate_up.numel() + self.w_down.numel())


register_part("feed_forward", "gated", GatedFeedForward)
