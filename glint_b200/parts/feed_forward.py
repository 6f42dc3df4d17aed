"""Dense gated feed-forward: down(act(gate x) * (up x)) without biases.

``activation`` 'gelu_tanh' is Gemma's GeGLU (src/transformer/forward.rs:273-318 with
src/tensor/ops.rs:169-178); 'silu' is the SwiGLU of the reference's other families
(src/tensor/ops.rs:157-164).  Gate and up are stacked into one matrix at load (exact).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorNeed
from .linear import linear
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

    def forward(self, normed, ctx):
        rt = self.rt
        T = normed.shape[0]
        act = rt.buffer("ffn.act", (T, self.intermediate_size))
        fused = False
        if rt.tensor_cores:
            from .. import ops_tensor
            if ops_tensor.gemm_supported(T, self.intermediate_size, self.hidden_size):
                ops_tensor.gemm_gated(normed, self.w_gate_up, act, self.activation, rt.status)
                fused = True
        if not fused:
            gu = linear(rt, normed, self.w_gate_up, out=rt.buffer("ffn.gate_up", (T, 2 * self.intermediate_size), torch.float32))
            ops.gated_act(gu, act, self.activation)
        return linear(rt, act, self.w_down, out=rt.buffer("ffn.y", (T, self.hidden_size), torch.float32))

    def parameter_bytes(self):
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def flops(self, tokens):
        return 2 * tokens * (self.w_gate_up.numel() + self.w_down.numel())


register_part("feed_forward", "gated", GatedFeedForward)
