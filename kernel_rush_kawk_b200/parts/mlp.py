"""SwiGLU feed-forward.

gu = h Wgu^T with Wgu = cat(Wgate, Wup) (engine/model.py:116,301 of
willzeng274/kernel-rush-kawk); a = round(round(silu(g)) * u) with
silu(g) = g / (1 + exp(-g)) in 32-bit (engine/kernels/swiglu.py:21-24,
engine/kernels/gemm.py:108-113); d = a Wdown^T. No biases.
"""

from __future__ import annotations

import torch

from .base import FeedForward, TensorSpec, register_feed_forward


class SwiGLU(FeedForward):
    """params: hidden, intermediate."""

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden"])
        self.intermediate = int(params["intermediate"])
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        return {
            "gate_proj": TensorSpec((self.intermediate, self.hidden)),
            "up_proj": TensorSpec((self.intermediate, self.hidden)),
            "down_proj": TensorSpec((self.hidden, self.intermediate)),
        }

    def bind(self, tensors, runtime):
        self.w_gate_up = torch.cat([tensors["gate_proj"], tensors["up_proj"]], dim=0).contiguous()
        self.w_down = tensors["down_proj"].contiguous()

    def forward(self, ctx, h):
        act = ctx.ops.gate_up_swiglu(h, self.w_gate_up, self.intermediate)
        return ctx.ops.linear(act, self.w_down)


register_feed_forward("swiglu", SwiGLU)
