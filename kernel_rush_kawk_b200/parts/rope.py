"""Rotate-half rotary position encoding: the tables.

inv_freq_i = 1 / theta^(2i/D) for i < D/2 and angle[p, i] = p * inv_freq_i, both
in 32-bit; cos and sin are taken in 32-bit and only then stored in the path's
dtype (engine/model.py:78-93 of willzeng274/kernel-rush-kawk). The reference
stores cat(angle, angle) so that column i and column i + D/2 share an angle;
here only the distinct half [positions, D/2] is kept and the kernel reads
column i for both halves. The rotation itself happens in the mixer's fused
q/k-norm + RoPE + cache-write kernel, which takes these tables as input.
"""

from __future__ import annotations

import torch

from .base import PositionEncoding, register_position


class RotaryTable(PositionEncoding):
    """params: theta, dim (the rotated width, here the head size), positions."""

    def __init__(self, params):
        super().__init__(params)
        self.theta = float(params["theta"])
        self.dim = int(params["dim"])
        self.positions = int(params["positions"])
        if self.dim % 2:
            raise ValueError(f"rotary dim must be even, got {self.dim}")
        self.cos = self.sin = None

    def bind(self, tensors, runtime):
        self.cos, self.sin = self.build(self.positions, runtime.device, runtime.dtype)

    def build(self, positions: int, device, dtype):
        # the few inverse frequencies are computed on the host, so that the table does not
        # depend on a device's pow(); products, cos and sin run on the device in float32
        exponent = torch.arange(0, self.dim, 2, dtype=torch.int64).to(torch.float32) / self.dim
        inv_freq = (1.0 / (self.theta ** exponent)).to(device)
        pos = torch.arange(positions, dtype=torch.float32, device=device)
        angle = pos[:, None] * inv_freq[None, :]
        return angle.cos().to(dtype).contiguous(), angle.sin().to(dtype).contiguous()

    def rotary_tables(self):
        return self.cos, self.sin


register_position("rope", RotaryTable)
