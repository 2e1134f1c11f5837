"""RMSNorm with the residual add folded in.

y = round(round(x * rsqrt(mean(x^2) + eps)) * w): the normalised value is
rounded to the path's dtype before the weight multiply, as the reference does
(engine/kernels/rmsnorm.py:30-45 of willzeng274/kernel-rush-kawk); with a
pending branch, s = round(x + branch) becomes the new residual stream first
(engine/kernels/add_rmsnorm.py:21-29). Mean, rsqrt and the products are 32-bit.
"""

from __future__ import annotations

from .base import Norm, Stream, TensorSpec, register_norm


class Normed:
    """Rows that a norm produces, computed on demand.

    A consumer either calls ``tensor()`` (the norm kernel runs once) or hands the
    object to ``ops.linear`` and friends, which may fold the add and the norm
    into their own prologue when few rows are in flight. Either way the new
    residual stream ``x_new`` is written exactly once."""

    __slots__ = ("ops", "x", "branch", "gain", "eps", "x_new", "_rows")

    def __init__(self, ops, x, branch, gain, eps, x_new):
        self.ops = ops
        self.x = x
        self.branch = branch
        self.gain = gain
        self.eps = eps
        self.x_new = x_new
        self._rows = None

    @property
    def done(self) -> bool:
        return self._rows is not None

    @property
    def shape(self):
        return self.x.shape

    def tensor(self):
        if self._rows is None:
            if self.branch is None:
                self._rows = self.ops.rmsnorm(self.x, self.gain, self.eps)
            else:
                self._rows = self.ops.add_rmsnorm(self.x, self.branch, self.gain, self.eps, self.x_new)
        return self._rows

    def mark_fused(self, rows=True) -> None:
        """Called by a kernel wrapper that did the add and the norm itself."""
        self._rows = rows


class RMSNorm(Norm):
    """params: size, eps."""

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.gain = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.size,), "gain")}

    def bind(self, tensors, runtime):
        self.gain = tensors["weight"]
        self.ops = runtime.ops

    def forward(self, ctx, stream: Stream) -> Normed:
        if stream.branch is None:
            return Normed(self.ops, stream.x, None, self.gain, self.eps, stream.x)
        x_new = ctx.ops.empty_like(stream.x)
        normed = Normed(self.ops, stream.x, stream.branch, self.gain, self.eps, x_new)
        stream.x = x_new
        stream.branch = None
        return normed


register_norm("rmsnorm", RMSNorm)
