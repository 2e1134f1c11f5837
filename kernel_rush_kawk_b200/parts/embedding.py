"""Token embedding and the output head.

x0[r] = table[ids[r]] (engine/model.py:291,315 of willzeng274/kernel-rush-kawk);
logits = h W^T at the wanted rows only, with W the embedding table when the
head is tied (engine/model.py:103-107,303). Logits leave in 32-bit.
"""

from __future__ import annotations

from .base import Embedding, Head, TensorSpec, register_embedding, register_head


class TokenEmbedding(Embedding):
    """params: vocab, hidden."""

    def __init__(self, params):
        super().__init__(params)
        self.vocab = int(params["vocab"])
        self.hidden = int(params["hidden"])
        self.table = None

    def tensor_specs(self):
        return {"table": TensorSpec((self.vocab, self.hidden), "table")}

    def bind(self, tensors, runtime):
        self.table = tensors["table"]

    def forward(self, ctx):
        return ctx.ops.embed(self.table, ctx.batch.tokens, ctx.batch.n_rows)


class OutputHead(Head):
    """params: vocab, hidden. The plan points "weight" at the embedding table's
    checkpoint name when the head is tied."""

    def __init__(self, params):
        super().__init__(params)
        self.vocab = int(params["vocab"])
        self.hidden = int(params["hidden"])
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab, self.hidden), "table")}

    def bind(self, tensors, runtime):
        self.weight = tensors["weight"]

    def forward(self, ctx, h):
        """h: normalised rows (a Normed or a tensor) of the wanted positions."""
        return ctx.ops.linear(h, self.weight, out_float32=True)


register_embedding("token_embedding", TokenEmbedding)
register_head("output_head", OutputHead)
