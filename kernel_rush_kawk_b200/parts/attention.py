"""Grouped-query attention with per-head q/k RMSNorm and rotary positions.

qkv = h Wqkv^T with Wqkv = cat(Wq, Wk, Wv) (engine/model.py:112-115,295 of
willzeng274/kernel-rush-kawk); every q and k head is normalised over the head
size with one gain shared by all heads and the model's eps, then rotated; v is
stored raw (engine/kernels/rope.py:19-30,139-144); a query at position p sees
keys 0..p (or the last ``window`` of them), scores scaled by 1/sqrt(head_dim),
softmax statistics in 32-bit, q head h reads kv head h // (heads / kv_heads)
(engine/kernels/attention.py:70-73,104-122); the output goes through Wo.

A run that reads another run's cache (``own_cache`` False) has no k/v
projections: it projects, normalises and rotates queries only.
"""

from __future__ import annotations

import math

import torch

from .base import KVNeed, Mixer, TensorSpec, register_mixer


class GQAttention(Mixer):
    """params: hidden, heads, kv_heads, head_dim, eps, qk_norm (bool), window
    (None or int), own_cache (bool), position (a PositionEncoding or None, set by
    the model builder)."""

    graph_safe = True

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.kv_heads = int(p["kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.eps = float(p["eps"])
        self.qk_norm = bool(p.get("qk_norm", True))
        self.window = p.get("window")
        self.own_cache = bool(p.get("own_cache", True))
        self.position = None
        if self.heads % self.kv_heads:
            raise ValueError(f"heads ({self.heads}) must be a multiple of kv_heads ({self.kv_heads})")
        self.scale = 1.0 / math.sqrt(self.head_dim)
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = None

    # -- declarations -----------------------------------------------------
    def tensor_specs(self):
        D = self.head_dim
        specs = {
            "q_proj": TensorSpec((self.heads * D, self.hidden)),
            "o_proj": TensorSpec((self.hidden, self.heads * D)),
        }
        if self.own_cache:
            specs["k_proj"] = TensorSpec((self.kv_heads * D, self.hidden))
            specs["v_proj"] = TensorSpec((self.kv_heads * D, self.hidden))
        if self.qk_norm:
            specs["q_norm"] = TensorSpec((D,), "gain")
            if self.own_cache:
                specs["k_norm"] = TensorSpec((D,), "gain")
        return specs

    def cache_need(self):
        return KVNeed(self.kv_heads, self.head_dim, self.window)

    def set_position(self, position) -> None:
        self.position = position

    def bind(self, tensors, runtime):
        self.ops = runtime.ops
        if self.own_cache:
            self.w_qkv = torch.cat([tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]], dim=0).contiguous()
        else:
            self.w_qkv = tensors["q_proj"].contiguous()
        self.w_o = tensors["o_proj"].contiguous()
        self.q_gain = tensors.get("q_norm")
        self.k_gain = tensors.get("k_norm")

    # -- compute ----------------------------------------------------------
    def forward(self, ctx, h, cache):
        ops = ctx.ops
        kv_in_row = self.kv_heads if self.own_cache else 0
        qkv = ops.linear(h, self.w_qkv)
        tables = self.position.rotary_tables() if self.position is not None else None
        cos, sin = tables if tables is not None else (None, None)
        attn = ops.rope_attention(qkv, self.heads, kv_in_row, self.head_dim, self.q_gain, self.k_gain, self.eps,
                                  cos, sin, ctx.batch, cache, self.scale, self.window)
        return ops.linear(attn, self.w_o)


register_mixer("gqa_attention", GQAttention)
