"""The kernels' interface restated in plain torch, for tests only.

Each method has the signature and meaning of the same method of the product's
CUDA bindings (``kernel_rush_kawk_b200/csrc/bindings.py``) and serves two ends:
the reference that each kernel is compared with on the GPU, and a stand-in
backend with which the engine's step, cache and generation logic can be run on
the CPU (the product itself has no CPU path and never imports this file).

Rounding follows the formulas of willzeng274/kernel-rush-kawk that
``tests/plain_qwen3.py`` cites: a value is rounded to the compute dtype wherever
the reference's BF16 path rounds; reductions are float32.
"""

from __future__ import annotations

import math

import torch

PAGE = 64


def _mix32(x: torch.Tensor) -> torch.Tensor:
    m = 0xFFFFFFFF
    x = x & m
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & m
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & m
    x = x ^ (x >> 16)
    return x


class TorchOps:
    def __init__(self, dtype=torch.float32):
        self.dtype = dtype

    def rt(self, t: torch.Tensor) -> torch.Tensor:
        """Round to the compute dtype, keep float32 for the next wide operation."""
        return t.to(self.dtype).float()

    # -- helpers -----------------------------------------------------------
    def empty_like(self, x):
        return torch.empty_like(x)

    def _resolve(self, x):
        return x.tensor() if hasattr(x, "tensor") and not isinstance(x, torch.Tensor) else x

    # -- elementwise and norms -----------------------------------------------
    def embed(self, table, tokens, n_rows):
        return table[tokens.long()].to(self.dtype)

    def rmsnorm(self, x, gain, eps):
        xf = x.float()
        n = self.rt(xf * torch.rsqrt((xf * xf).mean(dim=-1, keepdim=True) + eps))
        return (n * gain.float()).to(self.dtype)

    def add_rmsnorm(self, x, branch, gain, eps, x_new):
        s = (x.float() + branch.float()).to(self.dtype)
        x_new.copy_(s)
        return self.rmsnorm(s, gain, eps)

    def gather_rows(self, x, idx):
        return x[idx.long()]

    # -- matrix products -------------------------------------------------------
    def linear(self, x, w, out_float32=False):
        x = self._resolve(x)
        y = x.float() @ w.float().t()
        return y if out_float32 else y.to(self.dtype)

    def gate_up_swiglu(self, h, w_gate_up, intermediate):
        gu = self.linear(h, w_gate_up).float()
        g, u = gu[:, :intermediate], gu[:, intermediate:]
        return (self.rt(g / (1.0 + torch.exp(-g))) * u).to(self.dtype)

    # -- attention ----------------------------------------------------------
    def qk_norm_rope_write(self, qkv, heads, kv_in_row, head_dim, q_gain, k_gain, eps, cos, sin, batch, cache):
        D = head_dim
        half = cos.shape[1] if cos is not None else D // 2  # the rotated width is twice the tables' columns
        rows = qkv.shape[0]
        pos = batch.row_pos.long()
        view = qkv.view(rows, heads + 2 * kv_in_row, D)

        def norm_rope(x, gain):
            x = x.float()
            if gain is not None:
                r = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
                x = self.rt(gain.float() * self.rt(x * r))
            if cos is not None:
                c, s = cos[pos].float()[:, None, :], sin[pos].float()[:, None, :]
                x1, x2, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
                x = torch.cat([self.rt(self.rt(x1 * c) + self.rt(-x2 * s)),
                               self.rt(self.rt(x2 * c) + self.rt(x1 * s)), rest], dim=-1)
            return x.to(self.dtype)

        view[:, :heads] = norm_rope(view[:, :heads], q_gain)
        if kv_in_row:
            k = norm_rope(view[:, heads:heads + kv_in_row], k_gain)
            v = view[:, heads + kv_in_row:]
            slot = batch.seq_slot.long()[batch.row_seq.long()]
            page = cache.table.long()[slot, (pos // PAGE) % cache.width]
            off = pos % PAGE
            cache.k[page, :, off] = k
            cache.v[page, :, off] = v

    def rope_attention(self, qkv, heads, kv_in_row, head_dim, q_gain, k_gain, eps, cos, sin, batch, cache, scale,
                       window):
        self.qk_norm_rope_write(qkv, heads, kv_in_row, head_dim, q_gain, k_gain, eps, cos, sin, batch, cache)
        return self.attention(qkv, heads, kv_in_row, head_dim, batch, cache, scale, window)

    def attention(self, qkv, heads, kv_in_row, head_dim, batch, cache, scale, window):
        D = head_dim
        rows = qkv.shape[0]
        G = heads // cache.kv_heads
        q = qkv.view(rows, heads + 2 * kv_in_row, D)[:, :heads].float()
        out = torch.empty((rows, heads, D), dtype=torch.float32, device=qkv.device)
        table = cache.table.long()
        row0 = 0
        for slot, start, n in zip(batch.slots, batch.starts, batch.q_lens):
            total = start + n
            lo = 0 if window is None else max(0, start - window + 1)
            positions = torch.arange(lo, total, device=qkv.device)
            pages = table[slot, (positions // PAGE) % cache.width]
            k = cache.k[pages, :, positions % PAGE].float()  # [keys, kv_heads, D]
            v = cache.v[pages, :, positions % PAGE].float()
            qpos = torch.arange(start, total, device=qkv.device)
            visible = positions[None, :] <= qpos[:, None]
            if window is not None:
                visible &= positions[None, :] > qpos[:, None] - window
            for h in range(heads):
                s = (q[row0:row0 + n, h] @ k[:, h // G].t()) * scale
                s = s.masked_fill(~visible, float("-inf"))
                m = s.max(dim=-1, keepdim=True).values
                p = torch.exp(s - m)
                l = p.sum(dim=-1, keepdim=True)
                out[row0:row0 + n, h] = (self.rt(p) @ v[:, h // G]) / l
            row0 += n
        return out.to(self.dtype).view(rows, heads * D)

    # -- token selection ------------------------------------------------------
    def select_tokens(self, logits, temperature, seed, requests, step):
        logits = logits.float()
        if temperature == 0.0:
            return logits.argmax(dim=-1).to(torch.int32)
        n, vocab = logits.shape
        t = lambda v: torch.tensor(v & 0xFFFFFFFF, dtype=torch.int64)
        i = torch.arange(vocab, dtype=torch.int64)
        out = torch.empty(n, dtype=torch.int32)
        for r in range(n):
            key = _mix32(_mix32(_mix32(t(seed)) ^ t(int(requests[r]))) ^ t(step))
            h = _mix32(key ^ ((i * 0x9E3779B9) & 0xFFFFFFFF))
            u = ((h >> 9).float() + 0.5) / 8388608.0
            g = -torch.log(-torch.log(u))
            out[r] = int(torch.argmax(logits[r].cpu() / temperature + g))
        return out.to(logits.device)
