"""Plain, slow Qwen3 dense decoder used as the oracle of the test-suite.

This implementation rests on the formulas of willzeng274/kernel-rush-kawk (each
function cites the file and lines it restates); that project's forward passes
need a GPU and Triton, so only its loader, RoPE tables and attention oracle can
be run on a CPU (see ``tests/golden/make_golden.py`` for what was compared).

Whole sequences, no cache, one function per part, torch on the CPU, no code
shared with the product package. ``dtype`` is the dtype the arithmetic runs in
(float64 gives a truth for the 32-bit engine path; float32 is the default).
``rounding`` is ``None`` (every rounding is the identity: the 32-bit path) or
``torch.bfloat16``: then every place where the reference's BF16 path rounds a
value to bfloat16 rounds here too, while reductions stay wide.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path

import torch


# ----------------------------------------------------------------------------
# configuration and weights (engine/model.py:25-52, :96-130)
# ----------------------------------------------------------------------------

@dataclass
class PlainConfig:
    hidden: int
    intermediate: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    vocab: int
    eps: float
    rope_theta: float
    tie: bool

    @classmethod
    def from_dict(cls, raw: dict) -> "PlainConfig":
        """Key names and defaults of engine/model.py:39-52."""
        return cls(
            hidden=raw["hidden_size"],
            intermediate=raw["intermediate_size"],
            layers=raw["num_hidden_layers"],
            heads=raw["num_attention_heads"],
            kv_heads=raw["num_key_value_heads"],
            head_dim=raw.get("head_dim") or raw["hidden_size"] // raw["num_attention_heads"],
            vocab=raw["vocab_size"],
            eps=raw["rms_norm_eps"],
            rope_theta=raw["rope_theta"],
            tie=raw.get("tie_word_embeddings", False),
        )

    @classmethod
    def from_folder(cls, folder) -> "PlainConfig":
        return cls.from_dict(json.loads((Path(folder) / "config.json").read_text()))


def read_folder(folder) -> tuple[PlainConfig, dict[str, torch.Tensor]]:
    """Every tensor of every shard, by name (engine/model.py:67-75), as float32."""
    from safetensors import safe_open

    cfg = PlainConfig.from_folder(folder)
    tensors: dict[str, torch.Tensor] = {}
    for shard in sorted(Path(folder).glob("*.safetensors")):
        with safe_open(str(shard), framework="pt", device="cpu") as f:
            for name in f.keys():
                tensors[name] = f.get_tensor(name).float()
    return cfg, tensors


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------

def _rounder(rounding):
    if rounding is None:
        return lambda t: t
    return lambda t: t.to(rounding).to(t.dtype)


def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """x0[r] = embed[ids[r]] (engine/model.py:291, :315)."""
    return table[ids]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, rounding=None) -> torch.Tensor:
    """v = mean(x^2); n = round(x * rsqrt(v + eps)); y = round(n * w): the value is
    rounded before the weight multiply (engine/kernels/rmsnorm.py:30-45)."""
    rt = _rounder(rounding)
    v = (x * x).mean(dim=-1, keepdim=True)
    n = rt(x * torch.rsqrt(v + eps))
    return rt(n * w)


def residual_add(x: torch.Tensor, branch: torch.Tensor, rounding=None) -> torch.Tensor:
    """s = round(x + branch), the new residual stream (engine/kernels/add_rmsnorm.py:21-23)."""
    return _rounder(rounding)(x + branch)


def linear(x: torch.Tensor, w: torch.Tensor, rounding=None) -> torch.Tensor:
    """y = x W^T, weights [out, in], no bias, wide accumulate, rounded output
    (engine/model.py:295,299,301; engine/kernels/gemm.py:79-91)."""
    return _rounder(rounding)(x @ w.t())


def rope_tables(head_dim: int, theta: float, n_pos: int, dtype=torch.float32, rounding=None):
    """inv_freq_i = 1/theta^(2i/D); angle[p,i] = p*inv_freq_i computed in 32-bit;
    cos/sin rounded after the trigonometric function (engine/model.py:78-93).
    Returns the half tables [n_pos, D/2]; column i also serves column i + D/2."""
    rt = _rounder(rounding)
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    pos = torch.arange(n_pos, dtype=torch.float32)
    angle = pos[:, None] * inv_freq[None, :]  # float32 product, as the reference's fp32 matmul of rank 1
    return rt(angle.cos().to(dtype)), rt(angle.sin().to(dtype))


def head_norm_rope(x: torch.Tensor, w: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, eps: float,
                   rounding=None) -> torch.Tensor:
    """Per-head RMSNorm over D followed by rotate-half RoPE with the reference's
    rounding points (engine/kernels/rope.py:19-30).

    x [T, heads, D]; w [D]; cos, sin [T, D/2] (rows already picked by position)."""
    rt = _rounder(rounding)
    half = x.shape[-1] // 2
    r = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    y = rt(w * rt(x * r))
    y1, y2 = y[..., :half], y[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    o1 = rt(rt(y1 * c) + rt(-y2 * s))
    o2 = rt(rt(y2 * c) + rt(y1 * s))
    return torch.cat([o1, o2], dim=-1)


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None,
                         rounding=None) -> torch.Tensor:
    """s = (q.k) * 1/sqrt(D); query at position p sees keys 0..p (p-window+1..p with a
    window); softmax with wide max and sum; probabilities rounded before P.V; the
    sum divides once at the end; q head h reads kv head h // G
    (engine/kernels/attention.py:9-11, :70-73, :104-122; engine/model.py:130, :276).

    q [T, HQ, D]; k, v [T, HKV, D]; returns [T, HQ*D]."""
    rt = _rounder(rounding)
    T, HQ, D = q.shape
    HKV = k.shape[1]
    G = HQ // HKV
    scale = 1.0 / math.sqrt(D)
    idx = torch.arange(T)
    visible = idx[None, :] <= idx[:, None]
    if window is not None:
        visible &= idx[None, :] > idx[:, None] - window
    out = torch.empty((T, HQ, D), dtype=q.dtype)
    for h in range(HQ):
        kh = h // G
        s = (q[:, h] @ k[:, kh].t()) * scale
        s = s.masked_fill(~visible, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        p = torch.exp(s - m)
        l = p.sum(dim=-1, keepdim=True)
        out[:, h] = rt((rt(p) @ v[:, kh]) / l)
    return out.reshape(T, HQ * D)


def swiglu_mlp(h: torch.Tensor, w_gate, w_up, w_down, rounding=None) -> torch.Tensor:
    """g = round(h Wg^T); u = round(h Wu^T); a = round(round(silu(g)) * u) with
    silu(g) = g / (1 + exp(-g)); d = round(a Wd^T)
    (engine/kernels/swiglu.py:21-24; engine/kernels/gemm.py:108-113; engine/model.py:301)."""
    rt = _rounder(rounding)
    g = linear(h, w_gate, rounding)
    u = linear(h, w_up, rounding)
    a = rt(rt(g / (1.0 + torch.exp(-g))) * u)
    return linear(a, w_down, rounding)


def attention_block(x, w: dict, prefix: str, cfg: PlainConfig, cos, sin, window=None, rounding=None):
    """QKV projection, per-head q/k norm, RoPE, attention, output projection
    (engine/model.py:295-299; engine/kernels/rope.py:139-144: v stays raw)."""
    T = x.shape[0]
    q = linear(x, w[prefix + "self_attn.q_proj.weight"], rounding).view(T, cfg.heads, cfg.head_dim)
    k = linear(x, w[prefix + "self_attn.k_proj.weight"], rounding).view(T, cfg.kv_heads, cfg.head_dim)
    v = linear(x, w[prefix + "self_attn.v_proj.weight"], rounding).view(T, cfg.kv_heads, cfg.head_dim)
    q = head_norm_rope(q, w[prefix + "self_attn.q_norm.weight"], cos, sin, cfg.eps, rounding)
    k = head_norm_rope(k, w[prefix + "self_attn.k_norm.weight"], cos, sin, cfg.eps, rounding)
    a = causal_gqa_attention(q, k, v, window, rounding)
    return linear(a, w[prefix + "self_attn.o_proj.weight"], rounding)


def decoder_layer(x, w: dict, i: int, cfg: PlainConfig, cos, sin, window=None, rounding=None):
    """x += Attn(norm_in(x)); x += MLP(norm_post(x)) (engine/model.py:294-302)."""
    p = f"model.layers.{i}."
    h = rms_norm(x, w[p + "input_layernorm.weight"], cfg.eps, rounding)
    x = residual_add(x, attention_block(h, w, p, cfg, cos, sin, window, rounding), rounding)
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg.eps, rounding)
    d = swiglu_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"], rounding)
    return residual_add(x, d, rounding)


def forward_logits(cfg: PlainConfig, w: dict, ids, dtype=torch.float32, rounding=None, windows=None) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence (engine/model.py:284-303;
    the head is the embedding when tied, :103-107). Logits are not rounded.

    ``windows``: optional list with one entry per layer (None or a window length)."""
    ids = torch.as_tensor(ids, dtype=torch.int64)
    w = {k: t.to(dtype) for k, t in w.items()}
    cos, sin = rope_tables(cfg.head_dim, cfg.rope_theta, len(ids), dtype, rounding)
    x = embedding(w["model.embed_tokens.weight"], ids)
    for i in range(cfg.layers):
        x = decoder_layer(x, w, i, cfg, cos, sin, None if windows is None else windows[i], rounding)
    h = rms_norm(x, w["model.norm.weight"], cfg.eps, rounding)
    head = w["model.embed_tokens.weight"] if cfg.tie else w["lm_head.weight"]
    return h @ head.t()


# ----------------------------------------------------------------------------
# token selection
# ----------------------------------------------------------------------------

def greedy(logits: torch.Tensor) -> int:
    """argmax, lowest index on ties (engine/engine.py:193,196)."""
    return int(torch.argmax(logits.float(), dim=-1))


def _mix32(x: torch.Tensor) -> torch.Tensor:
    """A 32-bit integer mixing function (xor-shift, multiply) on int64 tensors."""
    m = 0xFFFFFFFF
    x = x & m
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & m
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & m
    x = x ^ (x >> 16)
    return x


def gumbel_uniforms(seed: int, request: int, step: int, vocab: int) -> torch.Tensor:
    """The counter-based uniforms in (0, 1) that temperature sampling draws: one per
    vocabulary entry from a 32-bit mixing hash keyed by (seed, request, step, index);
    the top 23 bits of the hash, plus a half, over 2^23. The reference selects greedily
    only; this restates the product's documented definition so that its sampler can be
    checked draw by draw."""
    t = lambda v: torch.tensor(v & 0xFFFFFFFF, dtype=torch.int64)
    key = _mix32(_mix32(_mix32(t(seed)) ^ t(request)) ^ t(step))
    i = torch.arange(vocab, dtype=torch.int64)
    h = _mix32(key ^ ((i * 0x9E3779B9) & 0xFFFFFFFF))
    return ((h >> 9).double() + 0.5) / 8388608.0


def sample_temperature(logits: torch.Tensor, temperature: float, seed: int, request: int, step: int) -> int:
    """Gumbel-max: argmax_i(logits_i / temperature - log(-log(u_i))), a draw from
    softmax(logits / temperature)."""
    u = gumbel_uniforms(seed, request, step, logits.numel())
    g = -torch.log(-torch.log(u))
    return int(torch.argmax(logits.double() / temperature + g))


def generate_greedy(cfg: PlainConfig, w: dict, prompt: list[int], n_new: int, dtype=torch.float32, rounding=None) -> list[int]:
    """Greedy continuation by recomputing the whole sequence for every token."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        tok = greedy(forward_logits(cfg, w, seq, dtype, rounding)[-1])
        out.append(tok)
        seq.append(tok)
    return out
