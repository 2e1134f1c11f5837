"""Shared by the tests: the tiny configurations, tolerances, comparison helpers.

Two tiny Qwen3 configurations that differ in every size and option:

            layers hidden heads kv  head_dim  inter vocab  theta  eps    head    window
  tiny_a      2     64     4    2     16      192   256   1e4    1e-6   tied    none
  tiny_b      3     96     6    2     32      256   384   1e6    1e-5   untied  none
  tiny_w      3     80     5    1     48      144   301   5e5    1e-5   untied  24 keys on layers 1, 2
  tiny_v      2     96     4    2     64      160   333   1e4    1e-6   tied    70 keys on both layers

tiny_a and tiny_b are the presets of the package; tiny_w adds sizes that are no
power of two (hidden 80, 5 heads in one group, head size 48, vocabulary 301)
and layers that see a window of keys only. tiny_v (not in ``TINY``: only the tests of long
windowed sequences use it) has the head size 64 of the tensor-core kernels and a window on every
layer, so that with a small ``step_tokens`` its ring of pages is shorter than its sequences.

Tolerances, fixed before any measurement:
* 32-bit path against the plain implementation run in float64:
  |d| <= FP32_TOL * max|ref|.
* bfloat16, one kernel against its plain reference with the same rounding points:
  |d| <= 0.02 * max|ref| + 1e-3, the form the reference uses for its own kernels
  (engine/kernels/gemm.py:442-447 of willzeng274/kernel-rush-kawk).
* bfloat16, whole-model logits against the plain implementation with bfloat16
  rounding points: |d| <= 0.05 * max|ref| + 1e-3. Two correct bfloat16
  implementations differ by one-ulp flips that later layers amplify; with the test
  weights below that noise measures 0.1 to 1 % of max|ref| between two orders of
  accumulation of the plain implementation itself (float32 against float64
  sums), while a wrong key or position moves the logits by 15 % and more. (The
  reference's own whole-model check allows 2.0 logits on logits of some tens:
  engine/engine.py:53-58,556.)
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

import plain_qwen3 as plain

FP32_TOL = 1e-4

TINY_W = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 80, "intermediate_size": 144,
    "num_hidden_layers": 3, "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 48, "vocab_size": 301,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "tie_word_embeddings": False, "max_position_embeddings": 2048,
    "sliding_window": 24, "layer_types": ["full_attention", "sliding_attention", "sliding_attention"],
}
TINY_V = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 96, "intermediate_size": 160,
    "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 333,
    "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": True, "max_position_embeddings": 2048,
    "sliding_window": 70, "layer_types": ["sliding_attention", "sliding_attention"],
}
TINY = ("tiny_a", "tiny_b", "tiny_w")
EXTRA = ("tiny_v",)
SEEDS = {"tiny_a": 11, "tiny_b": 22, "tiny_w": 33, "tiny_v": 44}
_DICTS = {"tiny_w": TINY_W, "tiny_v": TINY_V}


def tiny_config(name: str):
    from kernel_rush_kawk_b200 import Qwen3Config

    return Qwen3Config.from_dict(_DICTS[name]) if name in _DICTS else Qwen3Config.preset(name)


def write_tiny(folder, name: str) -> Path:
    """A model folder with random weights whose q/k gains are scaled up, so that
    attention is sharp and a wrong key or position moves the logits visibly; the
    weights' std is 0.04 so that tiny widths still give logits of order 1."""
    from kernel_rush_kawk_b200 import write_model_folder

    cfg = tiny_config(name)
    scale = {}
    for i in range(cfg.num_hidden_layers):
        scale[f"model.layers.{i}.self_attn.q_norm.weight"] = 1.5
        scale[f"model.layers.{i}.self_attn.k_norm.weight"] = 1.5
    return write_model_folder(folder, cfg, SEEDS[name], std=0.04, gain_std=0.1, scale=scale)


def windows_of(name: str):
    cfg = tiny_config(name)
    return [cfg.window_of(i) for i in range(cfg.num_hidden_layers)]


def prompts_for(name: str, lengths, seed=0):
    cfg = tiny_config(name)
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lengths]


_plain_cache: dict = {}


def plain_logits(folder, name: str, ids, dtype: str) -> torch.Tensor:
    """Logits [T, V] of the plain implementation for the path named ``dtype``:
    "float32" -> float64 arithmetic without rounding; "bfloat16" -> float32
    arithmetic with the reference's bfloat16 rounding points."""
    key = (str(folder), tuple(ids), dtype)
    if key not in _plain_cache:
        cfg, w = plain.read_folder(folder)
        if dtype == "float32":
            out = plain.forward_logits(cfg, w, ids, torch.float64, None, windows_of(name))
        else:
            out = plain.forward_logits(cfg, w, ids, torch.float32, torch.bfloat16, windows_of(name))
        _plain_cache[key] = out.float()
    return _plain_cache[key]


def tolerance(scale: float, dtype: str, kernel: bool = False) -> float:
    if dtype == "float32":
        return FP32_TOL * scale
    return (0.02 if kernel else 0.05) * scale + 1e-3


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "", kernel: bool = False) -> None:
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    scale = ref.abs().max().item()
    tol = tolerance(scale, dtype, kernel)
    err = (got - ref).abs().max().item()
    if err > tol:
        idx = (got - ref).abs().argmax().item()
        r, c = divmod(idx, got.shape[-1]) if got.dim() > 1 else (0, idx)
        raise AssertionError(f"{what}: max |d| = {err:.3e} > {tol:.3e} (max|ref| = {scale:.3e}) first at row {r}, column {c}")


def first_wrong_row(got: torch.Tensor, ref: torch.Tensor, dtype: str):
    scale = ref.abs().max().item()
    tol = tolerance(scale, dtype)
    bad = ((got.float().cpu() - ref.float().cpu()).abs() > tol).any(dim=-1).nonzero()
    return None if bad.numel() == 0 else int(bad[0])


def greedy_gap_allowed(cfg, w, seq, dtype: str, windows=None):
    """(reference logits at the last position of ``seq``, the gap below their maximum that a greedy
    token may have). In 32-bit the reference is the plain implementation in float64 and the gap is the
    32-bit tolerance. In bfloat16 the gap is the noise of bfloat16 arithmetic measured at this very
    position: twice the spread between the plain implementation's logits with float32 and with float64
    accumulation (same rounding points, two orders of summation), plus one bfloat16 step (2^-7) of
    the largest logit for the one-ulp flips that two correct implementations may differ by."""
    if dtype == "float32":
        ref = plain.forward_logits(cfg, w, seq, torch.float64, None, windows)[-1].float()
        return ref, 2 * FP32_TOL * ref.abs().max().item()
    a = plain.forward_logits(cfg, w, seq, torch.float32, torch.bfloat16, windows)[-1]
    b = plain.forward_logits(cfg, w, seq, torch.float64, torch.bfloat16, windows)[-1].float()
    return a, 2 * (a - b).abs().max().item() + a.abs().max().item() / 128


def assert_greedy_token(cfg, w, seq, tok: int, dtype: str, windows=None, what: str = "") -> None:
    """``tok`` continues ``seq`` greedily: it is the plain argmax, or lies below it by no more than
    ``greedy_gap_allowed``."""
    ref, allowed = greedy_gap_allowed(cfg, w, seq, dtype, windows)
    gap = ref.max().item() - ref[tok].item()
    assert gap <= allowed, f"{what}: token {tok} lies {gap:.4g} below the plain argmax {int(ref.argmax())} (allowed {allowed:.4g})"
