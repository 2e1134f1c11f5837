"""Seeded random weights, and a model folder written from them.

The reference has no random-weights mode. Every tensor is a function of (seed,
tensor name, element index) alone, so a value depends neither on the order or
the number of tensors nor on the device that computes it: the same numbers come
out of a CPU and out of a CUDA device, bit for bit. Matrices and tables are
normal(0, std), a norm's gain is 1 + normal(0, std); computed in float64, rounded
to float32 and then to bfloat16 (the values that a written folder stores, so the
32-bit path and the bfloat16 path start from the same numbers).

The generator is counter-based. Element pair j of a tensor hashes the counters 2j
and 2j + 1 with a 64-bit mixing function keyed by SHA-256(seed, name); the top 32
bits of each hash give u1, u2 in (0, 1), and the Box-Muller transform
sqrt(-2 ln u1) * (cos, sin)(2 pi u2) gives the pair's two normals. Logarithm, sine,
cosine and the square root are evaluated here from their series (Heron's iteration
for the root) with additions, multiplications and divisions only, which IEEE 754
rounds the same way everywhere; a library's log, cos or sqrt differs in the last
place between devices.
"""

from __future__ import annotations

import hashlib
import json
import math
from pathlib import Path

import torch

_MASK64 = (1 << 64) - 1
_LN2 = math.log(2.0)


def _signed(v: int) -> int:
    v &= _MASK64
    return v - (1 << 64) if v >> 63 else v


def _key_of(name: str, seed: int) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little")


def _hash32(counter: torch.Tensor, key: int) -> torch.Tensor:
    """Top 32 bits of a 64-bit mix of (counter, key), as int64 in [0, 2^32). int64 products wrap."""
    z = counter * _signed(0x9E3779B97F4A7C15) + _signed(key)
    z = z ^ ((z >> 30) & ((1 << 34) - 1))
    z = z * _signed(0xBF58476D1CE4E5B9)
    z = z ^ ((z >> 27) & ((1 << 37) - 1))
    z = z * _signed(0x94D049BB133111EB)
    z = z ^ ((z >> 31) & ((1 << 33) - 1))
    return (z >> 32) & 0xFFFFFFFF


def _horner(t: torch.Tensor, coefficients) -> torch.Tensor:
    acc = torch.full_like(t, coefficients[0])
    for c in coefficients[1:]:
        acc = acc * t
        acc = acc + c
    return acc


_LOG_SERIES = [1.0 / n for n in range(21, 0, -2)]                          # atanh series: 1/21 ... 1/3, 1
_COS_SERIES = [(-1.0) ** k / math.factorial(2 * k) for k in range(11, -1, -1)]
_SIN_SERIES = [(-1.0) ** k / math.factorial(2 * k + 1) for k in range(11, -1, -1)]


def _neg_two_log(a: torch.Tensor) -> torch.Tensor:
    """-2 ln((a + 1/2) / 2^32) for integers a in [0, 2^32), float64, from the series
    ln m = 2 atanh((m - 1) / (m + 1)) on the mantissa m in [sqrt(1/2), sqrt(2))."""
    m, e = torch.frexp(a.double() + 0.5)
    low = m < math.sqrt(0.5)
    m = torch.where(low, m * 2.0, m)
    e = torch.where(low, e - 1, e).double() - 32.0
    s = (m - 1.0) / (m + 1.0)
    ln_m = (s * 2.0) * _horner(s * s, _LOG_SERIES)
    return (ln_m + e * _LN2) * -2.0


def _sqrt(y: torch.Tensor) -> torch.Tensor:
    """Square root of positive float64 numbers by Heron's iteration from a fixed first guess: additions,
    multiplications and divisions only (a library's square root was seen to differ in the last place
    between a CPU and a GPU)."""
    m, e = torch.frexp(y)
    odd = (e & 1) == 1
    m = torch.where(odd, m * 2.0, m)         # m in [1/2, 2), e even
    e = torch.where(odd, e - 1, e)
    g = m * 0.5 + 0.5                        # within 7 % of sqrt(m); each step squares the relative error
    for _ in range(6):
        g = (g + m / g) * 0.5
    # times 2^(e/2), the power taken from a table of exact values (a pow() need not be exact)
    half = torch.div(e, 2, rounding_mode="floor").long()
    powers = torch.tensor([2.0 ** k for k in range(-600, 601)], dtype=torch.float64, device=y.device)
    return g * powers[(half + 600).clamp(0, 1200)]


def _cos_sin_turn(b: torch.Tensor):
    """cos and sin of 2 pi (b + 1/2) / 2^32 for integers b in [0, 2^32): the top two bits
    pick the quadrant, the rest an angle in (0, pi/2) whose series are summed."""
    quadrant = b >> 30
    theta = ((b & ((1 << 30) - 1)).double() + 0.5) * (math.pi / 2.0 / (1 << 30))
    t = theta * theta
    c = _horner(t, _COS_SERIES)
    s = _horner(t, _SIN_SERIES) * theta
    odd = (quadrant & 1) == 1
    cos = torch.where(odd, s, c)
    sin = torch.where(odd, c, s)
    cos = torch.where((quadrant == 1) | (quadrant == 2), -cos, cos)
    sin = torch.where(quadrant >= 2, -sin, sin)
    return cos, sin


def standard_normals(n: int, key: int, device="cpu") -> torch.Tensor:
    """n draws from normal(0, 1), float64, element i a function of (key, i) only."""
    device = torch.device(device)
    out = torch.empty(n + (n & 1), dtype=torch.float64, device=device)
    pairs = out.numel() // 2
    chunk = (1 << 24) if device.type == "cuda" else (1 << 16)  # pairs per pass: a CPU pass stays in cache
    view = out.view(pairs, 2)
    for first in range(0, pairs, chunk):
        j = torch.arange(first, min(first + chunk, pairs), dtype=torch.int64, device=device) * 2
        radius = _sqrt(_neg_two_log(_hash32(j, key)))
        cos, sin = _cos_sin_turn(_hash32(j + 1, key))
        view[first:first + j.numel(), 0] = radius * cos
        view[first:first + j.numel(), 1] = radius * sin
    return out[:n]


def random_tensor(name: str, spec, seed: int, std: float, device="cpu", gain_std: float | None = None) -> torch.Tensor:
    shape = tuple(spec.shape)
    n = math.prod(shape)
    z = standard_normals(n, _key_of(name, seed), device)
    if spec.role == "gain":
        z = z * (std if gain_std is None else gain_std) + 1.0
    else:
        z = z * std
    return z.float().to(torch.bfloat16).view(shape)


def random_tensors(expected: dict, seed: int, std: float = 0.02, device="cpu", gain_std: float | None = None) -> dict:
    """expected: full tensor name -> TensorSpec; returns name -> bfloat16 tensor."""
    return {name: random_tensor(name, spec, seed, std, device, gain_std) for name, spec in expected.items()}


def write_model_folder(folder, config, seed: int, std: float = 0.02, gain_std: float | None = None, scale: dict | None = None,
                       device="cpu") -> Path:
    """Write ``config.json`` and ``model.safetensors`` for a configuration and a seed.

    ``scale`` optionally multiplies named tensors (name -> factor) after drawing, for
    tests that want, say, sharper attention than plain random weights give. ``device``
    is where the numbers are computed; the file is the same wherever that is."""
    from safetensors.torch import save_file
    from ..engine.model import expected_tensors
    from ..config.registry import get_architecture

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    arch = get_architecture(config.architecture)
    plan = arch.plan(config)
    tensors = random_tensors(expected_tensors(plan), seed, std, device, gain_std)
    for name, factor in (scale or {}).items():
        tensors[name] = (tensors[name].float() * factor).to(torch.bfloat16)
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")
    save_file({k: v.cpu().contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
