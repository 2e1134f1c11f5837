"""Seeded random weights, and a model folder written from them.

The reference has no random-weights mode. Every tensor draws from a generator
of its own, seeded from the run's seed and the tensor's name, so a value does
not depend on the order or the number of tensors: matrices and tables are
normal(0, std), a norm's gain is 1 + normal(0, std); drawn in float32, then
rounded to bfloat16 (the values that a written folder stores, so the 32-bit
path and the bfloat16 path start from the same numbers). Values depend on the
device type the generator runs on (CPU and CUDA generators differ).
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch


def _seed_of(name: str, seed: int) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, spec, seed: int, std: float, device="cpu", gain_std: float | None = None) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_seed_of(name, seed))
    t = torch.empty(tuple(spec.shape), dtype=torch.float32, device=device)
    if spec.role == "gain":
        t.normal_(0.0, std if gain_std is None else gain_std, generator=gen)
        t += 1.0
    else:
        t.normal_(0.0, std, generator=gen)
    return t.to(torch.bfloat16)


def random_tensors(expected: dict, seed: int, std: float = 0.02, device="cpu", gain_std: float | None = None) -> dict:
    """expected: full tensor name -> TensorSpec; returns name -> bfloat16 tensor."""
    return {name: random_tensor(name, spec, seed, std, device, gain_std) for name, spec in expected.items()}


def write_model_folder(folder, config, seed: int, std: float = 0.02, gain_std: float | None = None, scale: dict | None = None) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for a configuration and a seed.

    ``scale`` optionally multiplies named tensors (name -> factor) after drawing, for
    tests that want, say, sharper attention than plain random weights give."""
    from safetensors.torch import save_file
    from ..engine.model import expected_tensors
    from ..config.registry import get_architecture

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    arch = get_architecture(config.architecture)
    plan = arch.plan(config)
    tensors = random_tensors(expected_tensors(plan), seed, std, "cpu", gain_std)
    for name, factor in (scale or {}).items():
        tensors[name] = (tensors[name].float() * factor).to(torch.bfloat16)
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
