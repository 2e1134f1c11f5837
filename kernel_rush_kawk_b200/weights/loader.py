"""Weights from safetensors, by tensor name.

Every tensor of every ``*.safetensors`` shard in the folder is looked at by name,
shards in sorted order, as the reference does (engine/model.py:67-75 of
willzeng274/kernel-rush-kawk; it reads no index file either). The reference
fails on the first missing name with a KeyError and on leftovers with another
(:105-106, :127-128) and checks no shapes; here all three kinds of fault are
collected and raised as one ``WeightError``.

Dtype policy. The compute dtype of the path is bfloat16 or float32.
* float32 path: every floating tensor is widened to float32 (exact).
* bfloat16 path: 16-bit floating tensors are kept as bfloat16. A tensor stored
  in 32-bit stays 32-bit if it is a vector (a norm's gain: the kernels take
  either); a matrix or table stored in 32-bit is rounded to bfloat16, because
  the matrix kernels of this path read bfloat16 only, and a warning says so.
* integer tensors become int32.
"""

from __future__ import annotations

import logging
from pathlib import Path

import torch

log = logging.getLogger(__name__)


class WeightError(RuntimeError):
    """The checkpoint does not fit the model. ``missing``, ``unexpected`` and
    ``wrong_shape`` (name -> (expected, found)) hold the details."""

    def __init__(self, folder, missing, unexpected, wrong_shape, other=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = dict(sorted(wrong_shape.items()))
        self.other = list(other)
        lines = [f"checkpoint at {folder} does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n}: expected {list(e)}, found {list(f)}" for n, (e, f) in self.wrong_shape.items()))
        lines.extend("  " + o for o in self.other)
        super().__init__("\n".join(lines))


def stored_dtype(role: str, ndim: int, file_dtype: torch.dtype, compute: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in (see the module text)."""
    if not file_dtype.is_floating_point:
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if file_dtype == torch.float32 and ndim == 1:
        return torch.float32
    return compute


def read_checkpoint(folder, expected: dict, device, compute: torch.dtype, duplicates=None) -> dict[str, torch.Tensor]:
    """expected: full tensor name -> TensorSpec. Returns name -> tensor on ``device``."""
    from safetensors import safe_open

    folder = Path(folder)
    shards = sorted(folder.glob("*.safetensors"))
    if not shards:
        raise FileNotFoundError(f"no *.safetensors under {folder}")
    duplicates = dict(duplicates or {})
    found: dict[str, torch.Tensor] = {}
    spare: dict[str, torch.Tensor] = {}
    unexpected, wrong_shape, other = [], {}, []
    for shard in shards:
        try:
            handle = safe_open(str(shard), framework="pt", device="cpu")
        except Exception as exc:  # a truncated or corrupt shard
            raise WeightError(folder, [], [], {}, [f"{shard.name} cannot be read: {exc}"]) from exc
        with handle as f:
            for name in f.keys():
                if name in found:
                    other.append(f"{name} is stored in more than one shard")
                    continue
                if name in expected:
                    shape = tuple(f.get_slice(name).get_shape())
                    want = tuple(expected[name].shape)
                    if shape != want:
                        wrong_shape[name] = (want, shape)
                        continue
                    t = f.get_tensor(name)
                    keep = stored_dtype(expected[name].role, t.dim(), t.dtype, compute)
                    if t.dtype == torch.float32 and keep != torch.float32:
                        log.warning("%s is stored in float32 and is rounded to %s for this path", name, keep)
                    found[name] = t.to(device=device, dtype=keep).contiguous()
                elif name in duplicates:
                    spare[name] = f.get_tensor(name)
                else:
                    unexpected.append(name)
    for name, tensor in spare.items():
        same_as = duplicates[name]
        if same_as in found and tensor.shape == found[same_as].shape and torch.equal(
                tensor.to(found[same_as].dtype), found[same_as].cpu()):
            continue
        other.append(f"{name} is present although the model ties it to {same_as}, and differs from it")
    missing = [n for n in expected if n not in found and n not in wrong_shape]
    if missing or unexpected or wrong_shape or other:
        raise WeightError(folder, missing, unexpected, wrong_shape, other)
    return found
