"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a ``PartSpec``: ``cls(spec.params)``. It declares the
tensors it owns (``tensor_specs``), takes them (``bind``), and computes
(``forward``). It never learns which model it sits in: sizes and constants are
parameters, checkpoint names live in the plan, and the cache hands it a view of
the storage its own ``cache_need`` asked for.

Registries map a kind name to a class, so that a plan can choose a part layer
by layer and so that a new part can be added without touching this package:

    register_mixer("my_mixer", MyMixer)

The same holds for the two parts that stand outside the layers, the embedding of
the tokens and the output head (``register_embedding``, ``register_head``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping


# ----------------------------------------------------------------------------
# what a part declares
# ----------------------------------------------------------------------------

@dataclass(frozen=True)
class TensorSpec:
    """Shape and role of one tensor a part owns.

    ``role`` decides dtype policy and random initialisation: "matrix" (compute
    dtype, normal(0, std)), "gain" (a norm's weight: 1 + normal(0, std)), "table"
    (an embedding: normal(0, std))."""

    shape: tuple[int, ...]
    role: str = "matrix"


@dataclass(frozen=True)
class KVNeed:
    """Keys and values for every position (``window`` None) or for the last
    ``window`` positions. Runs whose needs are equal share one storage group."""

    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """Per-sequence state of fixed size, zeroed when a slot is handed out.
    ``dtype`` is "compute" (the path's dtype) or "float32"."""

    shape: tuple[int, ...]
    dtype: str = "float32"


class Part:
    """Base of every part."""

    #: False if forward() reads data of the step on the host (lengths, a routing decision), so that a
    #: single-token step with this part cannot be replayed from a captured graph
    graph_safe = True

    def __init__(self, params: Mapping[str, Any]):
        self.params = dict(params)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def bind(self, tensors: dict, runtime) -> None:
        """Take this part's tensors (keyed as in ``tensor_specs``). ``runtime`` gives
        ``device``, ``dtype`` (torch dtype of the path) and ``ops`` (the kernels)."""

    def to_checkpoint(self) -> None:
        """Nothing to do by default; parts that fuse tensors keep the originals' names
        only in the plan, never on disk."""


class Norm(Part):
    def forward(self, ctx, stream: "Stream"):
        """Fold ``stream.branch`` into ``stream.x`` and return the normalised rows
        [rows, hidden]. After the call ``stream.branch`` is None."""
        raise NotImplementedError


class Embedding(Part):
    def forward(self, ctx):
        """The step's rows [rows, hidden] from ``ctx.batch.tokens``."""
        raise NotImplementedError


class Head(Part):
    def forward(self, ctx, h):
        """h: the normalised rows of the wanted positions (a tensor, or a norm's lazy result)
        -> float32 logits [rows, vocab]."""
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self):
        """KVNeed, StateNeed or None."""
        return None

    def forward(self, ctx, h, cache):
        """h [rows, hidden] normalised input -> branch [rows, hidden]. ``cache`` is
        the view of this run's storage (None if ``cache_need`` is None)."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h):
        raise NotImplementedError


class PositionEncoding(Part):
    def bind(self, tensors: dict, runtime) -> None:
        raise NotImplementedError

    def rotary_tables(self):
        """(cos, sin) each [positions, rotary_dim/2] in the path's dtype, or None if
        this encoding does not rotate queries and keys."""
        return None

    def on_embeddings(self, ctx, x):
        """Hook for encodings that act on the embedded tokens; returns x."""
        return x


class Block:
    """Arrangement of a layer's parts around the residual stream."""

    def __init__(self, mixer_norm: Norm, mixer: Mixer, feed_forward_norm: Norm, feed_forward: FeedForward):
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.feed_forward_norm = feed_forward_norm
        self.feed_forward = feed_forward

    def forward(self, ctx, stream: "Stream", cache) -> "Stream":
        raise NotImplementedError


class Stream:
    """The residual stream between parts: ``x`` [rows, hidden] and a branch output
    that has not been added yet. The next norm adds it (one fused kernel does the
    add, writes the new ``x`` and normalises), which is how the reference fuses the
    residual add with the following RMSNorm (engine/model.py:300-302)."""

    __slots__ = ("x", "branch")

    def __init__(self, x, branch=None):
        self.x = x
        self.branch = branch


# ----------------------------------------------------------------------------
# registries
# ----------------------------------------------------------------------------

_MIXERS: dict[str, type] = {}
_FEED_FORWARDS: dict[str, type] = {}
_NORMS: dict[str, type] = {}
_POSITIONS: dict[str, type] = {}
_BLOCKS: dict[str, type] = {}
_EMBEDDINGS: dict[str, type] = {}
_HEADS: dict[str, type] = {}


def _register(table: dict, what: str):
    def register(kind: str, cls: type) -> type:
        table[kind] = cls
        return cls
    register.__doc__ = f"Register a {what} class under a kind name (replaces an earlier entry)."
    return register


def _lookup(table: dict, what: str):
    def lookup(kind: str) -> type:
        try:
            return table[kind]
        except KeyError:
            raise KeyError(f"unknown {what} kind '{kind}'; registered: {sorted(table)}") from None
    return lookup


register_mixer = _register(_MIXERS, "mixer")
register_feed_forward = _register(_FEED_FORWARDS, "feed-forward")
register_norm = _register(_NORMS, "norm")
register_position = _register(_POSITIONS, "position encoding")
register_block = _register(_BLOCKS, "block arrangement")
register_embedding = _register(_EMBEDDINGS, "embedding")
register_head = _register(_HEADS, "output head")

mixer_class = _lookup(_MIXERS, "mixer")
feed_forward_class = _lookup(_FEED_FORWARDS, "feed-forward")
norm_class = _lookup(_NORMS, "norm")
position_class = _lookup(_POSITIONS, "position encoding")
block_class = _lookup(_BLOCKS, "block arrangement")
embedding_class = _lookup(_EMBEDDINGS, "embedding")
head_class = _lookup(_HEADS, "output head")
