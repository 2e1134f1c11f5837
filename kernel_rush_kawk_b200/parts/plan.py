"""The description of a model as data.

An architecture module turns its configuration into a ``ModelPlan``. The plan
names, layer by layer, which mixer, feed-forward, norm and block arrangement a
layer uses, with every size and constant as a parameter and every checkpoint
tensor by its full name; and it gives the order in which layers run as a list
of ``ScheduleEntry``. A schedule may name a layer twice (the weights are shared,
each run has its own cache) or let a run read the cache that an earlier run
wrote (``cache_from``), in which case it writes none of its own.

Nothing in this file knows an architecture. The weight loader, the cache and
the step function are all built from a plan.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Mapping


def _frozen(d: Mapping | None) -> Mapping:
    return MappingProxyType(dict(d or {}))


@dataclass(frozen=True)
class PartSpec:
    """One part: the registered kind, its parameters, and the checkpoint name of
    each tensor it owns (local key -> full tensor name)."""

    kind: str
    params: Mapping = field(default_factory=dict)
    tensors: Mapping = field(default_factory=dict)

    def __post_init__(self):
        object.__setattr__(self, "params", _frozen(self.params))
        object.__setattr__(self, "tensors", _frozen(self.tensors))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer and a feed-forward, each behind
    its own norm."""

    block: str  # registered arrangement, e.g. "prenorm"
    mixer_norm: PartSpec
    mixer: PartSpec
    feed_forward_norm: PartSpec
    feed_forward: PartSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. ``cache_from`` is the index of an earlier schedule entry
    whose cache this run reads instead of keeping one."""

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    position: PartSpec | None
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    stop_token_ids: tuple[int, ...] = ()
    #: checkpoint names that may be present although no part asks for them, if they
    #: equal the named other tensor (a tied head stored twice): name -> same-as name
    duplicates: Mapping = field(default_factory=dict)

    def __post_init__(self):
        object.__setattr__(self, "layers", tuple(self.layers))
        object.__setattr__(self, "schedule", tuple(self.schedule))
        object.__setattr__(self, "duplicates", _frozen(self.duplicates))
        n = len(self.layers)
        for i, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < n:
                raise ValueError(f"schedule entry {i} names layer {entry.layer}, the plan has {n}")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {entry.cache_from}, which does not run before it")
                if self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {entry.cache_from}, which keeps none itself")
