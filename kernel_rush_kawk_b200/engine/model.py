"""A model put together from a plan: parts built, weights bound, layers run.

This module knows no architecture. It builds the parts a ``ModelPlan`` names,
asks them which tensors they own, binds what the loader (or the random
initialiser) produced, tells the cache what each run of a layer needs, and runs
the schedule for one step's rows. The run order is the reference's
(engine/model.py:284-303 of willzeng274/kernel-rush-kawk: embed, layers, final
norm, head at the wanted rows) with its fusion of the residual add into the next
norm (:300-302).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts import base as parts_base
from ..parts.base import KVNeed, StateNeed, Stream, TensorSpec
from ..parts.plan import ModelPlan, PartSpec


@dataclass
class Runtime:
    device: torch.device
    dtype: torch.dtype
    ops: object


@dataclass
class _Built:
    spec: PartSpec
    part: object


def _build(spec: PartSpec, lookup, extra: dict | None = None) -> _Built:
    params = dict(spec.params)
    params.update(extra or {})
    return _Built(spec, lookup(spec.kind)(params))


class PartTree:
    """Every part of a plan, built but not yet bound to weights."""

    def __init__(self, plan: ModelPlan, max_context: int | None = None):
        import kernel_rush_kawk_b200.parts  # noqa: F401  (registers the built-in kinds)

        self.plan = plan
        positions = min(plan.max_positions, max_context) if max_context else plan.max_positions
        self.embedding = _build(plan.embedding, parts_base.embedding_class)
        self.head = _build(plan.head, parts_base.head_class)
        self.final_norm = _build(plan.final_norm, parts_base.norm_class)
        self.position = None
        if plan.position is not None:
            self.position = _build(plan.position, parts_base.position_class, {"positions": positions})
        self.layers = []
        for spec in plan.layers:
            mixer_norm = _build(spec.mixer_norm, parts_base.norm_class)
            mixer = _build(spec.mixer, parts_base.mixer_class)
            ffn_norm = _build(spec.feed_forward_norm, parts_base.norm_class)
            ffn = _build(spec.feed_forward, parts_base.feed_forward_class)
            if self.position is not None and hasattr(mixer.part, "set_position"):
                mixer.part.set_position(self.position.part)
            block = parts_base.block_class(spec.block)(mixer_norm.part, mixer.part, ffn_norm.part, ffn.part)
            self.layers.append((block, [mixer_norm, mixer, ffn_norm, ffn]))
        for i, entry in enumerate(plan.schedule):
            mixer = self.layers[entry.layer][0].mixer
            owns = getattr(mixer, "own_cache", True)
            if entry.cache_from is not None and owns and mixer.cache_need() is not None:
                raise ValueError(f"schedule entry {i} reads another run's cache but its mixer keeps one of its own "
                                 f"(build it with own_cache=False)")
            if entry.cache_from is None and not owns:
                raise ValueError(f"schedule entry {i}: its mixer keeps no cache, so the entry must name one to read")

    def all_parts(self) -> list[_Built]:
        out = [self.embedding, self.head, self.final_norm]
        if self.position is not None:
            out.append(self.position)
        for _, built in self.layers:
            out.extend(built)
        return out

    def expected_tensors(self) -> dict[str, TensorSpec]:
        """Full checkpoint name -> TensorSpec over all parts. Two parts may name the
        same tensor (a tied head) if they agree on its shape."""
        expected: dict[str, TensorSpec] = {}
        for built in self.all_parts():
            specs = built.part.tensor_specs()
            for key, tspec in specs.items():
                if key not in built.spec.tensors:
                    raise KeyError(f"the plan gives no checkpoint name for tensor '{key}' of a '{built.spec.kind}' part")
                name = built.spec.tensors[key]
                if name in expected and tuple(expected[name].shape) != tuple(tspec.shape):
                    raise ValueError(f"tensor {name} is used with shapes {expected[name].shape} and {tspec.shape}")
                expected.setdefault(name, tspec)
        return expected

    def cache_needs(self) -> list:
        needs = []
        for entry in self.plan.schedule:
            if entry.cache_from is not None:
                needs.append(("from", entry.cache_from))
            else:
                needs.append(self.layers[entry.layer][0].mixer.cache_need())
        return needs


def expected_tensors(plan: ModelPlan) -> dict[str, TensorSpec]:
    return PartTree(plan).expected_tensors()


class Model:
    """Parts bound to weights on a device, ready to run steps."""

    def __init__(self, plan: ModelPlan, runtime: Runtime, tensors: dict, max_context: int | None = None):
        self.plan = plan
        self.runtime = runtime
        self.tree = PartTree(plan, max_context)
        for built in self.tree.all_parts():
            mine = {key: tensors[built.spec.tensors[key]] for key in built.part.tensor_specs()}
            built.part.bind(mine, runtime)
        self.embedding = self.tree.embedding.part
        self.head = self.tree.head.part
        self.final_norm = self.tree.final_norm.part
        self.position = self.tree.position.part if self.tree.position is not None else None
        self.blocks = [block for block, _ in self.tree.layers]
        self.graph_safe = all(getattr(part, "graph_safe", False) for block in self.blocks
                              for part in (block.mixer_norm, block.mixer, block.feed_forward_norm, block.feed_forward))
        if self.position is not None:
            self.graph_safe = self.graph_safe and getattr(self.position, "graph_safe", False)

    def cache_needs(self) -> list:
        return self.tree.cache_needs()

    def forward(self, ctx, want_rows) -> torch.Tensor:
        """Run the schedule over ctx.batch's rows; return float32 logits
        [len(want_rows), vocab] (``want_rows``: int32 device tensor of row indices, or
        None for every row)."""
        ops = ctx.ops
        x = self.embedding.forward(ctx)
        if self.position is not None:
            x = self.position.on_embeddings(ctx, x)
        stream = Stream(x)
        for run, entry in enumerate(self.plan.schedule):
            stream = self.blocks[entry.layer].forward(ctx, stream, ctx.cache_view(run))
        if want_rows is not None and not getattr(ctx.batch, "want_all", False):  # all rows in order: nothing to gather
            stream.x = ops.gather_rows(stream.x, want_rows)
            if stream.branch is not None:
                stream.branch = ops.gather_rows(stream.branch, want_rows)
        h = self.final_norm.forward(ctx, stream)
        return self.head.forward(ctx, h)
