"""The Python entry point, in the reference's manner.

``Engine(model_path)`` and ``Engine.generate(input_ids, max_new_tokens)``, a
generator that yields one list of token ids per step, are the reference's own
entry (engine/engine.py:472,480,590 and README.md:59-70 of
willzeng274/kernel-rush-kawk). The defaults keep its meaning: greedy, no stop
token (EOS is an ordinary id), exactly ``max_new_tokens`` yields. Keyword
options add what the reference lacks: unequal prompt lengths need no option;
``temperature`` and ``seed`` sample; ``stop_token_ids`` end a sequence early (its
place then holds None); ``dtype`` picks the bfloat16 serving path or the true
float32 path. After a call ``Engine.last_stats`` holds the batch's times (the
reference logs the like: engine/engine.py:206,378); a kernel that flagged bad
input or gave up on a wait makes the call raise ``KernelError``.

Like the reference, which turns TF32 off at construction (engine.py:481-482),
the engine forbids reduced-precision matrix modes for the library products it
calls.
"""

from __future__ import annotations

import logging
import os
import time
from pathlib import Path

import torch

from ..cache.store import PAGE, SequenceCache
from ..config.registry import get_architecture, preset_config, read_config
from ..sampling.sampler import Sampler, SamplingParams
from ..weights.loader import read_checkpoint
from ..weights.random_init import random_tensors
from .generate import GenerationLoop, pages_needed
from .model import Model, PartTree, Runtime
from .step import StepEntry, Stepper

log = logging.getLogger(__name__)

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32,
}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return _DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


def _default_ops(device: torch.device, head_dims):
    if device.type != "cuda":
        raise RuntimeError("this engine computes with its CUDA extension only; there is no CPU path "
                           f"(asked for device '{device}')")
    from ..csrc import load_kernels
    return load_kernels(head_dims)


class Engine:
    def __init__(self, model_path=None, *, dtype="bfloat16", max_tokens: int | None = None, max_slots: int = 64,
                 max_context: int | None = None, use_cuda_graphs: bool = True, max_step_rows: int = 16384,
                 step_tokens: int = 2048, device="cuda:0", ops=None, _config=None, _tensors=None):
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        self.device = torch.device(device)
        self.dtype = parse_dtype(dtype)
        t0 = time.perf_counter()
        if _config is not None:
            self.architecture, self.config = get_architecture(_config.architecture), _config
        else:
            if model_path is None:
                raise ValueError("Engine needs a model folder (or use Engine.from_random)")
            self.architecture, self.config = read_config(model_path)
        self.model_path = None if model_path is None else Path(model_path)
        self.plan = self.architecture.plan(self.config)
        self.max_context = min(int(max_context or self.plan.max_positions), self.plan.max_positions)
        tree = PartTree(self.plan, self.max_context)
        head_dims = sorted({n.head_dim for n in tree.cache_needs() if hasattr(n, "head_dim")})
        self.ops = ops if ops is not None else _default_ops(self.device, head_dims)
        expected = tree.expected_tensors()
        if _tensors is None:
            tensors = read_checkpoint(self.model_path, expected, self.device, self.dtype, self.plan.duplicates)
        else:
            tensors = {}
            for name, spec in expected.items():
                t = _tensors[name]
                keep = self.dtype if (t.dim() > 1 or self.dtype == torch.float32) else t.dtype
                tensors[name] = t.to(device=self.device, dtype=keep).contiguous()
        self.model = Model(self.plan, Runtime(self.device, self.dtype, self.ops), tensors, self.max_context)
        self.max_slots = int(max_slots)
        self.max_tokens = max_tokens
        # the reference's own switch, same name and meaning (engine/engine.py:487)
        self.use_cuda_graphs = bool(use_cuda_graphs) and os.environ.get("ENGINE_NO_GRAPHS") is None
        self.max_step_rows = max_step_rows
        # the most tokens of one sequence in one pass where a layer keeps a window of keys: it sizes that
        # layer's ring of pages (window + step_tokens positions); longer steps are cut into passes
        self.step_tokens = int(step_tokens)
        self.cache = self.stepper = self.loop = None
        self.sampler = Sampler(self.ops, self.device)
        self.last_stats = None  # GenerationStats of the last batch that generate / generate_all ran
        if max_tokens is not None:
            self._build_cache(int(max_tokens), self.max_slots)
        log.info("engine ready in %.1fs (%s, %s)", time.perf_counter() - t0, self.plan.architecture, self.dtype)

    # -- construction -------------------------------------------------------
    @classmethod
    def from_random(cls, config, seed: int = 0, std: float = 0.02, **options) -> "Engine":
        """Random weights for a configuration (an instance, or a preset's name), drawn
        on the engine's device from (tensor name, seed)."""
        if isinstance(config, str):
            config = preset_config(config)
        arch = get_architecture(config.architecture)
        device = torch.device(options.get("device", "cuda:0"))
        expected = PartTree(arch.plan(config)).expected_tensors()
        tensors = random_tensors(expected, seed, std, device)
        return cls(None, _config=config, _tensors=tensors, **options)

    def _build_cache(self, max_tokens: int, max_slots: int) -> None:
        if self.cache is not None and self.cache.live:
            raise RuntimeError(f"the cache cannot be rebuilt while {self.cache.live} sequences are live in it "
                               "(an earlier generate() is still open: finish or close it first)")
        self.cache = self.stepper = self.loop = None  # drop the old storage and graphs first
        if self.device.type == "cuda":
            torch.cuda.empty_cache()
        self.cache = SequenceCache(self.model.cache_needs(), max_tokens, max_slots, self.max_context, self.device,
                                   self.dtype, step_tokens=self.step_tokens)
        self.stepper = Stepper(self.model, self.cache, self.ops, self.max_step_rows, self.use_cuda_graphs)
        self.loop = GenerationLoop(self.stepper, self.cache, self.sampler)

    def _ensure_cache(self, prompt_lens, max_new_tokens: int) -> None:
        """Without a fixed ``max_tokens`` the cache grows to what a call needs, as the
        reference rebuilds its plan for a new shape (engine/engine.py:562-588)."""
        pages = sum(pages_needed(n, max_new_tokens) for n in prompt_lens)
        slots = max(self.max_slots, min(len(prompt_lens), 1024))
        if self.cache is not None and (self.max_tokens is not None or (
                self.cache.n_pages >= pages and self.cache.max_slots >= min(len(prompt_lens), slots))):
            return
        self._build_cache(pages * PAGE, slots)

    # -- the reference's entry ------------------------------------------------
    def generate(self, input_ids, max_new_tokens: int, *, temperature: float = 0.0, seed: int = 0,
                 stop_token_ids=()):
        """Yield, per step, one token id per sequence (None once a sequence has ended
        on a stop token). All sequences start together; their lengths may differ.

        This is a generator: arguments are checked, and a cache without a fixed size is
        grown if the call needs more room, at the first ``next()``. One generation runs
        at a time: growing the cache while an earlier generator still holds sequences
        raises."""
        prompts = [list(map(int, row)) for row in input_ids]
        if max_new_tokens < 1 or not prompts:
            return
        for row in prompts:
            if len(row) + max_new_tokens - 1 > self.max_context:
                raise ValueError(f"a prompt of {len(row)} tokens plus {max_new_tokens} new ones exceeds "
                                 f"the context of {self.max_context}")
        self._ensure_cache([len(p) for p in prompts], max_new_tokens)
        try:
            yield from self.loop.run_batch(prompts, max_new_tokens, SamplingParams(temperature, seed), stop_token_ids)
        finally:
            self.last_stats = self.loop.stats
            log.info("generate: %s", self.last_stats.line())

    def generate_all(self, input_ids, max_new_tokens: int, *, temperature: float = 0.0, seed: int = 0,
                     stop_token_ids=(), max_batch: int | None = None) -> list:
        """Any number of requests, run as consecutive batches; returns each request's tokens."""
        prompts = [list(map(int, row)) for row in input_ids]
        if not prompts or max_new_tokens < 1:
            return [[] for _ in prompts]
        if self.max_tokens is None:  # no fixed size: room for the largest batch these requests can form
            lens = sorted((len(p) for p in prompts), reverse=True)[:max_batch or self.max_slots]
            self._ensure_cache(lens, max_new_tokens)
        try:
            return self.loop.run_requests(prompts, max_new_tokens, SamplingParams(temperature, seed), stop_token_ids,
                                          max_batch)
        finally:
            self.last_stats = self.loop.stats
            log.info("generate_all, last batch: %s", self.last_stats.line())

    # -- lower level, for replay and tests --------------------------------------
    def open_cache(self, max_tokens: int, max_slots: int | None = None) -> None:
        self.max_tokens = int(max_tokens)
        self._build_cache(self.max_tokens, int(max_slots or self.max_slots))

    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        return self.stepper.step(entries)
