"""The generation loop above the step function.

A batch of prompts of unequal lengths starts together: all prompts in one step,
then one token per live sequence per step. A sequence ends when it has produced
``max_new_tokens`` tokens or one of its stop tokens; it then gives its slot and
pages back and the batch goes on without it. ``run_requests`` runs as many
batches one after another as the requests need, each batch as large as the
cache allows.

The reference's loop (``GraphPlan.run``, engine/engine.py:438-469 of
willzeng274/kernel-rush-kawk) serves equal-length prompts, never stops on a
token (EOS is an ordinary id: AGENTS.md:19-21) and yields exactly
``max_new_tokens`` lists. With no stop tokens this loop yields the same.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..cache.store import PAGE
from ..sampling.sampler import SamplingParams
from .step import StepEntry


@dataclass
class Sequence:
    request: int
    prompt: list
    slot: int = -1
    produced: list = field(default_factory=list)
    finished: bool = False
    reason: str = ""


def pages_needed(prompt_len: int, max_new_tokens: int) -> int:
    """Pages a sequence may come to hold: the last generated token is never fed back."""
    return -(-(prompt_len + max(max_new_tokens - 1, 0)) // PAGE)


def split_into_batches(prompt_lens: list, max_new_tokens: int, max_slots: int, max_pages: int) -> list:
    """Consecutive requests are grouped while slots and pages last. Returns lists of
    request indices. A request that cannot fit even alone raises ValueError."""
    batches, current, pages = [], [], 0
    for i, n in enumerate(prompt_lens):
        need = pages_needed(n, max_new_tokens)
        if need > max_pages:
            raise ValueError(f"request {i} needs {need * PAGE} cached tokens; the cache holds {max_pages * PAGE}")
        if current and (len(current) >= max_slots or pages + need > max_pages):
            batches.append(current)
            current, pages = [], 0
        current.append(i)
        pages += need
    if current:
        batches.append(current)
    return batches


class GenerationLoop:
    def __init__(self, stepper, cache, sampler):
        self.stepper = stepper
        self.cache = cache
        self.sampler = sampler
        self.steps = 0

    def run_batch(self, prompts: list, max_new_tokens: int, sampling: SamplingParams = SamplingParams(),
                  stop_token_ids=(), first_request: int = 0):
        """Generator: yields, per step, a list with one entry per prompt: the new token
        id, or None for a sequence that ended at an earlier step."""
        if max_new_tokens < 1 or not prompts:
            return
        for i, p in enumerate(prompts):
            if len(p) == 0:
                raise ValueError(f"prompt {i} is empty")
        stops = frozenset(int(t) for t in stop_token_ids)
        seqs = [Sequence(first_request + i, list(p)) for i, p in enumerate(prompts)]
        try:
            for s in seqs:
                s.slot = self.cache.alloc()
            live = list(seqs)
            entries = [StepEntry(s.slot, s.prompt, [len(s.prompt) - 1]) for s in live]
            step = 0
            overlap = hasattr(self.sampler, "launch") and hasattr(self.stepper, "prepare_single_tokens")
            while live:
                logits = self.stepper.step(entries)
                requests = [s.request for s in live]
                if overlap and step + 1 < max_new_tokens:
                    # while the device computes: the host's share of the next step, as if nobody stopped
                    pending = self.sampler.launch(logits, sampling, requests, step)
                    self.stepper.prepare_single_tokens([s.slot for s in live])
                    tokens = self.sampler.finish(pending)
                else:
                    tokens = self.sampler.select(logits, sampling, requests, step)
                self.steps += 1
                out = [None] * len(seqs)
                still = []
                for s, tok in zip(live, tokens):
                    s.produced.append(tok)
                    out[s.request - first_request] = tok
                    if tok in stops:
                        s.finished, s.reason = True, "stop"
                    elif len(s.produced) >= max_new_tokens:
                        s.finished, s.reason = True, "length"
                    if s.finished:
                        self.cache.free(s.slot)
                        s.slot = -1
                    else:
                        still.append(s)
                live = still
                entries = [StepEntry(s.slot, [s.produced[-1]], [0]) for s in live]
                step += 1
                yield out
        finally:
            for s in seqs:
                if s.slot >= 0:
                    self.cache.free(s.slot)
                    s.slot = -1

    def run_requests(self, prompts: list, max_new_tokens: int, sampling: SamplingParams = SamplingParams(),
                     stop_token_ids=(), max_batch: int | None = None) -> list:
        """Run every request, batch after batch; returns each request's generated tokens."""
        max_slots = min(self.cache.max_slots, max_batch or self.cache.max_slots)
        batches = split_into_batches([len(p) for p in prompts], max_new_tokens, max_slots, self.cache.n_pages)
        results: list = [None] * len(prompts)
        for batch in batches:
            outs = [[] for _ in batch]
            for step_out in self.run_batch([prompts[i] for i in batch], max_new_tokens, sampling, stop_token_ids,
                                           first_request=batch[0]):
                for j, tok in enumerate(step_out):
                    if tok is not None:
                        outs[j].append(tok)
            for j, i in enumerate(batch):
                results[i] = outs[j]
        return results
