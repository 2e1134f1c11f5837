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

Like the reference's, which keeps up to three decode replays queued behind a ring
of pinned token buffers with one event each (engine.py:81-83,458-469), the loop
runs ahead of its consumer where the step function offers it (``open_decode_run``):
each single-token step takes its tokens on the device from the selection kernel of
the step before, so up to ``RUN_AHEAD`` steps are queued while the host reads an
earlier step's tokens. When a read shows that a sequence has stopped, nothing more
is queued; the steps already queued still ran that sequence (into pages it gives
back afterwards) and their tokens for it are dropped. The batch then goes on,
smaller, from the host's tokens.
"""

from __future__ import annotations

import time
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


@dataclass
class GenerationStats:
    """What one batch of ``run_batch`` took, by the host's clock. The reference logs
    the like per plan (``GraphPlan.stats`` and its log lines, engine/engine.py:87,206,378)."""
    sequences: int = 0
    prompt_tokens: int = 0
    prefill_ms: float = 0.0        # from the call to the first tokens on the host
    decode_steps: int = 0          # single-token steps whose tokens were read
    decode_ms: float = 0.0         # from the first tokens to the last ones
    new_tokens: int = 0

    @property
    def decode_ms_per_step(self) -> float:
        return self.decode_ms / self.decode_steps if self.decode_steps else 0.0

    @property
    def decode_tokens_per_s(self) -> float:
        decoded = self.new_tokens - self.sequences
        return decoded * 1000.0 / self.decode_ms if self.decode_ms > 0 and decoded > 0 else 0.0

    @property
    def prefill_tokens_per_s(self) -> float:
        return self.prompt_tokens * 1000.0 / self.prefill_ms if self.prefill_ms > 0 else 0.0

    def line(self) -> str:
        return (f"{self.sequences} sequences, {self.prompt_tokens} prompt tokens in {self.prefill_ms:.1f} ms "
                f"({self.prefill_tokens_per_s:.0f} tokens/s); {self.decode_steps} decode steps at "
                f"{self.decode_ms_per_step:.3f} ms ({self.decode_tokens_per_s:.0f} tokens/s)")


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
    RUN_AHEAD = 3  # single-token steps queued on the device while the host reads an earlier one

    def __init__(self, stepper, cache, sampler):
        self.stepper = stepper
        self.cache = cache
        self.sampler = sampler
        self.steps = 0
        self.stats = GenerationStats()  # of the last batch

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
        stats = self.stats = GenerationStats(len(seqs), sum(len(p) for p in prompts))
        t_begin = time.perf_counter()
        t_first = None

        def take(live, tokens):
            """Book one step's tokens; returns (what to yield, who goes on)."""
            out = [None] * len(seqs)
            still = []
            for s, tok in zip(live, tokens):
                if s.finished:  # stopped at a step read earlier: this one ran ahead of that news
                    continue
                s.produced.append(tok)
                stats.new_tokens += 1
                out[s.request - first_request] = tok
                if tok in stops:
                    s.finished, s.reason = True, "stop"
                elif len(s.produced) >= max_new_tokens:
                    s.finished, s.reason = True, "length"
                if not s.finished:
                    still.append(s)
            self.steps += 1
            return out, still

        def release(group):
            for s in group:
                if s.finished and s.slot >= 0:
                    self.cache.free(s.slot)
                    s.slot = -1

        try:
            for s in seqs:
                s.slot = self.cache.alloc()
            live = list(seqs)
            logits = self.stepper.step([StepEntry(s.slot, s.prompt, [len(s.prompt) - 1]) for s in live])
            tokens = self.sampler.select(logits, sampling, [s.request for s in live], 0)
            t_first = time.perf_counter()
            stats.prefill_ms = (t_first - t_begin) * 1e3
            out, still = take(live, tokens)
            release(live)
            live = still
            yield out
            open_run = getattr(self.stepper, "open_decode_run", None)
            while live:
                step = len(live[0].produced)  # every live sequence has produced this many tokens
                requests = [s.request for s in live]
                last = [s.produced[-1] for s in live]
                run = open_run([s.slot for s in live], last, sampling, requests, step, self.RUN_AHEAD) if open_run else None
                if run is None:  # one step at a time, tokens through the host
                    logits = self.stepper.step([StepEntry(s.slot, [t], [0]) for s, t in zip(live, last)])
                    tokens = self.sampler.select(logits, sampling, requests, step)
                    stats.decode_steps += 1
                    stats.decode_ms = (time.perf_counter() - t_first) * 1e3
                    out, still = take(live, tokens)
                    release(live)
                    live = still
                    yield out
                    continue
                # the last token of a sequence is never fed back: max_new_tokens - step steps remain
                to_launch = max_new_tokens - step
                group, stopping = live, False
                while True:
                    while to_launch > 0 and not stopping and run.in_flight < self.RUN_AHEAD:
                        run.launch()
                        to_launch -= 1
                    if run.in_flight == 0:
                        break
                    tokens = run.collect()
                    stats.decode_steps += 1
                    stats.decode_ms = (time.perf_counter() - t_first) * 1e3
                    out, still = take(group, tokens)
                    stopping = stopping or len(still) < len(live)
                    live = still
                    if any(t is not None for t in out):
                        yield out
                release(group)
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
