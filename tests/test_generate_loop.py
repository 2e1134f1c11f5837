"""The generation loop's decisions (no GPU): who is live, who ends, what is given
back, how requests are split into batches. The step function and the sampler are
scripted stand-ins; the loop is the product's."""

import pytest
import torch

from kernel_rush_kawk_b200.cache import SequenceCache
from kernel_rush_kawk_b200.engine.generate import GenerationLoop, pages_needed, split_into_batches
from kernel_rush_kawk_b200.parts.base import KVNeed
from kernel_rush_kawk_b200.sampling import SamplingParams


class ScriptedStepper:
    """Returns, as "logits", the slots of the step's entries; records what it was asked."""

    def __init__(self, cache):
        self.cache, self.calls = cache, []

    def step(self, entries):
        self.calls.append([(e.slot, list(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            self.cache.reserve(e.slot, self.cache.length[e.slot] + len(e.tokens))
            self.cache.advance(e.slot, len(e.tokens))
        return torch.zeros(len(entries), 4)


class ScriptedSampler:
    """Request r produces script[r][step]."""

    def __init__(self, script):
        self.script, self.calls = script, []

    def select(self, logits, params, requests, step):
        self.calls.append((list(requests), step))
        return [self.script[r][step] for r in requests]


def make(script, max_tokens=64 * 16, max_slots=4):
    cache = SequenceCache([KVNeed(1, 8)], max_tokens, max_slots, 64 * 8, "cpu", torch.float32)
    stepper, sampler = ScriptedStepper(cache), ScriptedSampler(script)
    return GenerationLoop(stepper, cache, sampler), cache, stepper, sampler


def test_unequal_prompts_one_step_then_one_token_each():
    loop, cache, stepper, sampler = make({0: [10, 11, 12], 1: [20, 21, 22]})
    out = list(loop.run_batch([[1, 2, 3], [4]], 3))
    assert out == [[10, 20], [11, 21], [12, 22]]
    first, second = stepper.calls[0], stepper.calls[1]
    assert [(t, w) for _, t, w in first] == [([1, 2, 3], [2]), ([4], [0])]  # whole prompts, last place wanted
    assert [(t, w) for _, t, w in second] == [([10], [0]), ([20], [0])]
    assert len(stepper.calls) == 3  # the last token is never fed back
    assert cache.live == 0
    cache.check()


def test_stop_tokens_and_earlier_ends():
    loop, cache, stepper, sampler = make({0: [5, 99, 7, 8], 1: [6, 6, 6, 99], 2: [99, 1, 1, 1]})
    out = list(loop.run_batch([[1], [2, 2], [3]], 4, stop_token_ids=[99]))
    assert out == [[5, 6, 99], [99, 6, None], [None, 6, None], [None, 99, None]]
    assert [len(c) for c in stepper.calls] == [3, 2, 1, 1]  # the batch shrinks as sequences end
    assert sampler.calls == [([0, 1, 2], 0), ([0, 1], 1), ([1], 2), ([1], 3)]
    assert cache.live == 0


def test_slots_come_back_when_the_consumer_stops_early_or_a_step_fails():
    loop, cache, stepper, _ = make({0: [1, 2, 3]})
    it = loop.run_batch([[7, 7]], 3)
    next(it)
    it.close()
    assert cache.live == 0

    def boom(entries):
        raise RuntimeError("device lost")
    stepper.step = boom
    with pytest.raises(RuntimeError):
        list(loop.run_batch([[7]], 2))
    assert cache.live == 0
    cache.check()


def test_nothing_to_do_and_bad_input():
    loop, cache, _, _ = make({})
    assert list(loop.run_batch([[1]], 0)) == [] and list(loop.run_batch([], 3)) == []
    with pytest.raises(ValueError, match="empty"):
        list(loop.run_batch([[1], []], 2))


def test_requests_are_split_into_batches_by_slots_and_pages():
    assert pages_needed(64, 1) == 1 and pages_needed(64, 2) == 2 and pages_needed(1, 64) == 1
    assert split_into_batches([10] * 5, 4, max_slots=2, max_pages=100) == [[0, 1], [2, 3], [4]]
    assert split_into_batches([100, 100, 100], 30, max_slots=8, max_pages=6) == [[0, 1], [2]]
    with pytest.raises(ValueError, match="request 1 needs"):
        split_into_batches([10, 1000], 4, 8, 4)


def test_batches_run_one_after_another_and_reuse_slots():
    script = {r: [100 + r, 200 + r] for r in range(5)}
    script[3] = [99, 0]
    loop, cache, stepper, sampler = make(script, max_slots=2)
    results = loop.run_requests([[1]] * 5, 2, SamplingParams(), stop_token_ids=[99])
    assert results == [[100, 200], [101, 201], [102, 202], [99], [104, 204]]
    slots_used = {slot for call in stepper.calls for slot, _, _ in call}
    assert slots_used <= {0, 1}  # five requests went through two slots
    assert [c[0] for c in sampler.calls if c[1] == 0] == [[0, 1], [2, 3], [4]]
    assert cache.live == 0
    cache.check()


class ScriptedRun:
    """A stand-in for the step function's DecodeRun: steps are "queued" by counting them, and a
    collected step yields request r's script[r][step]."""

    def __init__(self, owner, slots, requests, first_step, depth):
        self.owner, self.slots, self.requests, self.step, self.depth = owner, slots, requests, first_step, depth
        self.launched = self.collected = 0

    @property
    def in_flight(self):
        return self.launched - self.collected

    def launch(self):
        assert self.in_flight < self.depth
        for s in self.slots:
            self.owner.cache.reserve(s, self.owner.cache.length[s] + 1)
            self.owner.cache.advance(s, 1)
        self.launched += 1
        self.owner.most_in_flight = max(self.owner.most_in_flight, self.in_flight)

    def collect(self):
        step = self.step + self.collected
        self.collected += 1
        self.owner.collected.append((list(self.requests), step))
        return [self.owner.script[r][step] for r in self.requests]


class RunAheadStepper(ScriptedStepper):
    def __init__(self, cache, script):
        super().__init__(cache)
        self.script, self.runs, self.collected, self.most_in_flight = script, [], [], 0

    def open_decode_run(self, slots, tokens, sampling, requests, first_step, depth):
        self.runs.append((list(requests), list(tokens), first_step))
        return ScriptedRun(self, list(slots), list(requests), first_step, depth)


def make_ahead(script, max_slots=4):
    cache = SequenceCache([KVNeed(1, 8)], 64 * 16, max_slots, 64 * 8, "cpu", torch.float32)
    stepper = RunAheadStepper(cache, script)
    return GenerationLoop(stepper, cache, ScriptedSampler(script)), cache, stepper


def test_steps_run_ahead_of_the_consumer_and_never_past_the_last_token():
    loop, cache, stepper = make_ahead({0: list(range(10, 17)), 1: list(range(20, 27))})
    out = list(loop.run_batch([[1, 2], [3]], 7))
    assert out == [[10 + t, 20 + t] for t in range(7)]
    assert stepper.runs == [([0, 1], [10, 20], 1)]  # one run from the first tokens on
    assert stepper.most_in_flight == GenerationLoop.RUN_AHEAD
    assert [c[1] for c in stepper.collected] == [1, 2, 3, 4, 5, 6]  # the seventh token is never fed back
    assert cache.live == 0 and max(cache.length) == 0
    cache.check()


def test_a_stop_read_late_drops_what_ran_ahead_for_that_sequence_only():
    """Request 0 stops at step 2. Steps 3 and 4 were queued before the host read that: request 1's
    tokens from them count, request 0's are dropped, and a new run goes on with request 1 alone."""
    script = {0: [5, 6, 99, 1, 2, 3, 4, 5], 1: [7, 8, 9, 10, 11, 12, 13, 14]}
    loop, cache, stepper = make_ahead(script)
    out = list(loop.run_batch([[1], [2]], 8, stop_token_ids=[99]))
    assert out == [[5, 7], [6, 8], [99, 9], [None, 10], [None, 11], [None, 12], [None, 13], [None, 14]]
    assert stepper.runs[0] == ([0, 1], [5, 7], 1)
    assert stepper.runs[1][0] == [1] and stepper.runs[1][1] == [script[1][stepper.runs[1][2] - 1]]
    assert cache.live == 0
    cache.check()


def test_a_lone_sequence_that_stops_yields_nothing_after_its_stop():
    loop, cache, stepper = make_ahead({0: [1, 99, 3, 4, 5, 6]})
    assert list(loop.run_batch([[4]], 6, stop_token_ids=[99])) == [[1], [99]]
    assert cache.live == 0
