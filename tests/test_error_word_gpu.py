"""The kernels' error word on the serving path: a bounded wait that runs out, a bad id that reaches
the device, and what generation does about them. Nothing here faults or hangs the device: the
waiting kernel gives up after a millisecond on a barrier that nobody arrives at, and the gather
kernel bounds-checks the id, writes zeros and sets the word."""

import pytest
import torch

from helpers import prompts_for

pytestmark = pytest.mark.gpu


def engine_of(folders, name="tiny_a", **kw):
    from kernel_rush_kawk_b200 import Engine

    return Engine(folders[name], dtype="bfloat16", max_slots=4, **kw)


def test_a_wait_that_runs_out_sets_the_word_and_check_raises(folders):
    from kernel_rush_kawk_b200.csrc import KernelError

    engine = engine_of(folders)
    ops = engine.ops
    ops.check()
    ops.selftest_wait_runs_out(limit_us=1000)
    with pytest.raises(KernelError, match="ran out"):
        ops.check()
    ops.check()  # the word was cleared: the context is as usable as before
    assert len(list(engine.generate(prompts_for("tiny_a", [5]), 3))) == 3


def test_generate_raises_on_a_flag_and_the_next_request_is_right(folders):
    from kernel_rush_kawk_b200.csrc import KernelError

    engine = engine_of(folders)
    prompts = prompts_for("tiny_a", [9, 4], seed=41)
    want = list(engine.generate(prompts, 10))
    # a token id beyond the table reaches the gather kernel directly: it writes a zero row and sets the word
    bad = torch.tensor([5, 100000], dtype=torch.int32, device="cuda")
    rows = engine.ops.embed(engine.model.embedding.table, bad, 2)
    torch.cuda.synchronize()
    assert rows[1].abs().max().item() == 0
    with pytest.raises(KernelError, match="token id"):
        list(engine.generate(prompts, 10))
    assert engine.cache.live == 0, "the failed call gave its slots back"
    engine.cache.check()
    assert list(engine.generate(prompts, 10)) == want, "the flag is cleared by the raise; the next request is served"


def test_a_flag_raised_while_steps_run_ahead_surfaces_with_their_tokens(folders):
    from kernel_rush_kawk_b200.csrc import KernelError

    engine = engine_of(folders)
    prompts = prompts_for("tiny_a", [7, 3], seed=42)
    it = engine.generate(prompts, 12)
    next(it)
    next(it)
    engine.ops.selftest_wait_runs_out(limit_us=500)  # lands between queued steps
    with pytest.raises(KernelError):
        for _ in it:
            pass
    assert engine.cache.live == 0
    assert len(list(engine.generate(prompts, 4))) == 4


def test_a_multi_token_step_ends_with_a_look_at_the_word(folders):
    from kernel_rush_kawk_b200 import StepEntry
    from kernel_rush_kawk_b200.csrc import KernelError

    engine = engine_of(folders, max_tokens=1024)
    slot = engine.cache.alloc()
    engine.ops.selftest_wait_runs_out(limit_us=500)
    with pytest.raises(KernelError):
        engine.step([StepEntry(slot, [1, 2, 3], [2])])
    engine.cache.free(slot)
    slot = engine.cache.alloc()
    assert engine.step([StepEntry(slot, [1, 2, 3], [2])]).shape[0] == 1
    engine.cache.free(slot)


def test_rebuilding_the_cache_gives_its_memory_back(folders):
    """Without a fixed ``max_tokens`` the cache is rebuilt when a call needs more room; the old storage
    must go (no part of the engine may keep the old cache alive)."""
    engine = engine_of(folders)
    list(engine.generate(prompts_for("tiny_a", [5]), 2))
    torch.cuda.synchronize()
    sizes = []
    for n in (400, 900, 1500):
        list(engine.generate(prompts_for("tiny_a", [n]), 2))
        torch.cuda.synchronize()
        sizes.append((engine.cache.bytes(), torch.cuda.memory_allocated()))
    growth_cache = sizes[-1][0] - sizes[0][0]
    growth_alloc = sizes[-1][1] - sizes[0][1]
    assert growth_alloc <= growth_cache + (8 << 20), f"allocated memory grew by {growth_alloc}, the cache itself by {growth_cache}"
