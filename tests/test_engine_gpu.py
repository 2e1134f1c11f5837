"""The engine against the plain implementation, on the GPU, in 32-bit and bfloat16:
whole requests, the last 32 tokens one by one, unequal batches with slot reuse,
long decoding, first tokens, greedy generation through the entry point."""

import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY, assert_close, plain_logits, prompts_for

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")
_engines: dict = {}


def engine_for(folders, name, dtype, graphs=True):
    from kernel_rush_kawk_b200 import Engine

    key = (name, dtype, graphs)
    if key not in _engines:
        _engines[key] = Engine(folders[name], dtype=dtype, max_tokens=8192, max_slots=8, use_cuda_graphs=graphs)
    return _engines[key]


def run_schedule(engine, sequences, prompt_lens):
    """All requests start together with their prompts (all positions wanted), then
    go on one token each, teacher-forced, until each sequence is used up; shorter
    ones end earlier. Returns the logits [len, vocab] of every request."""
    from kernel_rush_kawk_b200 import StepEntry

    cache = engine.cache
    slots = [cache.alloc() for _ in sequences]
    got = [[] for _ in sequences]
    out = engine.step([StepEntry(s, seq[:p], list(range(p))) for s, seq, p in zip(slots, sequences, prompt_lens)])
    row = 0
    for i, p in enumerate(prompt_lens):
        got[i].append(out[row:row + p].float().cpu())
        row += p
    fed = list(prompt_lens)
    live = [i for i in range(len(sequences)) if fed[i] < len(sequences[i])]
    for i in range(len(sequences)):
        if i not in live:
            cache.free(slots[i])
    while live:
        out = engine.step([StepEntry(slots[i], [sequences[i][fed[i]]], [0]) for i in live]).float().cpu()
        still = []
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1])
            fed[i] += 1
            if fed[i] < len(sequences[i]):
                still.append(i)
            else:
                cache.free(slots[i])
        live = still
    cache.check()
    return [torch.cat(g) for g in got]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", TINY)
def test_each_request_alone_and_whole(folders, name, dtype):
    engine = engine_for(folders, name, dtype)
    for seq in prompts_for(name, [1, 2, 7, 64, 65, 150], seed=1):
        got = run_schedule(engine, [seq], [len(seq)])[0]
        assert_close(got, plain_logits(folders[name], name, seq, dtype), dtype, f"{name} whole, {len(seq)} tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", TINY)
def test_last_32_tokens_one_by_one(folders, name, dtype):
    engine = engine_for(folders, name, dtype)
    for seq in prompts_for(name, [33, 100, 130], seed=2):
        got = run_schedule(engine, [seq], [len(seq) - 32])[0]
        assert_close(got, plain_logits(folders[name], name, seq, dtype), dtype, f"{name} last 32 of {len(seq)}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", TINY)
def test_unequal_batches_one_after_another(folders, name, dtype):
    """Two batches through the same cache: the second reuses the slots and pages the
    first gave back, with other lengths, so stale keys would show."""
    engine = engine_for(folders, name, dtype)
    for seed, lengths, prompt_lens in ((3, [40, 9, 101, 70], [5, 8, 66, 64]), (4, [77, 130, 12], [70, 1, 11])):
        seqs = prompts_for(name, lengths, seed=seed)
        got = run_schedule(engine, seqs, prompt_lens)
        for seq, g in zip(seqs, got):
            assert_close(g, plain_logits(folders[name], name, seq, dtype), dtype,
                         f"{name} batch seed {seed}, request of {len(seq)}")
    assert engine.cache.live == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(folders, dtype):
    name = "tiny_w"
    engine = engine_for(folders, name, dtype)
    seq = prompts_for(name, [260], seed=5)[0]
    got = run_schedule(engine, [seq], [3])[0]
    assert_close(got, plain_logits(folders[name], name, seq, dtype), dtype, "long decoding over four pages")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", TINY)
def test_graph_and_eager_decode_agree(folders, name, dtype):
    seqs = prompts_for(name, [20, 45], seed=6)
    a = run_schedule(engine_for(folders, name, dtype, True), seqs, [10, 30])
    b = run_schedule(engine_for(folders, name, dtype, False), seqs, [10, 30])
    for x, y in zip(a, b):
        assert torch.equal(x, y), "a captured decode step must compute what the eager step computes"


@pytest.mark.parametrize("name", TINY)
def test_batch_company_changes_nothing_in_32_bit(folders, name):
    """In the 32-bit path a request's logits do not depend on what else is in the batch,
    nor on where in the cache it lies: bit-equal."""
    engine = engine_for(folders, name, "float32")
    seqs = prompts_for(name, [50, 90, 17], seed=7)
    alone = run_schedule(engine, [seqs[0]], [30])[0]
    held = engine.cache.alloc()  # shifts the slots and pages the next run gets
    together = run_schedule(engine, seqs, [30, 64, 2])[0]
    engine.cache.free(held)
    assert torch.equal(alone, together)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", TINY)
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    from kernel_rush_kawk_b200 import Engine

    engine = Engine(folders[name], dtype=dtype, max_slots=4)
    prompts = prompts_for(name, [5, 11, 17], seed=8)
    steps = list(engine.generate(prompts, 8))
    assert len(steps) == 8 and all(len(s) == 3 for s in steps)
    cfg, w = plain.read_folder(folders[name])
    from helpers import assert_greedy_token, windows_of
    for i, prompt in enumerate(prompts):
        seq = list(prompt)
        for t in range(8):
            # the engine's token is the plain argmax, or ties with it within the noise of the arithmetic
            assert_greedy_token(cfg, w, seq, steps[t][i], dtype, windows_of(name), f"{name} {dtype} request {i} step {t}")
            seq.append(steps[t][i])
    # a second call with other prompts reuses the slots (the reference's advice: two
    # consecutive generations with different prompts, OPTIMIZATION_GUIDE.md:412-418)
    again = list(engine.generate(prompts_for(name, [9, 3], seed=9), 4))
    assert len(again) == 4 and engine.cache.live == 0


def test_temperature_sampling_through_the_entry_point(folders):
    """tiny_b, temperature 0.8, fixed seed: each sampled token is the plain sampler's draw
    from the engine's own 32-bit logits for the same (seed, request, step)."""
    from kernel_rush_kawk_b200 import Engine

    name = "tiny_b"
    engine = Engine(folders[name], dtype="float32", max_slots=4)
    prompts = prompts_for(name, [1, 7, 13, 24], seed=10)
    steps = list(engine.generate(prompts, 10, temperature=0.8, seed=1234))
    cfg, w = plain.read_folder(folders[name])
    for i, prompt in enumerate(prompts):
        seq = list(prompt)
        for t in range(10):
            ref = plain.forward_logits(cfg, w, seq, torch.float64)[-1]
            want = plain.sample_temperature(ref, 0.8, 1234, i, t)
            assert steps[t][i] == want, (i, t)
            seq.append(steps[t][i])
    # the same request alone draws the same tokens: a draw does not depend on the batch
    alone = [s[0] for s in engine.generate([prompts[0]], 10, temperature=0.8, seed=1234)]
    assert alone == [s[0] for s in steps]


@pytest.mark.parametrize("dtype", DTYPES)
def test_stop_tokens_end_a_sequence_early(folders, dtype):
    """Request 0 stops on its third token. The loop had queued steps beyond that one; the other
    request's tokens must be what they are without any stop, at every step, and request 0's place
    holds None from then on."""
    from kernel_rush_kawk_b200 import Engine

    name = "tiny_a"
    engine = Engine(folders[name], dtype=dtype, max_slots=4)
    prompts = prompts_for(name, [6, 9, 70], seed=11)
    free_run = list(engine.generate(prompts, 12))
    stop = free_run[2][0]  # the third token of request 0
    steps = list(engine.generate(prompts, 12, stop_token_ids=[stop]))
    assert len(steps) == 12
    ended = [None, None, None]
    for t, step in enumerate(steps):
        for r in range(3):
            if ended[r] is not None:
                assert step[r] is None, (t, r)
            else:
                assert step[r] == free_run[t][r], f"request {r} at step {t}: {step[r]} against {free_run[t][r]} without a stop"
                if step[r] == stop:
                    ended[r] = t
    assert ended[0] is not None and ended[0] <= 2
    assert engine.cache.live == 0
    engine.cache.check()
    # a batch right after it, on the slots and pages just given back
    again = list(engine.generate(prompts, 12))
    assert again == free_run


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_steps_fed_on_the_device_choose_the_same_tokens(folders, graphs, temperature):
    """``decode_on_device`` runs single-token steps without a host round trip (the selection kernel writes
    each step's tokens and positions into the next step's batch description). It must choose exactly the
    tokens that the generation loop chooses with the host in between, for unequal prompts, greedily and
    with temperature sampling, across a page boundary."""
    from kernel_rush_kawk_b200 import StepEntry

    name, dtype = "tiny_b", "bfloat16"
    engine = engine_for(folders, name, dtype, graphs)
    prompts = prompts_for(name, [60, 5, 33], seed=21)
    new = 12
    by_loop = list(engine.generate(prompts, new, temperature=temperature, seed=7))
    cache = engine.cache
    slots = [cache.alloc() for _ in prompts]
    logits = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    first = engine.ops.select_tokens(logits, temperature, 7, torch.arange(3, dtype=torch.int32, device="cuda"), 0).tolist()
    assert first == by_loop[0]
    rest = engine.stepper.decode_on_device(slots, first, new - 1, temperature=temperature, seed=7, first_step=1).tolist()
    assert rest == by_loop[1:], "device-fed steps must choose what the host-driven loop chooses"
    for s in slots:
        cache.free(s)
    cache.check()
    engine.ops.check()
