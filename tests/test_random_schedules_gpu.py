"""Random schedules against the plain implementation: one to eight requests of random lengths start together
with a random piece of their prompts, bring the rest of their prompts in a second step, then go on one token
each in a shuffled order of entries until each is used up (shorter ones end earlier and give their slots back);
batch after batch through the same cache. In 32-bit and in bfloat16, on the three tiny configurations."""

import random
import zlib

import pytest
import torch

from helpers import TINY, assert_close, plain_logits, tiny_config

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", TINY)
def test_random_schedules(folders, name, dtype):
    from kernel_rush_kawk_b200 import Engine, StepEntry

    rnd = random.Random(zlib.crc32(f"{name} {dtype}".encode()))  # the same schedules in every run
    vocab = tiny_config(name).vocab_size
    engine = Engine(folders[name], dtype=dtype, max_tokens=4096, max_slots=8, max_context=512)
    cache = engine.cache
    for batch_no in range(5):
        n = rnd.randint(1, 8)
        seqs = [[rnd.randrange(vocab) for _ in range(rnd.randint(1, 200))] for _ in range(n)]
        cuts = [rnd.randint(1, len(s)) for s in seqs]
        first = [rnd.randint(1, c) for c in cuts]
        slots = [cache.alloc() for _ in seqs]
        got = [[] for _ in seqs]
        out = engine.step([StepEntry(sl, s[:f], list(range(f))) for sl, s, f in zip(slots, seqs, first)]).float().cpu()
        row = 0
        for i, f in enumerate(first):
            got[i].append(out[row:row + f])
            row += f
        more = [i for i in range(n) if first[i] < cuts[i]]
        if more:
            out = engine.step([StepEntry(slots[i], seqs[i][first[i]:cuts[i]], list(range(cuts[i] - first[i])))
                               for i in more]).float().cpu()
            row = 0
            for i in more:
                k = cuts[i] - first[i]
                got[i].append(out[row:row + k])
                row += k
        fed = list(cuts)
        live = [i for i in range(n) if fed[i] < len(seqs[i])]
        for i in range(n):
            if i not in live:
                cache.free(slots[i])
        while live:
            rnd.shuffle(live)
            out = engine.step([StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live]).float().cpu()
            still = []
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1])
                fed[i] += 1
                if fed[i] < len(seqs[i]):
                    still.append(i)
                else:
                    cache.free(slots[i])
            live = still
        cache.check()
        engine.ops.check()
        for i, seq in enumerate(seqs):
            assert_close(torch.cat(got[i]), plain_logits(folders[name], name, seq, dtype), dtype,
                         f"{name} {dtype}, batch {batch_no}, request {i} of {len(seq)} tokens")
    assert cache.live == 0
