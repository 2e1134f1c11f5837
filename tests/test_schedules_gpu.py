"""Schedules that only show on the device: a window's ring of pages that wraps, a step cut into
passes, more requests than slots, and the 8B and 14B workloads at two layers."""

import pytest
import torch

import plain_qwen3 as plain
from helpers import assert_close, assert_greedy_token, plain_logits, prompts_for, windows_of

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")


def feed(engine, slot, seq, pieces, tail_one_by_one=True):
    """One request: its tokens in the given pieces (every place wanted), then one by one."""
    from kernel_rush_kawk_b200 import StepEntry

    got, at = [], 0
    for n in pieces:
        got.append(engine.step([StepEntry(slot, seq[at:at + n], list(range(n)))]).float().cpu())
        at += n
    while at < len(seq):
        got.append(engine.step([StepEntry(slot, [seq[at]], [0])]).float().cpu())
        at += 1
    return torch.cat(got)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,step_tokens", [("tiny_v", 64), ("tiny_w", 40)])
def test_a_windowed_sequence_outgrows_its_ring_of_pages(folders, name, step_tokens, dtype):
    """With ``step_tokens`` 64 and a window of 70 the ring holds 4 pages (256 positions), with 40 and 24
    it holds 2; the sequences run to 700 positions, so every ring entry is reused many times: by
    passes of a whole prompt, by pieces that end on and beside a page boundary, and token by token.
    tiny_v has head size 64 (the tensor-core prefill kernel and the fused single-token kernel)."""
    from kernel_rush_kawk_b200 import Engine

    engine = Engine(folders[name], dtype=dtype, max_tokens=4096, max_slots=3, step_tokens=step_tokens)
    ring = [g.width for g in engine.cache._kv_groups if g.need.window is not None]
    assert ring and max(ring) * 64 < 500, f"the ring ({ring} pages) must be shorter than the sequences"
    seqs = prompts_for(name, [700, 500, 330], seed=31)
    refs = [plain_logits(folders[name], name, s, dtype) for s in seqs]
    cache = engine.cache
    # (1) whole: one step of 700 tokens, cut into passes that go round the ring
    slot = cache.alloc()
    assert_close(feed(engine, slot, seqs[0], [700]), refs[0], dtype, f"{name} whole through a wrapping ring")
    cache.free(slot)
    # (2) pieces: 2 tokens, up to a page boundary, across several pages, then 150 tokens one by one
    slot = cache.alloc()
    assert_close(feed(engine, slot, seqs[1], [2, 62, 100, 186]), refs[1], dtype, f"{name} pieces, then token by token")
    cache.free(slot)
    # (3) almost all token by token
    slot = cache.alloc()
    assert_close(feed(engine, slot, seqs[2], [3]), refs[2], dtype, f"{name} token by token round the ring")
    cache.free(slot)
    cache.check()
    engine.ops.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_step_cut_into_passes_on_the_device(folders, dtype):
    """``max_step_rows`` 48: a batch of 100 + 30 + 75 tokens runs as passes of at most 48 rows, a pass
    holding pieces of several requests; wanted places come back in the order asked."""
    from kernel_rush_kawk_b200 import Engine, StepEntry

    name = "tiny_w"
    engine = Engine(folders[name], dtype=dtype, max_tokens=2048, max_slots=4, max_step_rows=48, step_tokens=40)
    seqs = prompts_for(name, [100, 30, 75], seed=32)
    refs = [plain_logits(folders[name], name, s, dtype) for s in seqs]
    slots = [engine.cache.alloc() for _ in seqs]
    wants = [[99, 0, 47, 48], [29], [74, 40, 39]]
    before = engine.stepper.passes
    out = engine.step([StepEntry(sl, s, w) for sl, s, w in zip(slots, seqs, wants)])
    assert engine.stepper.passes - before >= 5
    want = torch.stack([refs[i][w] for i, ws in enumerate(wants) for w in ws])
    assert_close(out, want, dtype, "cut step on the device, order of wanted places")
    # and the cache it left serves the next tokens
    nxt = prompts_for(name, [1, 1, 1], seed=33)
    out = engine.step([StepEntry(sl, t, [0]) for sl, t in zip(slots, nxt)])
    want = torch.stack([plain_logits(folders[name], name, s + t, dtype)[-1] for s, t in zip(seqs, nxt)])
    assert_close(out, want, dtype, "the token after a cut step")
    for s in slots:
        engine.cache.free(s)
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_more_requests_than_slots_run_batch_after_batch(folders, dtype):
    """Seven requests of unequal lengths through three slots: ``generate_all`` forms batches, each on
    the slots and pages the one before gave back; every token is checked against the plain
    implementation on the request's own sequence."""
    from kernel_rush_kawk_b200 import Engine

    name = "tiny_b"
    engine = Engine(folders[name], dtype=dtype, max_tokens=64 * 9, max_slots=3)
    prompts = prompts_for(name, [70, 3, 40, 129, 1, 64, 17], seed=34)
    outs = engine.generate_all(prompts, 6)
    assert [len(o) for o in outs] == [6] * 7
    assert engine.cache.live == 0
    engine.cache.check()
    cfg, w = plain.read_folder(folders[name])
    for i, (p, o) in enumerate(zip(prompts, outs)):
        seq = list(p)
        for t, tok in enumerate(o):
            assert_greedy_token(cfg, w, seq, tok, dtype, windows_of(name), f"request {i} step {t}")
            seq.append(tok)
    # the same requests one by one give the same tokens (a batch's company and its slots change nothing)
    if dtype == "float32":
        for i in (0, 3, 6):
            assert engine.generate_all([prompts[i]], 6)[0] == outs[i]


@pytest.mark.parametrize("sizes", ["qwen3_8b", "qwen3_14b"])
def test_the_larger_workloads_at_two_layers(tmp_path, sizes):
    """The 8B layer sizes (hidden 4096, intermediate 12288, untied head, greedy) and the 14B ones (hidden
    5120, 40 query heads in groups of five, intermediate 17408, temperature 0.7) with two layers and a
    smaller vocabulary: an unequal batch through ``Engine.generate``. Greedy tokens are checked against the
    plain implementation; sampled tokens against the plain sampler's draw from the engine's own logits."""
    from kernel_rush_kawk_b200 import Engine, Qwen3Config, StepEntry, write_model_folder

    base = Qwen3Config.preset(sizes).to_dict()
    cfg_ = Qwen3Config.from_dict({**base, "num_hidden_layers": 2, "vocab_size": 8192})
    scale = {f"model.layers.{i}.self_attn.{n}_norm.weight": 1.5 for i in range(2) for n in ("q", "k")}
    folder = write_model_folder(tmp_path / sizes, cfg_, 91, std=0.02, gain_std=0.05, scale=scale, device="cuda")
    g = torch.Generator().manual_seed(35)
    lengths = [300, 97, 512, 130] if sizes == "qwen3_8b" else [260, 64, 333, 129, 40, 2]
    prompts = [torch.randint(0, 8192, (n,), generator=g).tolist() for n in lengths]
    temperature = 0.0 if sizes == "qwen3_8b" else 0.7
    steps_n = 6
    engine = Engine(folder, dtype="bfloat16", max_slots=8)
    steps = list(engine.generate(prompts, steps_n, temperature=temperature, seed=5))
    assert len(steps) == steps_n and engine.cache.live == 0
    engine.ops.check()
    cfg, w = plain.read_folder(folder)
    if temperature == 0.0:
        for i in (1, 3):  # two of the requests, every step
            seq = list(prompts[i])
            for t in range(steps_n):
                assert_greedy_token(cfg, w, seq, steps[t][i], "bfloat16", None, f"{sizes} request {i} step {t}")
                seq.append(steps[t][i])
    else:
        # teacher-forced: the engine's logits for the sequences it generated, then the plain sampler's draws
        engine.open_cache(64 * 64, 8)
        slots = [engine.cache.alloc() for _ in prompts]
        logits = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).cpu()
        for t in range(steps_n):
            for i in range(len(prompts)):
                assert steps[t][i] == plain.sample_temperature(logits[i], temperature, 5, i, t), (sizes, i, t)
            if t + 1 < steps_n:
                logits = engine.step([StepEntry(s, [steps[t][i]], [0]) for i, s in enumerate(slots)]).cpu()
        ref = plain.forward_logits(cfg, w, prompts[4] + [s[4] for s in steps[:-1]], torch.float32, torch.bfloat16)[-1]
        assert_close(logits[4][None], ref[None], "bfloat16", f"{sizes}: logits behind the last draw of request 4")
        for s in slots:
            engine.cache.free(s)
