"""The Qwen3-4B layer sizes (hidden 2560, 32 query / 8 kv heads of 128, intermediate 9728,
vocabulary 151,936, tied head, theta 5e6) with two layers and random weights: the sizes at
which the serving kernels really run (tcgen05 attention and logits GEMM, 4- and 8-warp decode
GEMVs, cluster-merged decode attention), against the plain implementation, in 32-bit and in
bfloat16, whole and token by token, alone and in an unequal batch."""

import pytest
import torch

import plain_qwen3 as plain
from helpers import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def big_folder(tmp_path_factory):
    from kernel_rush_kawk_b200 import Qwen3Config, write_model_folder

    base = Qwen3Config.preset("qwen3_4b").to_dict()
    cfg = Qwen3Config.from_dict({**base, "num_hidden_layers": 2})
    scale = {f"model.layers.{i}.self_attn.{n}_norm.weight": 1.5 for i in range(2) for n in ("q", "k")}
    return write_model_folder(tmp_path_factory.mktemp("big") / "m", cfg, 77, std=0.02, gain_std=0.05, scale=scale)


@pytest.fixture(scope="module")
def sequences(big_folder):
    g = torch.Generator().manual_seed(5)
    return [torch.randint(0, 151936, (n,), generator=g).tolist() for n in (150, 40, 9)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_four_b_layer_sizes_against_plain(big_folder, sequences, dtype):
    from kernel_rush_kawk_b200 import Engine, StepEntry

    cfg, w = plain.read_folder(big_folder)
    rounding = None if dtype == "float32" else torch.bfloat16
    wide = torch.float64 if dtype == "float32" else torch.float32
    refs = [plain.forward_logits(cfg, w, s, wide, rounding).float() for s in sequences]
    engine = Engine(big_folder, dtype=dtype, max_tokens=1024, max_slots=4)
    cache = engine.cache
    # (1) the longest request whole: 150 tokens x 4 group members = tiles of the tcgen05 kernel in bfloat16
    slot = cache.alloc()
    out = engine.step([StepEntry(slot, sequences[0], list(range(len(sequences[0]))))])
    cache.free(slot)
    assert_close(out, refs[0], dtype, f"4B sizes, whole, {dtype}")
    # (2) an unequal batch: prompts, then one token each until every sequence is used up
    cuts = [130, 20, 1]
    slots = [cache.alloc() for _ in sequences]
    got = [[] for _ in sequences]
    out = engine.step([StepEntry(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, sequences, cuts)])
    row = 0
    for i, c in enumerate(cuts):
        got[i].append(out[row:row + c].float().cpu())
        row += c
    fed = list(cuts)
    while any(f < len(s) for f, s in zip(fed, sequences)):
        live = [i for i in range(3) if fed[i] < len(sequences[i])]
        out = engine.step([StepEntry(slots[i], [sequences[i][fed[i]]], [0]) for i in live]).float().cpu()
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1])
            fed[i] += 1
    for i, ref in enumerate(refs):
        assert_close(torch.cat(got[i]), ref, dtype, f"4B sizes, batch, request {i}, {dtype}")
    for s in slots:
        cache.free(s)
    cache.check()
    engine.ops.check()


def test_fourteen_b_layer_sizes_against_plain(tmp_path):
    """The Qwen3-14B layer sizes (hidden 5120, 40 query / 8 kv heads: groups of five, intermediate 17408,
    untied head, theta 1e6) with one layer and a smaller vocabulary, in bfloat16: other tile counts and
    a group size that does not divide the 128-row query tiles, whole and token by token in a batch."""
    from kernel_rush_kawk_b200 import Engine, Qwen3Config, StepEntry, write_model_folder

    base = Qwen3Config.preset("qwen3_14b").to_dict()
    cfg14 = Qwen3Config.from_dict({**base, "num_hidden_layers": 1, "vocab_size": 32000})
    scale = {f"model.layers.0.self_attn.{n}_norm.weight": 1.5 for n in ("q", "k")}
    folder = write_model_folder(tmp_path / "m14", cfg14, 78, std=0.02, gain_std=0.05, scale=scale)
    g = torch.Generator().manual_seed(6)
    seqs = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (140, 35)]
    cfg, w = plain.read_folder(folder)
    refs = [plain.forward_logits(cfg, w, s, torch.float32, torch.bfloat16).float() for s in seqs]
    engine = Engine(folder, dtype="bfloat16", max_tokens=1024, max_slots=4)
    cache = engine.cache
    slot = cache.alloc()
    out = engine.step([StepEntry(slot, seqs[0], list(range(len(seqs[0]))))])
    cache.free(slot)
    assert_close(out, refs[0], "bfloat16", "14B sizes, whole")
    cuts = [128, 30]
    slots = [cache.alloc() for _ in seqs]
    got = [[] for _ in seqs]
    out = engine.step([StepEntry(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cuts)])
    row = 0
    for i, c in enumerate(cuts):
        got[i].append(out[row:row + c].float().cpu())
        row += c
    fed = list(cuts)
    while any(f < len(s) for f, s in zip(fed, seqs)):
        live = [i for i in range(2) if fed[i] < len(seqs[i])]
        out = engine.step([StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live]).float().cpu()
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1])
            fed[i] += 1
    for i, ref in enumerate(refs):
        assert_close(torch.cat(got[i]), ref, "bfloat16", f"14B sizes, batch, request {i}")
    for s in slots:
        cache.free(s)
    cache.check()
    engine.ops.check()


def test_device_fed_steps_at_the_four_b_sizes(big_folder, sequences):
    """The benchmark's way of stepping (tokens fed on the device, captured graph) against the generation
    loop at the 4B layer sizes: the same greedy tokens."""
    from kernel_rush_kawk_b200 import Engine, StepEntry

    engine = Engine(big_folder, dtype="bfloat16", max_tokens=2048, max_slots=4)
    prompts = [s[:n] for s, n in zip(sequences, (140, 40, 9))]
    by_loop = list(engine.generate(prompts, 8))
    cache = engine.cache
    slots = [cache.alloc() for _ in prompts]
    logits = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    first = logits.argmax(dim=-1).tolist()
    assert first == by_loop[0]
    rest = engine.stepper.decode_on_device(slots, first, 7, first_step=1).tolist()
    assert rest == by_loop[1:]
    for s in slots:
        cache.free(s)
    cache.check()
    engine.ops.check()


def test_many_sequences_take_the_tma_fed_attention(big_folder):
    """28 sequences x 8 kv heads are more (sequence, kv head) items than the cluster kernel is used for: the
    single-token steps of this batch run the TMA-fed attention kernel inside the captured step. Lengths
    straddle page boundaries (one sequence starts its third page during the steps); logits of several
    requests against the plain implementation at every step."""
    from kernel_rush_kawk_b200 import Engine, StepEntry

    cfg, w = plain.read_folder(big_folder)
    g = torch.Generator().manual_seed(8)
    lengths = [5, 64, 63, 130, 127, 1, 70, 33] + [9 + 3 * i for i in range(20)]
    steps = 4
    seqs = [torch.randint(0, 151936, (n + steps,), generator=g).tolist() for n in lengths]
    engine = Engine(big_folder, dtype="bfloat16", max_tokens=28 * 256, max_slots=28)
    cache = engine.cache
    slots = [cache.alloc() for _ in seqs]
    checked = [1, 2, 3, 4, 5, 27]
    refs = {i: plain.forward_logits(cfg, w, seqs[i], torch.float32, torch.bfloat16).float() for i in checked}
    for i0 in range(0, 28, 7):  # prompts in four steps of seven requests
        part = list(range(i0, i0 + 7))
        engine.step([StepEntry(slots[i], seqs[i][:lengths[i]], []) for i in part])
    for t in range(steps):
        out = engine.step([StepEntry(slots[i], [seqs[i][lengths[i] + t]], [0]) for i in range(28)]).float().cpu()
        for i in checked:
            assert_close(out[i][None], refs[i][lengths[i] + t][None], "bfloat16", f"request {i} ({lengths[i]} tokens), decode step {t}")
    assert engine.ops.use_tma_decode_attention
    for s in slots:
        cache.free(s)
    cache.check()
    engine.ops.check()
