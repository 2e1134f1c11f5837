"""The engine's step, cache and generation logic on the CPU, with the kernels replaced
by their plain torch restatement (tests/torch_ops.py). The product has no CPU path;
this checks everything around the kernels where no GPU is at hand."""

import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY, assert_close, plain_logits, prompts_for
from torch_ops import TorchOps


def cpu_engine(folders, name, **kw):
    from kernel_rush_kawk_b200 import Engine

    args = dict(dtype="float32", device="cpu", ops=TorchOps(torch.float32), max_tokens=2048, max_slots=6,
                use_cuda_graphs=False)
    args.update(kw)
    return Engine(folders[name], **args)


def test_the_product_refuses_to_run_without_cuda(folders):
    from kernel_rush_kawk_b200 import Engine

    with pytest.raises(RuntimeError, match="CUDA"):
        Engine(folders["tiny_a"], device="cpu")


@pytest.mark.parametrize("name", TINY)
def test_whole_pieces_and_single_tokens_agree_with_plain(folders, name):
    from kernel_rush_kawk_b200 import StepEntry

    engine = cpu_engine(folders, name)
    seqs = prompts_for(name, [70, 9, 131], seed=21)
    refs = [plain_logits(folders[name], name, s, "float32") for s in seqs]
    slots = [engine.cache.alloc() for _ in seqs]
    cuts = [(30, 60), (1, 5), (64, 128)]
    got = [[] for _ in seqs]
    out = engine.step([StepEntry(sl, s[:c[0]], list(range(c[0]))) for sl, s, c in zip(slots, seqs, cuts)])
    r = 0
    for i, c in enumerate(cuts):
        got[i].append(out[r:r + c[0]]); r += c[0]
    out = engine.step([StepEntry(sl, s[c[0]:c[1]], list(range(c[1] - c[0]))) for sl, s, c in zip(slots, seqs, cuts)])
    r = 0
    for i, c in enumerate(cuts):
        got[i].append(out[r:r + c[1] - c[0]]); r += c[1] - c[0]
    fed = [c[1] for c in cuts]
    while any(f < len(s) for f, s in zip(fed, seqs)):
        live = [i for i in range(len(seqs)) if fed[i] < len(seqs[i])]
        out = engine.step([StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live])
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1]); fed[i] += 1
    for i, ref in enumerate(refs):
        assert_close(torch.cat(got[i]), ref, "float32", f"{name} request {i}")
    for s in slots:
        engine.cache.free(s)
    engine.cache.check()


def test_a_step_too_large_for_one_pass_is_cut(folders):
    from kernel_rush_kawk_b200 import StepEntry

    name = "tiny_w"  # has window layers: the per-sequence piece is bounded by the ring
    engine = cpu_engine(folders, name, max_step_rows=48, step_tokens=40)
    seqs = prompts_for(name, [100, 30], seed=22)
    slots = [engine.cache.alloc() for _ in seqs]
    before = engine.stepper.passes
    out = engine.step([StepEntry(sl, s, [len(s) - 1, 0]) for sl, s in zip(slots, seqs)])
    assert engine.stepper.passes - before >= 3
    want = torch.stack([plain_logits(folders[name], name, seqs[0], "float32")[-1],
                        plain_logits(folders[name], name, seqs[0], "float32")[0],
                        plain_logits(folders[name], name, seqs[1], "float32")[-1],
                        plain_logits(folders[name], name, seqs[1], "float32")[0]])
    assert_close(out, want, "float32", "cut step, order of wanted places")


def test_step_refuses_bad_input(folders):
    from kernel_rush_kawk_b200 import StepEntry

    engine = cpu_engine(folders, "tiny_a")
    slot = engine.cache.alloc()
    for entry, message in ((StepEntry(slot, [256], [0]), "vocabulary"), (StepEntry(slot, [-1], [0]), "vocabulary"),
                           (StepEntry(slot, [], []), "no tokens"), (StepEntry(slot, [1], [1]), "wanted place"),
                           (StepEntry(3, [1], [0]), "not held")):
        with pytest.raises(ValueError, match=message):
            engine.step([entry])
    with pytest.raises(ValueError, match="twice"):
        engine.step([StepEntry(slot, [1], [0]), StepEntry(slot, [2], [0])])
    assert engine.step([]).shape == (0, 256)
    assert engine.cache.length[slot] == 0  # nothing was consumed


def test_generation_on_the_cpu_stand_in(folders):
    name = "tiny_b"
    engine = cpu_engine(folders, name, max_tokens=None)
    prompts = prompts_for(name, [1, 7, 13], seed=23)
    steps = list(engine.generate(prompts, 5))
    cfg, w = plain.read_folder(folders[name])
    for i, p in enumerate(prompts):
        assert [s[i] for s in steps] == plain.generate_greedy(cfg, w, p, 5)
    with pytest.raises(ValueError, match="context"):
        list(engine.generate([[1] * 9000], 4))
