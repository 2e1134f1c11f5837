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


def test_attention_part_with_a_rotation_of_part_of_the_head_on_the_stand_in():
    """Tables narrower than half the head rotate the first `2 * columns` elements of a head only (pairs
    (i, i + rot/2); the norm is over the whole head). The attention part passes them through as they are;
    here with the kernels' torch restatement, whole and in pieces, against the computation written out."""
    from kernel_rush_kawk_b200.cache import SequenceCache
    from kernel_rush_kawk_b200.engine.model import Runtime
    from kernel_rush_kawk_b200.engine.step import BatchMeta, StepContext
    from kernel_rush_kawk_b200.parts import GQAttention, RotaryTable

    dtype = torch.float32
    rt = Runtime(torch.device("cpu"), dtype, TorchOps(dtype))
    H, HQ, HKV, D, ROT, T, EPS = 40, 4, 2, 24, 8, 70, 1e-5
    g = torch.Generator().manual_seed(5)
    rnd = lambda *shape: torch.randn(shape, generator=g)
    part = GQAttention({"hidden": H, "heads": HQ, "kv_heads": HKV, "head_dim": D, "eps": EPS})
    rope = RotaryTable({"theta": 1e4, "dim": ROT, "positions": 128})
    rope.bind({}, rt)
    part.set_position(rope)
    w = {"q_proj": 0.1 * rnd(HQ * D, H), "k_proj": 0.1 * rnd(HKV * D, H), "v_proj": 0.1 * rnd(HKV * D, H),
         "o_proj": 0.1 * rnd(H, HQ * D), "q_norm": 1.5 + 0.1 * rnd(D), "k_norm": 0.8 + 0.1 * rnd(D)}
    part.bind(dict(w), rt)
    h = rnd(T, H)
    pc, ps = plain.rope_tables(ROT, 1e4, T)

    def norm_rotate(x, gain):
        y = gain * (x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + EPS))
        y1, y2, rest = y[..., :ROT // 2], y[..., ROT // 2:ROT], y[..., ROT:]
        c, s = pc[:, None, :], ps[:, None, :]
        return torch.cat([y1 * c - y2 * s, y2 * c + y1 * s, rest], dim=-1)

    q = norm_rotate(plain.linear(h, w["q_proj"]).view(T, HQ, D), w["q_norm"])
    k = norm_rotate(plain.linear(h, w["k_proj"]).view(T, HKV, D), w["k_norm"])
    v = plain.linear(h, w["v_proj"]).view(T, HKV, D)
    want = plain.linear(plain.causal_gqa_attention(q, k, v), w["o_proj"])

    for pieces in ([T], [33, 30, 1, 1, 1, 1, 1, 1, 1]):
        cache = SequenceCache([part.cache_need()], 128, 2, 128, rt.device, dtype, step_tokens=64)
        slot = cache.alloc()
        got, start = [], 0
        for n in pieces:
            cache.reserve(slot, start + n)
            cache.sync()
            meta = BatchMeta(n, 1, 0, rt.device)
            meta.fill([slot], [start], [[0] * n], [])
            got.append(part.forward(StepContext(rt.ops, meta, cache), h[start:start + n], cache.view(0)))
            cache.advance(slot, n)
            start += n
        assert_close(torch.cat(got), want, "float32", f"partial rotation on the stand-in, pieces {pieces}")
