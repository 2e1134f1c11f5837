"""Each part alone against the plain implementation, and the generality of the
assembly: a toy mixer with state of its own, a layer that runs twice, a run that
reads another run's cache; a feed-forward that routes rows to experts and a learned
position table -- registered, built and stepped from this file without a change to
the package."""

import math
from dataclasses import dataclass
from types import SimpleNamespace

import pytest
import torch

import plain_qwen3 as plain
from helpers import assert_close

pytestmark = pytest.mark.gpu

DTYPES = (torch.float32, torch.bfloat16)
NAME = {torch.float32: "float32", torch.bfloat16: "bfloat16"}


def runtime(dtype):
    from kernel_rush_kawk_b200.csrc import load_kernels
    from kernel_rush_kawk_b200.engine.model import Runtime

    return Runtime(torch.device("cuda:0"), dtype, load_kernels(()))


def rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


def context(rt, slots, starts, q_lens, cache):
    from kernel_rush_kawk_b200.engine.step import BatchMeta, StepContext

    rows = sum(q_lens)
    meta = BatchMeta(rows, len(slots), 0, rt.device)
    meta.fill(slots, starts, [[0] * n for n in q_lens], [])
    return StepContext(rt.ops, meta, cache)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part_folds_the_pending_branch(dtype):
    from kernel_rush_kawk_b200.parts import RMSNorm, Stream

    rt = runtime(dtype)
    rounding = None if dtype == torch.float32 else torch.bfloat16
    part = RMSNorm({"size": 100, "eps": 1e-5})
    gain = (1 + 0.1 * rand((100,), 1)).to(dtype)
    part.bind({"weight": gain.cuda()}, rt)
    x, b = rand((6, 100), 2, 3.0).to(dtype), rand((6, 100), 3).to(dtype)
    ctx = SimpleNamespace(ops=rt.ops)
    stream = Stream(x.cuda(), b.cuda())
    h = part.forward(ctx, stream).tensor()
    s = plain.residual_add(x.float(), b.float(), rounding)
    assert stream.branch is None and torch.equal(stream.x.float().cpu(), s)
    assert_close(h, plain.rms_norm(s, gain.float(), 1e-5, rounding), NAME[dtype], "norm part", kernel=True)
    alone = part.forward(ctx, Stream(x.cuda())).tensor()
    assert_close(alone, plain.rms_norm(x.float(), gain.float(), 1e-5, rounding), NAME[dtype], "norm part", kernel=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rotary_table_part(dtype):
    from kernel_rush_kawk_b200.parts import RotaryTable

    part = RotaryTable({"theta": 5e5, "dim": 48, "positions": 300})
    part.bind({}, runtime(dtype))
    cos, sin = part.rotary_tables()
    pc, ps = plain.rope_tables(48, 5e5, 300, torch.float32, None if dtype == torch.float32 else torch.bfloat16)
    assert cos.shape == (300, 24) and cos.dtype == dtype
    assert (cos.float().cpu() - pc).abs().max() < (1e-5 if dtype == torch.float32 else 8e-3)
    assert (sin.float().cpu() - ps).abs().max() < (1e-5 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part_alone(dtype, window):
    """hidden 72, 6 heads in 3 groups, head size 16 (6*16 != 72); a whole sequence in one
    step, then the same sequence in two steps."""
    from kernel_rush_kawk_b200.cache import SequenceCache
    from kernel_rush_kawk_b200.parts import GQAttention, RotaryTable

    rt = runtime(dtype)
    rounding = None if dtype == torch.float32 else torch.bfloat16
    H, HQ, HKV, D, T = 72, 6, 3, 16, 90
    part = GQAttention({"hidden": H, "heads": HQ, "kv_heads": HKV, "head_dim": D, "eps": 1e-6, "window": window})
    rope = RotaryTable({"theta": 1e4, "dim": D, "positions": 256})
    rope.bind({}, rt)
    part.set_position(rope)
    w = {"q_proj": rand((HQ * D, H), 1, 0.1), "k_proj": rand((HKV * D, H), 2, 0.1), "v_proj": rand((HKV * D, H), 3, 0.1),
         "o_proj": rand((H, HQ * D), 4, 0.1), "q_norm": 1.5 + 0.1 * rand((D,), 5), "k_norm": 1.5 + 0.1 * rand((D,), 6)}
    w = {k: v.to(dtype) for k, v in w.items()}
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    part.bind({k: v.cuda() for k, v in w.items()}, rt)
    h = rand((T, H), 7).to(dtype)
    cfg = plain.PlainConfig(H, 0, 1, HQ, HKV, D, 0, 1e-6, 1e4, False)
    names = {f"L.self_attn.{k}.weight": v.float() for k, v in w.items()}
    pc, ps = plain.rope_tables(D, 1e4, T, torch.float32, rounding)
    want = plain.attention_block(h.float(), names, "L.", cfg, pc, ps, window, rounding)
    for pieces in ([T], [50, 40]):
        cache = SequenceCache([part.cache_need()], 256, 2, 256, rt.device, dtype, step_tokens=64)
        slot = cache.alloc()
        got, start = [], 0
        for n in pieces:
            cache.reserve(slot, start + n)
            cache.sync()
            ctx = context(rt, [slot], [start], [n], cache)
            got.append(part.forward(ctx, h[start:start + n].cuda(), cache.view(0)))
            cache.advance(slot, n)
            start += n
        assert_close(torch.cat(got), want, NAME[dtype], f"attention part, pieces {pieces}", kernel=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_part_with_a_rotation_of_part_of_the_head(dtype):
    """Another position encoding for the same mixer: tables that cover the first 24 of a head's 48 elements.
    The attention part takes them as they are (the rotated width is the tables' own); whole, in two pieces,
    and with the last tokens one by one, against a plain whole-sequence computation written out here."""
    from kernel_rush_kawk_b200.cache import SequenceCache
    from kernel_rush_kawk_b200.parts import GQAttention, RotaryTable

    rt = runtime(dtype)
    rounding = None if dtype == torch.float32 else torch.bfloat16
    rnd = (lambda x: x) if rounding is None else (lambda x: x.to(rounding).float())
    H, HQ, HKV, D, ROT, T, EPS = 80, 4, 2, 48, 24, 75, 1e-5
    part = GQAttention({"hidden": H, "heads": HQ, "kv_heads": HKV, "head_dim": D, "eps": EPS})
    rope = RotaryTable({"theta": 1e4, "dim": ROT, "positions": 128})
    rope.bind({}, rt)
    part.set_position(rope)
    w = {"q_proj": rand((HQ * D, H), 1, 0.1), "k_proj": rand((HKV * D, H), 2, 0.1), "v_proj": rand((HKV * D, H), 3, 0.1),
         "o_proj": rand((H, HQ * D), 4, 0.1), "q_norm": 1.5 + 0.1 * rand((D,), 5), "k_norm": 0.8 + 0.1 * rand((D,), 6)}
    w = {k: v.to(dtype) for k, v in w.items()}
    part.bind({k: v.cuda() for k, v in w.items()}, rt)
    h = rand((T, H), 7).to(dtype)

    # the plain computation: per-head norm over all 48 elements, pairs (i, i + 12) of the first 24 rotated
    pc, ps = plain.rope_tables(ROT, 1e4, T, torch.float32, rounding)
    f = {k: v.float() for k, v in w.items()}

    def norm_rotate(x, gain):
        r = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + EPS)
        y = rnd(gain * rnd(x * r))
        y1, y2, rest = y[..., :ROT // 2], y[..., ROT // 2:ROT], y[..., ROT:]
        c, s_ = pc[:, None, :], ps[:, None, :]
        return torch.cat([rnd(rnd(y1 * c) + rnd(-y2 * s_)), rnd(rnd(y2 * c) + rnd(y1 * s_)), rest], dim=-1)

    q = norm_rotate(plain.linear(h.float(), f["q_proj"], rounding).view(T, HQ, D), f["q_norm"])
    k = norm_rotate(plain.linear(h.float(), f["k_proj"], rounding).view(T, HKV, D), f["k_norm"])
    v = plain.linear(h.float(), f["v_proj"], rounding).view(T, HKV, D)
    want = plain.linear(plain.causal_gqa_attention(q, k, v, None, rounding), f["o_proj"], rounding)

    for pieces in ([T], [40, 35], [70, 1, 1, 1, 1, 1]):
        cache = SequenceCache([part.cache_need()], 128, 2, 128, rt.device, dtype, step_tokens=64)
        slot = cache.alloc()
        got, start = [], 0
        for n in pieces:
            cache.reserve(slot, start + n)
            cache.sync()
            ctx = context(rt, [slot], [start], [n], cache)
            got.append(part.forward(ctx, h[start:start + n].cuda(), cache.view(0)))
            cache.advance(slot, n)
            start += n
        assert_close(torch.cat(got), want, NAME[dtype], f"attention part with a partial rotation, pieces {pieces}", kernel=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part_and_block_alone(dtype):
    from kernel_rush_kawk_b200.cache import SequenceCache
    from kernel_rush_kawk_b200.parts import GQAttention, PreNormBlock, RMSNorm, RotaryTable, Stream, SwiGLU

    rt = runtime(dtype)
    rounding = None if dtype == torch.float32 else torch.bfloat16
    H, I, HQ, HKV, D, T = 80, 208, 5, 1, 16, 40
    ffn = SwiGLU({"hidden": H, "intermediate": I})
    wf = {"gate_proj": rand((I, H), 1, 0.1).to(dtype), "up_proj": rand((I, H), 2, 0.1).to(dtype),
          "down_proj": rand((H, I), 3, 0.1).to(dtype)}
    ffn.bind({k: v.cuda() for k, v in wf.items()}, rt)
    h = rand((T, H), 4).to(dtype)
    ctx = SimpleNamespace(ops=rt.ops)
    want = plain.swiglu_mlp(h.float(), wf["gate_proj"].float(), wf["up_proj"].float(), wf["down_proj"].float(), rounding)
    assert_close(ffn.forward(ctx, h.cuda()), want, NAME[dtype], "swiglu part", kernel=True)

    attn = GQAttention({"hidden": H, "heads": HQ, "kv_heads": HKV, "head_dim": D, "eps": 1e-5})
    rope = RotaryTable({"theta": 1e6, "dim": D, "positions": 128})
    rope.bind({}, rt)
    attn.set_position(rope)
    wa = {"q_proj": rand((HQ * D, H), 5, 0.1), "k_proj": rand((HKV * D, H), 6, 0.1), "v_proj": rand((HKV * D, H), 7, 0.1),
          "o_proj": rand((H, HQ * D), 8, 0.1), "q_norm": 1 + 0.1 * rand((D,), 9), "k_norm": 1 + 0.1 * rand((D,), 10)}
    wa = {k: v.to(dtype) for k, v in wa.items()}
    attn.bind({k: v.cuda() for k, v in wa.items()}, rt)
    n1, n2 = RMSNorm({"size": H, "eps": 1e-5}), RMSNorm({"size": H, "eps": 1e-5})
    g1, g2 = (1 + 0.1 * rand((H,), 11)).to(dtype), (1 + 0.1 * rand((H,), 12)).to(dtype)
    n1.bind({"weight": g1.cuda()}, rt)
    n2.bind({"weight": g2.cuda()}, rt)
    block = PreNormBlock(n1, attn, n2, ffn)
    cache = SequenceCache([attn.cache_need()], 128, 1, 128, rt.device, dtype)
    slot = cache.alloc()
    cache.reserve(slot, T)
    cache.sync()
    x = rand((T, H), 13).to(dtype)
    stream = block.forward(context(rt, [slot], [0], [T], cache), Stream(x.cuda()), cache.view(0))
    got = plain.residual_add(stream.x.float().cpu(), stream.branch.float().cpu(), rounding)
    cfg = plain.PlainConfig(H, I, 1, HQ, HKV, D, 0, 1e-5, 1e6, False)
    names = {f"model.layers.0.self_attn.{k}.weight": v.float() for k, v in wa.items()}
    names.update({f"model.layers.0.mlp.{k}.weight": v.float() for k, v in wf.items()})
    names["model.layers.0.input_layernorm.weight"] = g1.float()
    names["model.layers.0.post_attention_layernorm.weight"] = g2.float()
    pc, ps = plain.rope_tables(D, 1e6, T, torch.float32, rounding)
    want = plain.decoder_layer(x.float(), names, 0, cfg, pc, ps, None, rounding)
    assert_close(got, want, NAME[dtype], "block alone", kernel=True)


# ---------------------------------------------------------------------------------
# A toy architecture defined here: layer 0 attention, layer 1 a mixer with state of its
# own, layer 2 attention that reads run 1's... and a schedule that names layer 0 twice.
# ---------------------------------------------------------------------------------
def register_toy():
    from kernel_rush_kawk_b200.config import ModelConfig, register_architecture
    from kernel_rush_kawk_b200.parts import (Embedding, LayerSpec, Mixer, ModelPlan, PartSpec, ScheduleEntry, StateNeed,
                                             TensorSpec, register_embedding, register_mixer)

    class ScaledEmbedding(Embedding):
        """x0[r] = round(table[ids[r]] * scale): an embedding kind of the test's own."""

        def __init__(self, params):
            super().__init__(params)
            self.vocab, self.hidden, self.scale = int(params["vocab"]), int(params["hidden"]), float(params["scale"])

        def tensor_specs(self):
            return {"table": TensorSpec((self.vocab, self.hidden), "table")}

        def bind(self, tensors, runtime):
            self.table = tensors["table"]

        def forward(self, ctx):
            x = ctx.ops.embed(self.table, ctx.batch.tokens, ctx.batch.n_rows)
            return (x.float() * self.scale).to(x.dtype)

    register_embedding("test_scaled_embedding", ScaledEmbedding)

    class DecayMixer(Mixer):
        """s_t = decay * s_{t-1} + h_t (state [hidden] per sequence, float32); out_t = s_t W^T."""

        def __init__(self, params):
            super().__init__(params)
            self.hidden, self.decay = int(params["hidden"]), float(params["decay"])
            # A step of several tokens scans them in order and reads the step's lengths on the host. With
            # "on_device" a single-token step touches device arrays only, so it can be captured and queued
            # ahead of the host; without it the part declares that its steps cannot be.
            self.on_device = bool(params.get("on_device", False))
            self.graph_safe = self.on_device

        def tensor_specs(self):
            return {"mix": TensorSpec((self.hidden, self.hidden))}

        def cache_need(self):
            return StateNeed((self.hidden,), "float32")

        def bind(self, tensors, runtime):
            self.w = tensors["mix"]

        def forward(self, ctx, h, cache):
            rows = h.tensor().float()
            if self.on_device and ctx.batch.is_decode:  # one token each: row r belongs to sequence r
                slots = ctx.batch.seq_slot.long()
                s = cache.state[slots] * self.decay + rows
                cache.state.index_copy_(0, slots, s)
                return (s.to(self.w.dtype).float() @ self.w.float().t()).to(self.w.dtype)
            out = torch.empty_like(rows)
            r = 0
            for slot, n in zip(ctx.batch.slots, ctx.batch.q_lens):
                s = cache.state[slot]
                for t in range(n):
                    s = self.decay * s + rows[r + t]
                    out[r + t] = s
                cache.state[slot] = s
                r += n
            return (out.to(self.w.dtype).float() @ self.w.float().t()).to(self.w.dtype)

    register_mixer("test_decay", DecayMixer)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        hidden: int = 48
        vocab: int = 97
        state_on_device: bool = False
        architecture = "ToyDecoderForTests"

        @classmethod
        def from_dict(cls, raw):
            return cls(raw.get("hidden", 48), raw.get("vocab", 97), bool(raw.get("state_on_device", False)))

        def to_dict(self):
            return {"architectures": [self.architecture], "hidden": self.hidden, "vocab": self.vocab,
                    "state_on_device": self.state_on_device}

        @classmethod
        def preset_names(cls):
            return ["toy_small"]

        @classmethod
        def preset(cls, name):
            assert name == "toy_small"
            return cls(48, 61)

    def plan(cfg):
        H = cfg.hidden
        norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": 1e-5}, {"weight": name})
        ffn = lambda i: PartSpec("swiglu", {"hidden": H, "intermediate": 64},
                                 {k: f"l{i}.ffn.{k}" for k in ("gate_proj", "up_proj", "down_proj")})
        attn = lambda i, own: PartSpec(
            "gqa_attention", {"hidden": H, "heads": 4, "kv_heads": 2, "head_dim": 16, "eps": 1e-5, "own_cache": own},
            {k: f"l{i}.attn.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")})
        layers = [
            LayerSpec("prenorm", norm("l0.n1"), attn(0, True), norm("l0.n2"), ffn(0)),
            LayerSpec("prenorm", norm("l1.n1"), PartSpec("test_decay", {"hidden": H, "decay": 0.5,
                                                                      "on_device": cfg.state_on_device}, {"mix": "l1.mix"}),
                      norm("l1.n2"), ffn(1)),
            LayerSpec("prenorm", norm("l2.n1"), attn(2, False), norm("l2.n2"), ffn(2)),
        ]
        # layer 0 runs twice (two caches), the state mixer in between, then a layer with
        # queries only that reads the keys and values of the second run of layer 0
        schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(2, cache_from=2)]
        return ModelPlan("ToyDecoderForTests", H, cfg.vocab,
                         PartSpec("test_scaled_embedding", {"vocab": cfg.vocab, "hidden": H, "scale": 3.0}, {"table": "embed"}),
                         PartSpec("rope", {"theta": 1e4, "dim": 16}), tuple(layers), tuple(schedule), norm("final"),
                         PartSpec("output_head", {"vocab": cfg.vocab, "hidden": H}, {"weight": "embed"}), 512)

    register_architecture("ToyDecoderForTests", ToyConfig, plan)
    return ToyConfig()


def toy_plain(w, ids, rounding):
    """The toy model, whole sequence, from the plain implementation's functions."""
    rt = (lambda t: t) if rounding is None else (lambda t: t.to(rounding).float())
    T = len(ids)
    cos, sin = plain.rope_tables(16, 1e4, T, torch.float32, rounding)
    cfg = SimpleNamespace(heads=4, kv_heads=2, head_dim=16, eps=1e-5)
    x = rt(w["embed"][torch.tensor(ids)] * 3.0)

    def attn(h, i, kv=None):
        q = plain.linear(h, w[f"l{i}.attn.q_proj"], rounding).view(T, 4, 16)
        q = plain.head_norm_rope(q, w[f"l{i}.attn.q_norm"], cos, sin, 1e-5, rounding)
        if kv is None:
            k = plain.linear(h, w[f"l{i}.attn.k_proj"], rounding).view(T, 2, 16)
            v = plain.linear(h, w[f"l{i}.attn.v_proj"], rounding).view(T, 2, 16)
            kv = (plain.head_norm_rope(k, w[f"l{i}.attn.k_norm"], cos, sin, 1e-5, rounding), v)
        a = plain.causal_gqa_attention(q, kv[0], kv[1], None, rounding)
        return plain.linear(a, w[f"l{i}.attn.o_proj"], rounding), kv

    def decay(h):
        s, out = torch.zeros(h.shape[1]), []
        for t in range(T):
            s = 0.5 * s + h[t]
            out.append(s)
        return rt(rt(torch.stack(out)) @ w["l1.mix"].t())

    def ffn(x, i):
        h = plain.rms_norm(x, w[f"l{i}.n2"], 1e-5, rounding)
        d = plain.swiglu_mlp(h, w[f"l{i}.ffn.gate_proj"], w[f"l{i}.ffn.up_proj"], w[f"l{i}.ffn.down_proj"], rounding)
        return plain.residual_add(x, d, rounding)

    kv2 = None
    for run, layer in enumerate((0, 1, 0, 2)):
        h = plain.rms_norm(x, w[f"l{layer}.n1"], 1e-5, rounding)
        if layer == 1:
            branch = decay(h)
        elif layer == 2:
            branch, _ = attn(h, 2, kv2)
        else:
            branch, kv = attn(h, 0)
            if run == 2:
                kv2 = kv
        x = ffn(plain.residual_add(x, branch, rounding), layer)
    return plain.rms_norm(x, w["final"], 1e-5, rounding) @ w["embed"].t()


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_architecture_with_a_state_mixer_a_repeated_layer_and_a_shared_cache(dtype, tmp_path):
    from kernel_rush_kawk_b200 import Engine, StepEntry, write_model_folder
    from safetensors.torch import load_file

    cfg = register_toy()
    folder = write_model_folder(tmp_path / "toy", cfg, 5, std=0.08, gain_std=0.1)
    engine = Engine(folder, dtype=NAME[dtype], max_tokens=1024, max_slots=4)
    assert not engine.model.graph_safe and not engine.stepper.use_graphs
    assert "l2.attn.k_proj" not in load_file(str(folder / "model.safetensors"))  # queries only
    w = {k: v.float() for k, v in load_file(str(folder / "model.safetensors")).items()}
    g = torch.Generator().manual_seed(3)
    seqs = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (70, 9)]
    refs = [toy_plain(w, s, None if dtype == torch.float32 else torch.bfloat16) for s in seqs]
    # whole, then prompt + single tokens in an unequal batch
    for cuts in ([70, 9], [40, 3]):
        slots = [engine.cache.alloc() for _ in seqs]
        got = [[] for _ in seqs]
        out = engine.step([StepEntry(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cuts)])
        got[0].append(out[:cuts[0]]); got[1].append(out[cuts[0]:])
        fed = list(cuts)
        while any(f < len(s) for f, s in zip(fed, seqs)):
            live = [i for i in range(2) if fed[i] < len(seqs[i])]
            out = engine.step([StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live])
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1]); fed[i] += 1
        for i in range(2):
            assert_close(torch.cat(got[i]), refs[i], NAME[dtype], f"toy model, cuts {cuts}, request {i}")
        for s in slots:
            engine.cache.free(s)
    engine.cache.check()
    toks = list(engine.generate([seqs[1]], 3))
    assert len(toks) == 3
    # the architecture's own preset, by name, through the registry: random weights, a few tokens
    from kernel_rush_kawk_b200.config import preset_config
    assert preset_config("toy_small").vocab == 61
    small = Engine.from_random("toy_small", seed=1, std=0.08, dtype=NAME[dtype], max_slots=2)
    assert small.plan.vocab_size == 61 and len(list(small.generate([[1, 2, 3]], 2))) == 2


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_state_mixer_whose_single_token_steps_stay_on_the_device_is_captured_and_runs_ahead(dtype, tmp_path):
    """The same toy architecture with its state mixer's single-token path on device arrays only: the model
    is then safe to capture, its steps replay from a graph and the generation loop queues them ahead of
    the host. Logits equal the plain implementation's, and generation equals that of the engine whose
    steps go through the host one by one."""
    import dataclasses

    from kernel_rush_kawk_b200 import Engine, StepEntry, write_model_folder
    from safetensors.torch import load_file

    cfg = dataclasses.replace(register_toy(), state_on_device=True)
    folder = write_model_folder(tmp_path / "toy_dev", cfg, 5, std=0.08, gain_std=0.1)
    engine = Engine(folder, dtype=NAME[dtype], max_tokens=1024, max_slots=4)
    assert engine.model.graph_safe and engine.stepper.use_graphs
    w = {k: v.float() for k, v in load_file(str(folder / "model.safetensors")).items()}
    g = torch.Generator().manual_seed(3)
    seqs = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (70, 9)]
    refs = [toy_plain(w, s, None if dtype == torch.float32 else torch.bfloat16) for s in seqs]
    cuts = [40, 3]
    slots = [engine.cache.alloc() for _ in seqs]
    got = [[] for _ in seqs]
    out = engine.step([StepEntry(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cuts)])
    got[0].append(out[:cuts[0]]); got[1].append(out[cuts[0]:])
    fed = list(cuts)
    while any(f < len(s) for f, s in zip(fed, seqs)):
        live = [i for i in range(2) if fed[i] < len(seqs[i])]
        out = engine.step([StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live])
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1].clone()); fed[i] += 1
    for i in range(2):
        assert_close(torch.cat(got[i]), refs[i], NAME[dtype], f"toy model with device state, request {i}")
    for s in slots:
        engine.cache.free(s)
    assert engine.stepper._graphs, "single-token steps were captured"
    prompts = [seqs[0][:20], seqs[1]]
    ahead = list(engine.generate(prompts, 9))
    by_host = list(Engine(folder, dtype=NAME[dtype], max_tokens=1024, max_slots=4, use_cuda_graphs=False).generate(prompts, 9))
    assert ahead == by_host
    engine.cache.check()


# ---------------------------------------------------------------------------------
# A second toy architecture defined here: positions learned as a table added to the
# embeddings (no rotation) and a feed-forward that routes every row to one of three
# experts. Neither kind exists in the package.
# ---------------------------------------------------------------------------------
def register_routed_toy():
    from kernel_rush_kawk_b200.config import ModelConfig, register_architecture
    from kernel_rush_kawk_b200.parts import (FeedForward, Head, LayerSpec, ModelPlan, PartSpec, PositionEncoding,
                                             ScheduleEntry, TensorSpec, register_feed_forward, register_head,
                                             register_position)

    class CappedHead(Head):
        """logits = cap * tanh((h W^T) / cap), in 32-bit: an output head of the test's own."""

        def __init__(self, params):
            super().__init__(params)
            self.vocab, self.hidden, self.cap = int(params["vocab"]), int(params["hidden"]), float(params["cap"])

        def tensor_specs(self):
            return {"weight": TensorSpec((self.vocab, self.hidden), "table")}

        def bind(self, tensors, runtime):
            self.weight = tensors["weight"]

        def forward(self, ctx, h):
            return self.cap * torch.tanh(ctx.ops.linear(h, self.weight, out_float32=True) / self.cap)

    register_head("test_capped_head", CappedHead)

    class LearnedPositions(PositionEncoding):
        """x_t += table[position of t]; queries and keys are not rotated."""

        def __init__(self, params):
            super().__init__(params)
            self.rows, self.hidden = int(params["table_rows"]), int(params["hidden"])

        def tensor_specs(self):
            return {"table": TensorSpec((self.rows, self.hidden))}

        def bind(self, tensors, runtime):
            self.table = tensors["table"]

        def on_embeddings(self, ctx, x):
            pos = ctx.batch.row_pos.long()  # a device array: nothing is read on the host
            return (x.float() + self.table[pos].float()).to(x.dtype)

    class RoutedSwiGLU(FeedForward):
        """Router logits and their softmax in 32-bit; every row goes to its best expert (a SwiGLU of its own)
        and comes back scaled by that expert's probability."""

        graph_safe = False  # the rows of each expert are counted on the host

        def __init__(self, params):
            super().__init__(params)
            self.hidden, self.inter, self.experts = int(params["hidden"]), int(params["intermediate"]), int(params["experts"])

        def tensor_specs(self):
            specs = {"router": TensorSpec((self.experts, self.hidden))}
            for e in range(self.experts):
                specs[f"gate_up_{e}"] = TensorSpec((2 * self.inter, self.hidden))
                specs[f"down_{e}"] = TensorSpec((self.hidden, self.inter))
            return specs

        def bind(self, tensors, runtime):
            self.t = tensors

        def forward(self, ctx, h):
            rows = h.tensor()
            logits = rows.float() @ self.t["router"].float().t()
            prob, best = torch.softmax(logits, dim=-1).max(dim=-1)
            out = torch.zeros_like(rows)
            for e in range(self.experts):
                idx = (best == e).nonzero().flatten()
                if idx.numel() == 0:
                    continue
                part = rows.index_select(0, idx).contiguous()
                act = ctx.ops.gate_up_swiglu(part, self.t[f"gate_up_{e}"], self.inter)
                y = ctx.ops.linear(act, self.t[f"down_{e}"])
                out.index_copy_(0, idx, (y.float() * prob[idx, None]).to(rows.dtype))
            return out

    register_position("test_learned_positions", LearnedPositions)
    register_feed_forward("test_routed_swiglu", RoutedSwiGLU)

    @dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        hidden: int = 64
        vocab: int = 113
        architecture = "ToyRoutedForTests"

        @classmethod
        def from_dict(cls, raw):
            return cls(raw.get("hidden", 64), raw.get("vocab", 113))

        def to_dict(self):
            return {"architectures": [self.architecture], "hidden": self.hidden, "vocab": self.vocab}

    def plan(cfg):
        H = cfg.hidden
        norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": 1e-6}, {"weight": name})
        attn = lambda i: PartSpec(
            "gqa_attention", {"hidden": H, "heads": 4, "kv_heads": 1, "head_dim": 32, "eps": 1e-6, "qk_norm": False},
            {k: f"l{i}.attn.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj")})
        names = lambda i: {"router": f"l{i}.moe.router", **{f"gate_up_{e}": f"l{i}.moe.gate_up_{e}" for e in range(3)},
                           **{f"down_{e}": f"l{i}.moe.down_{e}" for e in range(3)}}
        routed = lambda i: PartSpec("test_routed_swiglu", {"hidden": H, "intermediate": 32, "experts": 3}, names(i))
        layers = [LayerSpec("prenorm", norm(f"l{i}.n1"), attn(i), norm(f"l{i}.n2"), routed(i)) for i in range(2)]
        return ModelPlan("ToyRoutedForTests", H, cfg.vocab,
                         PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": H}, {"table": "embed"}),
                         PartSpec("test_learned_positions", {"table_rows": 256, "hidden": H}, {"table": "positions"}),
                         tuple(layers), (ScheduleEntry(0), ScheduleEntry(1)), norm("final"),
                         PartSpec("test_capped_head", {"vocab": cfg.vocab, "hidden": H, "cap": 2.0}, {"weight": "head"}), 256)

    register_architecture("ToyRoutedForTests", RoutedConfig, plan)
    return RoutedConfig()


def routed_plain(w, ids, rounding):
    """The routed toy model, whole sequence; also returns every row's routing margin per layer."""
    rt = (lambda t: t) if rounding is None else (lambda t: t.to(rounding).float())
    T = len(ids)
    x = rt(w["embed"][torch.tensor(ids)] + w["positions"][:T])
    margins = []
    for i in range(2):
        h = plain.rms_norm(x, w[f"l{i}.n1"], 1e-6, rounding)
        q = plain.linear(h, w[f"l{i}.attn.q_proj"], rounding).view(T, 4, 32)
        k = plain.linear(h, w[f"l{i}.attn.k_proj"], rounding).view(T, 1, 32)
        v = plain.linear(h, w[f"l{i}.attn.v_proj"], rounding).view(T, 1, 32)
        a = plain.causal_gqa_attention(q, k, v, None, rounding)
        x = plain.residual_add(x, plain.linear(a, w[f"l{i}.attn.o_proj"], rounding), rounding)
        h = plain.rms_norm(x, w[f"l{i}.n2"], 1e-6, rounding)
        logits = h @ w[f"l{i}.moe.router"].t()
        prob = torch.softmax(logits, dim=-1)
        top2 = logits.topk(2, dim=-1).values
        margins.append(top2[:, 0] - top2[:, 1])
        best = prob.argmax(dim=-1)
        out = torch.zeros_like(h)
        for e in range(3):
            rows = best == e
            gu = w[f"l{i}.moe.gate_up_{e}"]
            y = plain.swiglu_mlp(h[rows], gu[:32], gu[32:], w[f"l{i}.moe.down_{e}"], rounding)
            out[rows] = rt(y * prob[rows, e][:, None])
        x = plain.residual_add(x, out, rounding)
    logits = 2.0 * torch.tanh((plain.rms_norm(x, w["final"], 1e-6, rounding) @ w["head"].t()) / 2.0)
    return logits, torch.stack(margins).min(dim=0).values


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_architecture_with_learned_positions_and_a_routed_feed_forward(dtype, tmp_path):
    from kernel_rush_kawk_b200 import Engine, StepEntry, write_model_folder
    from safetensors.torch import load_file

    cfg = register_routed_toy()
    scale = {f"l{i}.moe.router": 12.0 for i in range(2)}  # clear routing decisions
    folder = write_model_folder(tmp_path / "routed", cfg, 9, std=0.08, gain_std=0.1, scale=scale)
    engine = Engine(folder, dtype=NAME[dtype], max_tokens=1024, max_slots=4)
    assert not engine.model.graph_safe and not engine.stepper.use_graphs
    w = {k: v.float() for k, v in load_file(str(folder / "model.safetensors")).items()}
    g = torch.Generator().manual_seed(4)
    seqs = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (80, 12)]
    rounding = None if dtype == torch.float32 else torch.bfloat16
    refs, margins = zip(*[routed_plain(w, s, rounding) for s in seqs])
    used = set()
    for cuts in ([80, 12], [50, 2]):
        slots = [engine.cache.alloc() for _ in seqs]
        got = [[] for _ in seqs]
        out = engine.step([StepEntry(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cuts)])
        got[0].append(out[:cuts[0]]); got[1].append(out[cuts[0]:])
        fed = list(cuts)
        while any(f < len(s) for f, s in zip(fed, seqs)):
            live = [i for i in range(2) if fed[i] < len(seqs[i])]
            out = engine.step([StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live])
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1]); fed[i] += 1
        for i in range(2):
            # a row whose two best experts are nearly tied may go either way once rounding differs:
            # such rows, and the rows after them in the sequence, are left out
            close_call = (margins[i] < (1e-3 if dtype == torch.float32 else 0.15)).nonzero().flatten()
            keep = int(close_call[0]) if close_call.numel() else len(seqs[i])
            used.add(keep)
            assert_close(torch.cat(got[i])[:keep], refs[i][:keep], NAME[dtype], f"routed toy, cuts {cuts}, request {i}")
        for s in slots:
            engine.cache.free(s)
    assert max(used) >= 12, "the routing margins left nothing to compare"
    engine.cache.check()
    assert len(list(engine.generate([seqs[1]], 3))) == 3
