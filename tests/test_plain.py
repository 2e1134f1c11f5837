"""The plain implementation: properties of its own, and agreement with the outputs of
the reference's CPU-runnable code that tests/golden/make_golden.py recorded."""

import math
from pathlib import Path

import pytest
import torch

import plain_qwen3 as plain
from helpers import tiny_config, write_tiny

GOLDEN = Path(__file__).parent / "golden" / "golden_tiny.safetensors"


@pytest.fixture(scope="module")
def golden():
    from safetensors.torch import load_file

    return load_file(str(GOLDEN))


def test_golden_rope_tables(golden):
    """cos/sin as the reference's rope_tables builds them (engine/model.py:78-93), bf16,
    cat(angle, angle): the plain half tables must equal both halves."""
    for name in ("tiny_a", "tiny_b"):
        cfg = tiny_config(name)
        cos, sin = plain.rope_tables(cfg.head_dim, cfg.rope_theta, 96, torch.float32, torch.bfloat16)
        half = cfg.head_dim // 2
        for mine, ref in ((cos, golden[f"{name}.cos"]), (sin, golden[f"{name}.sin"])):
            assert torch.equal(mine.to(torch.bfloat16), ref[:, :half])
            assert torch.equal(ref[:, :half], ref[:, half:])
        assert abs(golden[f"{name}.scale"].item() - 1 / math.sqrt(cfg.head_dim)) < 1e-7


def test_golden_attention_oracle(golden):
    """The reference's reference_attention (engine/kernels/attention.py:255-276): R new
    rows at pos[b], row t sees keys 0..pos[b]+t. The plain attention over the whole
    sequence gives the same rows."""
    q, k, v, pos, want = (golden[f"attn.{n}"] for n in ("q", "k", "v", "pos", "out"))
    B, HQ, R, D = q.shape
    for b in range(B):
        p = int(pos[b])
        L = p + R
        qq = torch.zeros((L, HQ, D))
        qq[p:] = q[b].transpose(0, 1)
        out = plain.causal_gqa_attention(qq, k[b, :, :L].transpose(0, 1), v[b, :, :L].transpose(0, 1))
        got = out.view(L, HQ, D)[p:]
        assert torch.allclose(got, want[b], atol=2e-6, rtol=1e-5)


def test_golden_fused_layouts_and_tied_head(golden, tmp_path):
    """The reference concatenates q, k, v rows and gate, up rows (engine/model.py:112-116)
    and aliases the head to the embedding when tied (:103-107); this package's parts
    build the same fused matrices from the same folder."""
    from kernel_rush_kawk_b200 import write_model_folder
    from kernel_rush_kawk_b200.engine.model import Model, Runtime
    from kernel_rush_kawk_b200.config.registry import read_config
    from kernel_rush_kawk_b200.weights import read_checkpoint

    folder = write_model_folder(tmp_path / "a", tiny_config("tiny_a"), 101)
    arch, cfg = read_config(folder)
    plan = arch.plan(cfg)
    from kernel_rush_kawk_b200.engine.model import PartTree

    tensors = read_checkpoint(folder, PartTree(plan).expected_tensors(), "cpu", torch.bfloat16, plan.duplicates)
    model = Model(plan, Runtime(torch.device("cpu"), torch.bfloat16, None), tensors, 96)
    assert torch.equal(model.blocks[0].mixer.w_qkv, golden["tiny_a.layer0.wqkv"])
    assert torch.equal(model.blocks[1].feed_forward.w_gate_up, golden["tiny_a.layer1.wgu"])
    assert golden["tiny_a.lm_head_is_embed"].item() == 1 and model.head.weight is model.embedding.table
    assert golden["tiny_b.lm_head_is_embed"].item() == 0
    assert torch.equal(model.position.cos.to(torch.bfloat16), golden["tiny_a.cos"][:, :cfg.head_dim // 2])


def test_rms_norm_is_the_formula():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.0]])
    w = torch.tensor([1.0, 2.0, 3.0, 4.0])
    got = plain.rms_norm(x, w, 0.0)
    assert torch.allclose(got, torch.tensor([[3 / 2.5, 8 / 2.5, 0.0, 0.0]]))
    r = plain.rms_norm(x, w, 0.0, torch.bfloat16)
    assert torch.equal(r, r.bfloat16().float())


def test_rope_scores_depend_on_distance_only():
    D, theta = 16, 10000.0
    cos, sin = plain.rope_tables(D, theta, 64)
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, D, generator=g), torch.randn(1, 1, D, generator=g)
    w = torch.ones(D)

    def score(pq, pk):
        a = plain.head_norm_rope(q, w, cos[pq:pq + 1], sin[pq:pq + 1], 1e-6)
        b = plain.head_norm_rope(k, w, cos[pk:pk + 1], sin[pk:pk + 1], 1e-6)
        return (a * b).sum().item()

    assert abs(score(10, 3) - score(47, 40)) < 1e-4
    assert abs(score(10, 3) - score(10, 4)) > 1e-4


def test_logits_at_a_position_do_not_depend_on_later_tokens(tmp_path):
    folder = write_tiny(tmp_path / "b", "tiny_b")
    cfg, w = plain.read_folder(folder)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab, (20,), generator=g).tolist()
    a = plain.forward_logits(cfg, w, ids)
    b = plain.forward_logits(cfg, w, ids[:12] + [(t + 1) % cfg.vocab for t in ids[12:]])
    assert torch.allclose(a[:12], b[:12], atol=1e-6) and not torch.allclose(a[12:], b[12:], atol=1e-3)


def test_a_window_hides_older_keys(tmp_path):
    folder = write_tiny(tmp_path / "w", "tiny_w")
    cfg, w = plain.read_folder(folder)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg.vocab, (60,), generator=g).tolist()
    full = plain.forward_logits(cfg, w, ids)
    windowed = plain.forward_logits(cfg, w, ids, windows=[None, 24, 24])
    assert torch.allclose(full[:24], windowed[:24], atol=1e-6)
    assert not torch.allclose(full[40:], windowed[40:], atol=1e-3)


def test_gqa_head_to_group_mapping():
    """q head h reads kv head h // G: with two groups whose values differ, heads 0..G-1
    return group 0's value."""
    T, HQ, HKV, D = 3, 4, 2, 8
    q = torch.zeros(T, HQ, D)
    k = torch.zeros(T, HKV, D)
    v = torch.zeros(T, HKV, D)
    v[:, 0], v[:, 1] = 1.0, 2.0
    out = plain.causal_gqa_attention(q, k, v).view(T, HQ, D)
    assert torch.all(out[:, :2] == 1.0) and torch.all(out[:, 2:] == 2.0)


def test_sampling_definition():
    logits = torch.tensor([2.0, 1.0, 0.0])
    assert plain.greedy(torch.tensor([1.0, 3.0, 3.0])) == 1
    u = plain.gumbel_uniforms(1, 2, 3, 1000)
    assert 0 < u.min() and u.max() < 1 and not torch.equal(u, plain.gumbel_uniforms(1, 2, 4, 1000))
    counts = torch.zeros(3)
    for step in range(4000):
        counts[plain.sample_temperature(logits, 1.0, 5, 0, step)] += 1
    assert torch.allclose(counts / 4000, torch.softmax(logits, -1), atol=0.03)
