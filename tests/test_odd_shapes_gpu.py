"""Configurations at the edges of what the kernels take: head size 256, one kv head for 32 query heads,
as many kv heads as query heads with a window on every layer, widths that are no multiple of 8 or 32, an
intermediate size that is no multiple of 8. Each against the plain implementation, in 32-bit and in bfloat16:
an unequal batch of prompts, then one token each."""

import pytest
import torch

import plain_qwen3 as plain
from helpers import assert_close

pytestmark = pytest.mark.gpu

BASE = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "rms_norm_eps": 1e-6, "rope_theta": 1e4,
        "tie_word_embeddings": True, "max_position_embeddings": 1024}
ODD = {
    "head_256": dict(hidden_size=96, intermediate_size=160, num_hidden_layers=2, num_attention_heads=2,
                     num_key_value_heads=1, head_dim=256, vocab_size=211),
    "group_of_32": dict(hidden_size=72, intermediate_size=200, num_hidden_layers=2, num_attention_heads=32,
                        num_key_value_heads=1, head_dim=16, vocab_size=97, tie_word_embeddings=False),
    "every_head_its_own_keys_and_a_window": dict(
        hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=8,
        head_dim=64, vocab_size=500, sliding_window=70, layer_types=["sliding_attention", "sliding_attention"]),
    "sizes_off_every_grid": dict(hidden_size=120, intermediate_size=100, num_hidden_layers=1, num_attention_heads=6,
                                 num_key_value_heads=3, head_dim=80, vocab_size=1001, tie_word_embeddings=False,
                                 rms_norm_eps=1e-5, rope_theta=5e5),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ODD))
def test_odd_configuration_against_plain(name, dtype, tmp_path):
    from kernel_rush_kawk_b200 import Engine, Qwen3Config, StepEntry, write_model_folder

    cfg = Qwen3Config.from_dict({**BASE, **ODD[name]})
    scale = {f"model.layers.{i}.self_attn.{n}_norm.weight": 1.5 for i in range(cfg.num_hidden_layers) for n in ("q", "k")}
    folder = write_model_folder(tmp_path / name, cfg, 41, std=0.04, gain_std=0.1, scale=scale)
    pcfg, w = plain.read_folder(folder)
    windows = [cfg.window_of(i) for i in range(cfg.num_hidden_layers)]
    g = torch.Generator().manual_seed(8)
    seqs = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (150, 20, 71)]
    wide, rounding = (torch.float64, None) if dtype == "float32" else (torch.float32, torch.bfloat16)
    refs = [plain.forward_logits(pcfg, w, s, wide, rounding, windows).float() for s in seqs]
    engine = Engine(folder, dtype=dtype, max_tokens=2048, max_slots=4)
    cache = engine.cache
    cuts = [140, 3, 64]
    slots = [cache.alloc() for _ in seqs]
    got = [[] for _ in seqs]
    out = engine.step([StepEntry(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cuts)])
    row = 0
    for i, c in enumerate(cuts):
        got[i].append(out[row:row + c].float().cpu())
        row += c
    fed = list(cuts)
    while any(f < len(s) for f, s in zip(fed, seqs)):
        live = [i for i in range(len(seqs)) if fed[i] < len(seqs[i])]
        out = engine.step([StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live]).float().cpu()
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1])
            fed[i] += 1
    for i, ref in enumerate(refs):
        assert_close(torch.cat(got[i]), ref, dtype, f"{name}, request {i}, {dtype}")
    for s in slots:
        cache.free(s)
    cache.check()
    engine.ops.check()
