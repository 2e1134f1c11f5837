"""Weights by name, their errors, and seeded random weights (no GPU)."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from helpers import tiny_config
from kernel_rush_kawk_b200 import WeightError, write_model_folder
from kernel_rush_kawk_b200.config.registry import get_architecture
from kernel_rush_kawk_b200.engine.model import expected_tensors
from kernel_rush_kawk_b200.weights import random_tensors, read_checkpoint, stored_dtype


def expected(name):
    cfg = tiny_config(name)
    plan = get_architecture(cfg.architecture).plan(cfg)
    return plan, expected_tensors(plan)


def test_expected_names_are_the_checkpoints_own():
    _, exp = expected("tiny_b")
    assert exp["model.layers.2.self_attn.q_proj.weight"].shape == (6 * 32, 96)
    assert exp["model.layers.0.self_attn.k_norm.weight"].shape == (32,)
    assert exp["model.layers.1.mlp.down_proj.weight"].shape == (96, 256)
    assert exp["lm_head.weight"].shape == (384, 96) and len(exp) == 3 + 3 * 11
    _, tied = expected("tiny_a")
    assert "lm_head.weight" not in tied  # the head reads model.embed_tokens.weight


def test_random_weights_depend_on_name_and_seed_only():
    _, exp = expected("tiny_a")
    a = random_tensors(exp, 5)
    b = random_tensors(dict(reversed(list(exp.items()))), 5)
    assert all(torch.equal(a[n], b[n]) for n in exp)
    c = random_tensors(exp, 6)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    assert abs(a["model.norm.weight"].float().mean().item() - 1.0) < 0.02
    assert abs(a["model.embed_tokens.weight"].float().std().item() - 0.02) < 0.002
    assert a["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_folder_round_trip(tmp_path):
    plan, exp = expected("tiny_b")
    folder = write_model_folder(tmp_path / "m", tiny_config("tiny_b"), 9)
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["Qwen3ForCausalLM"]
    got = read_checkpoint(folder, exp, "cpu", torch.bfloat16)
    want = random_tensors(exp, 9)
    assert all(torch.equal(got[n], want[n]) for n in exp)
    wide = read_checkpoint(folder, exp, "cpu", torch.float32)
    assert all(t.dtype == torch.float32 for t in wide.values())
    assert torch.equal(wide["lm_head.weight"], want["lm_head.weight"].float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    plan, exp = expected("tiny_a")
    folder = write_model_folder(tmp_path / "m", tiny_config("tiny_a"), 1)
    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.o_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError) as err:
        read_checkpoint(folder, exp, "cpu", torch.bfloat16)
    e = err.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert e.wrong_shape == {"model.layers.0.self_attn.o_proj.weight": ((64, 64), (64, 32))}
    text = str(e)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "expected [64, 64], found [64, 32]"):
        assert piece in text


def test_no_shards_and_a_truncated_shard(tmp_path):
    _, exp = expected("tiny_a")
    (tmp_path / "empty").mkdir()
    with pytest.raises(FileNotFoundError):
        read_checkpoint(tmp_path / "empty", exp, "cpu", torch.bfloat16)
    folder = write_model_folder(tmp_path / "m", tiny_config("tiny_a"), 1)
    data = (folder / "model.safetensors").read_bytes()
    (folder / "model.safetensors").write_bytes(data[:len(data) // 2])
    with pytest.raises(WeightError, match="cannot be read"):
        read_checkpoint(folder, exp, "cpu", torch.bfloat16)


def test_a_tied_head_stored_twice(tmp_path):
    plan, exp = expected("tiny_a")
    folder = write_model_folder(tmp_path / "m", tiny_config("tiny_a"), 1)
    tensors = load_file(str(folder / "model.safetensors"))
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, str(folder / "model.safetensors"))
    read_checkpoint(folder, exp, "cpu", torch.bfloat16, plan.duplicates)  # equal: accepted
    with pytest.raises(WeightError, match="unexpected"):
        read_checkpoint(folder, exp, "cpu", torch.bfloat16)  # not declared: unexpected
    tensors["lm_head.weight"] = tensors["lm_head.weight"] + 1
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError, match="differs"):
        read_checkpoint(folder, exp, "cpu", torch.bfloat16, plan.duplicates)


def test_sharded_folder_and_dtype_policy(tmp_path):
    plan, exp = expected("tiny_a")
    folder = write_model_folder(tmp_path / "m", tiny_config("tiny_a"), 1)
    tensors = load_file(str(folder / "model.safetensors"))
    (folder / "model.safetensors").unlink()
    names = sorted(tensors)
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()  # a vector stored in 32-bit stays so
    tensors["model.layers.0.mlp.down_proj.weight"] = tensors["model.layers.0.mlp.down_proj.weight"].float()
    save_file({n: tensors[n] for n in names[:10]}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({n: tensors[n] for n in names[10:]}, str(folder / "model-00002-of-00002.safetensors"))
    got = read_checkpoint(folder, exp, "cpu", torch.bfloat16)
    assert got["model.norm.weight"].dtype == torch.float32
    assert got["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert stored_dtype("table", 1, torch.int64, torch.bfloat16) == torch.int32
    assert stored_dtype("matrix", 2, torch.float16, torch.float32) == torch.float32
