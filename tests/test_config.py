"""Configuration and registry (no GPU)."""

import json

import pytest

from kernel_rush_kawk_b200 import ConfigError, Qwen3Config, read_config, register_architecture
from kernel_rush_kawk_b200.config.registry import get_architecture, known_architectures

BASE = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 64, "intermediate_size": 192, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 256, "rms_norm_eps": 1e-6, "rope_theta": 10000.0}


def test_presets_read_and_differ():
    a, b = Qwen3Config.preset("tiny_a"), Qwen3Config.preset("tiny_b")
    for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "head_dim", "vocab_size",
                "rms_norm_eps", "rope_theta", "tie_word_embeddings"):
        assert getattr(a, key) != getattr(b, key), key
    big = Qwen3Config.preset("qwen3_4b")
    assert (big.hidden_size, big.head_dim, big.num_attention_heads * big.head_dim) == (2560, 128, 4096)
    with pytest.raises(ConfigError, match="unknown preset"):
        Qwen3Config.preset("nope")


def test_reference_defaults():
    cfg = Qwen3Config.from_dict(BASE)
    assert cfg.head_dim == 16 and cfg.tie_word_embeddings is False  # engine/model.py:47,51 of the reference
    assert Qwen3Config.from_dict({**BASE, "head_dim": 32}).head_dim == 32


@pytest.mark.parametrize("change, message", [
    ({"rms_norm_eps": None}, "rms_norm_eps"), ({"rope_theta": None}, "rope_theta"),
    ({"hidden_size": "64"}, "hidden_size"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"), ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"), ({"vocab_size": 0}, "positive"),
    ({"eos_token_id": 999}, "vocabulary"), ({"use_sliding_window": True, "max_window_layers": 1}, "sliding_window"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
])
def test_bad_values_are_refused(change, message):
    raw = {k: v for k, v in {**BASE, **change}.items() if v is not None}
    with pytest.raises(ConfigError, match=message):
        Qwen3Config.from_dict(raw)


def test_window_layers():
    cfg = Qwen3Config.from_dict({**BASE, "use_sliding_window": True, "sliding_window": 8, "max_window_layers": 1})
    assert cfg.window_layers == (1,) and cfg.window_of(0) is None and cfg.window_of(1) == 8
    cfg = Qwen3Config.from_dict({**BASE, "sliding_window": 8, "layer_types": ["sliding_attention", "full_attention"]})
    assert cfg.window_layers == (0,)
    assert Qwen3Config.from_dict({**BASE, "sliding_window": 8, "use_sliding_window": False}).sliding_window is None


def test_round_trip_through_config_json(tmp_path):
    for cfg in (Qwen3Config.preset("tiny_b"),
                Qwen3Config.from_dict({**BASE, "sliding_window": 8, "layer_types": ["sliding_attention", "full_attention"],
                                       "eos_token_id": [1, 2]})):
        (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
        arch, again = read_config(tmp_path)
        assert again == cfg and arch.name == "Qwen3ForCausalLM"


def test_registry():
    assert "Qwen3ForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="unknown architecture 'Llama"):
        read_config({**BASE, "architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        read_config({k: v for k, v in BASE.items() if k != "architectures"})
    with pytest.raises(ConfigError, match="no config.json"):
        read_config("/nonexistent/folder")
    register_architecture("ToyForTests", Qwen3Config, lambda cfg: None)
    assert get_architecture("ToyForTests").config_class is Qwen3Config


def test_plan_is_data():
    cfg = Qwen3Config.preset("tiny_b")
    plan = get_architecture(cfg.architecture).plan(cfg)
    assert len(plan.layers) == 3 and [e.layer for e in plan.schedule] == [0, 1, 2]
    mixer = plan.layers[1].mixer
    assert mixer.kind == "gqa_attention" and mixer.params["head_dim"] == 32 and mixer.params["eps"] == 1e-5
    assert mixer.tensors["q_norm"] == "model.layers.1.self_attn.q_norm.weight"
    assert plan.head.tensors["weight"] == "lm_head.weight"
    tied = get_architecture(cfg.architecture).plan(Qwen3Config.preset("tiny_a"))
    assert tied.head.tensors["weight"] == "model.embed_tokens.weight"
