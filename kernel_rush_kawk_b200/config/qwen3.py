"""Typed configuration of the Qwen3 dense decoder (``Qwen3ForCausalLM``).

The keys and their defaults follow the reference's reader (engine/model.py:39-52
of willzeng274/kernel-rush-kawk): ``head_dim`` is optional and defaults to
``hidden_size // num_attention_heads``; ``tie_word_embeddings`` defaults to
False; ``rms_norm_eps`` and ``rope_theta`` have no default. The reference
ignores every other key of config.json; the ones that would change the
arithmetic are read here so that an unsupported value is an error rather than a
silently different model.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, asdict
from pathlib import Path

from .base import ConfigError, ModelConfig, positive, require

PRESET_DIR = Path(__file__).parent / "presets"


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 32768
    #: None: every layer sees all keys. Otherwise the layers listed in
    #: ``window_layers`` see only the last ``sliding_window`` keys.
    sliding_window: int | None = None
    window_layers: tuple[int, ...] = ()
    eos_token_ids: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"

    architecture = "Qwen3ForCausalLM"

    # ------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        hidden = require(raw, "hidden_size", int)
        heads = require(raw, "num_attention_heads", int)
        positive("num_attention_heads", heads)
        head_dim = raw.get("head_dim") or hidden // heads
        layers = require(raw, "num_hidden_layers", int)

        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act '{act}' is not supported: the Qwen3 feed-forward here is SwiGLU with silu")
        if raw.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not supported: the Qwen3 projections here have no bias")
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError(f"rope_scaling {raw['rope_scaling']!r} is not supported: only unscaled RoPE")

        window, window_layers = cls._read_window(raw, layers)

        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        else:
            eos_ids = tuple(int(e) for e in eos)

        cfg = cls(
            hidden_size=hidden,
            intermediate_size=require(raw, "intermediate_size", int),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=require(raw, "num_key_value_heads", int),
            head_dim=int(head_dim),
            vocab_size=require(raw, "vocab_size", int),
            rms_norm_eps=require(raw, "rms_norm_eps", float),
            rope_theta=require(raw, "rope_theta", float),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            max_position_embeddings=int(raw.get("max_position_embeddings", 32768)),
            sliding_window=window,
            window_layers=window_layers,
            eos_token_ids=eos_ids,
            torch_dtype=str(raw.get("torch_dtype", raw.get("dtype", "bfloat16"))),
        )
        cfg.validate()
        return cfg

    @staticmethod
    def _read_window(raw: dict, layers: int) -> tuple[int | None, tuple[int, ...]]:
        """Which layers see a window of keys only. ``layer_types`` (one entry per
        layer, "full_attention" or "sliding_attention") wins; otherwise, with
        ``use_sliding_window``, the layers from ``max_window_layers`` on. The
        reference runs every layer with all keys (engine/model.py:276,
        engine/kernels/attention.py:111) and reads none of these keys."""
        window = raw.get("sliding_window")
        types = raw.get("layer_types")
        if types is not None:
            if len(types) != layers:
                raise ConfigError(f"layer_types has {len(types)} entries for {layers} layers")
            bad = sorted(set(types) - {"full_attention", "sliding_attention"})
            if bad:
                raise ConfigError(f"layer_types holds unknown kinds {bad}")
            chosen = tuple(i for i, t in enumerate(types) if t == "sliding_attention")
        elif raw.get("use_sliding_window", False):
            first = int(raw.get("max_window_layers", layers))
            chosen = tuple(range(first, layers))
        else:
            chosen = ()
        if not chosen:
            return None, ()
        if not isinstance(window, int) or isinstance(window, bool) or window <= 0:
            raise ConfigError(f"layers {list(chosen)} use a sliding window but sliding_window is {window!r}")
        return window, chosen

    def validate(self) -> None:
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "vocab_size", "rms_norm_eps", "rope_theta",
                     "max_position_embeddings"):
            positive(name, getattr(self, name))
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even for rotate-half RoPE")
        for tok in self.eos_token_ids:
            if not 0 <= tok < self.vocab_size:
                raise ConfigError(f"eos_token_id {tok} lies outside the vocabulary of {self.vocab_size}")

    # ------------------------------------------------------------------
    def to_dict(self) -> dict:
        """config.json content that reads back to an equal configuration."""
        d = asdict(self)
        window_layers = d.pop("window_layers")
        eos = d.pop("eos_token_ids")
        d["architectures"] = [self.architecture]
        d["model_type"] = "qwen3"
        d["hidden_act"] = "silu"
        d["attention_bias"] = False
        if eos:
            d["eos_token_id"] = eos[0] if len(eos) == 1 else list(eos)
        if window_layers:
            d["layer_types"] = ["sliding_attention" if i in window_layers else "full_attention"
                                for i in range(self.num_hidden_layers)]
        else:
            d.pop("sliding_window")
        return d

    @classmethod
    def preset_names(cls) -> list[str]:
        return sorted(p.stem for p in PRESET_DIR.glob("*.json"))

    @classmethod
    def preset(cls, name: str) -> "Qwen3Config":
        """A named configuration kept as a JSON file beside this module."""
        path = PRESET_DIR / f"{name}.json"
        if not path.is_file():
            raise ConfigError(f"unknown preset '{name}'; known presets: {cls.preset_names()}")
        return cls.from_dict(json.loads(path.read_text()))

    def window_of(self, layer: int) -> int | None:
        return self.sliding_window if layer in self.window_layers else None
