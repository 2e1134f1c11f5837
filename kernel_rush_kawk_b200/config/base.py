"""What every architecture's configuration has in common.

A configuration is a frozen dataclass read from the architecture's own
``config.json`` keys. It holds numbers only; how they turn into layers is the
business of the architecture module that is registered beside it
(``config/registry.py``).
"""

from __future__ import annotations

import json
from pathlib import Path


class ConfigError(ValueError):
    """A config.json that this library cannot run: a missing key, a value out of
    range, or an option of the architecture that is not implemented."""


class ModelConfig:
    """Base class of typed configurations; subclasses are frozen dataclasses."""

    #: the name found in config.json's ``architectures``
    architecture: str = ""

    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict:
        raise NotImplementedError

    @classmethod
    def preset_names(cls) -> list[str]:
        """Names of the configurations this class keeps ready (none by default)."""
        return []

    @classmethod
    def preset(cls, name: str) -> "ModelConfig":
        raise ConfigError(f"unknown preset '{name}'; known presets: {cls.preset_names()}")

    @classmethod
    def from_json(cls, path) -> "ModelConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        if not path.is_file():
            raise ConfigError(f"no config.json at {path}")
        try:
            raw = json.loads(path.read_text())
        except json.JSONDecodeError as exc:
            raise ConfigError(f"{path} is not valid JSON: {exc}") from exc
        if not isinstance(raw, dict):
            raise ConfigError(f"{path} must hold a JSON object")
        return cls.from_dict(raw)


def require(raw: dict, key: str, kind, what: str = ""):
    """Fetch a required key and check its type; one clear error otherwise."""
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks the required key '{key}'{what}")
    value = raw[key]
    if kind is float and isinstance(value, int) and not isinstance(value, bool):
        value = float(value)
    if kind is int and isinstance(value, bool) or not isinstance(value, kind):
        raise ConfigError(f"config.json key '{key}' must be {kind.__name__}, got {value!r}")
    return value


def positive(name: str, value) -> None:
    if not value > 0:
        raise ConfigError(f"config.json key '{name}' must be positive, got {value!r}")
