"""One registry from an architecture's name to its configuration and model.

``config.json["architectures"][0]`` picks the entry. An entry is a typed
configuration class and a function that turns a configuration into a
``ModelPlan`` (``parts/plan.py``): the list of layers, their parts and the
order in which they run. Everything downstream (weights, cache, step function)
is built from the plan and never asks which architecture it serves.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from .base import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    plan: Callable  # (config) -> ModelPlan


_REGISTRY: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, plan: Callable) -> None:
    """Add (or replace) an architecture. ``plan(config)`` returns a ModelPlan."""
    _REGISTRY[name] = Architecture(name, config_class, plan)


def known_architectures() -> list[str]:
    _load_builtin()
    return sorted(_REGISTRY)


def get_architecture(name: str) -> Architecture:
    _load_builtin()
    try:
        return _REGISTRY[name]
    except KeyError:
        raise ConfigError(f"unknown architecture '{name}'; registered: {sorted(_REGISTRY)}") from None


def architecture_name(raw: dict) -> str:
    names = raw.get("architectures")
    if not names or not isinstance(names, (list, tuple)):
        raise ConfigError("config.json lacks 'architectures' (a list with the model class name)")
    return str(names[0])


def read_config(folder_or_dict) -> tuple[Architecture, ModelConfig]:
    """Read a model folder's config.json (or take its content as a dict) and return
    the registered architecture with the typed configuration."""
    if isinstance(folder_or_dict, dict):
        raw = folder_or_dict
    else:
        path = Path(folder_or_dict)
        path = path / "config.json" if path.is_dir() else path
        if not path.is_file():
            raise ConfigError(f"no config.json at {path}")
        try:
            raw = json.loads(path.read_text())
        except json.JSONDecodeError as exc:
            raise ConfigError(f"{path} is not valid JSON: {exc}") from exc
    arch = get_architecture(architecture_name(raw))
    return arch, arch.config_class.from_dict(raw)


def preset_config(name: str) -> ModelConfig:
    """The named ready-made configuration of whichever registered architecture keeps one of that name."""
    _load_builtin()
    known = {}
    for arch in _REGISTRY.values():
        names = arch.config_class.preset_names()
        if name in names:
            return arch.config_class.preset(name)
        known[arch.name] = names
    raise ConfigError(f"unknown preset '{name}'; known presets by architecture: {known}")


_builtin_loaded = False


def _load_builtin() -> None:
    global _builtin_loaded
    if not _builtin_loaded:
        _builtin_loaded = True
        from ..models import qwen3  # noqa: F401  (registers itself on import)
