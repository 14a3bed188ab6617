"""Typed configuration base and the architecture registry.

A model folder's `config.json` names its architecture in `architectures[0]`.
The registry maps that name to a configuration class (which parses and checks
the architecture's own keys) and to a builder (which turns the typed
configuration into a `ModelSpec`: parts chosen layer by layer plus the order in
which layers run).  Nothing outside an architecture's own module knows its keys.

The reference has a single hard-wired `ModelConfig` (include/model.h:58-81) whose
checks (src/load.cc:315-363) are kept in spirit by `LlamaConfig.validate`.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Any, Callable, Dict, Tuple, Type


class ConfigError(ValueError):
    """A `config.json` that is missing a key, has a wrong type or breaks a rule."""


@dataclass
class ModelConfig:
    """Base of every typed configuration."""

    architecture: str = ""

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        """The `config.json` content that `from_dict` reads back unchanged."""
        raise NotImplementedError

    def validate(self) -> None:
        raise NotImplementedError

    def field_names(self):
        return [f.name for f in fields(self)]


_REGISTRY: Dict[str, Tuple[Type[ModelConfig], Callable]] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig], builder: Callable) -> None:
    """Register `name` (as written in `architectures`) with its config class and
    its builder `builder(config) -> ModelSpec`.  Registering a name twice
    replaces the earlier entry, which lets tests register toy architectures."""
    _REGISTRY[name] = (config_cls, builder)


def known_architectures():
    return sorted(_REGISTRY)


def lookup_architecture(name: str):
    if name not in _REGISTRY:
        raise ConfigError(
            f"unknown architecture {name!r}; known: {', '.join(known_architectures()) or '(none)'}")
    return _REGISTRY[name]


def architecture_of(raw: Dict[str, Any]) -> str:
    archs = raw.get("architectures")
    if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a list with exactly one name")
    return archs[0]


def config_from_dict(raw: Dict[str, Any]) -> ModelConfig:
    """Pick the configuration class by `architectures[0]`, parse and validate."""
    if not isinstance(raw, dict):
        raise ConfigError("config.json: top level must be an object")
    name = architecture_of(raw)
    config_cls, _ = lookup_architecture(name)
    config = config_cls.from_dict(raw)
    config.architecture = name
    config.validate()
    return config


def load_config(folder) -> ModelConfig:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from None
    return config_from_dict(raw)


def save_config(config: ModelConfig, folder) -> None:
    Path(folder).mkdir(parents=True, exist_ok=True)
    (Path(folder) / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")


# ---- small typed getters shared by configuration classes ------------------- #
def take_int(raw, key, default=None, minimum=None):
    if key not in raw or raw[key] is None:
        if default is None:
            raise ConfigError(f"config.json: missing required key {key!r}")
        return default
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config.json: {key!r} must be an integer, got {value!r}")
    if minimum is not None and value < minimum:
        raise ConfigError(f"config.json: {key!r} must be >= {minimum}, got {value}")
    return value


def take_float(raw, key, default=None):
    if key not in raw or raw[key] is None:
        if default is None:
            raise ConfigError(f"config.json: missing required key {key!r}")
        return float(default)
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: {key!r} must be a number, got {value!r}")
    value = float(value)
    if value != value or value in (float("inf"), float("-inf")):
        raise ConfigError(f"config.json: {key!r} must be finite, got {value!r}")
    return value


def take_bool(raw, key, default):
    if key not in raw or raw[key] is None:
        return default
    value = raw[key]
    if not isinstance(value, bool):
        raise ConfigError(f"config.json: {key!r} must be true or false, got {value!r}")
    return value
