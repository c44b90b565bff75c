"""One registry from an architecture's name (config.json ``architectures[0]``) to its
typed configuration and to the function that describes it with parts."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable

from .model_config import ConfigError

_ARCHITECTURES: dict[str, tuple[type, Callable]] = {}
_BY_MODEL_TYPE: dict[str, str] = {}


def register_architecture(name: str, config_cls: type, spec_builder: Callable, model_type: str | None = None) -> None:
    """``config_cls.from_dict(json)`` must validate; ``spec_builder(config)`` returns a ModelSpec.
    ``model_type`` lets a config.json without an ``architectures`` key find this entry."""
    _ARCHITECTURES[name] = (config_cls, spec_builder)
    if model_type:
        _BY_MODEL_TYPE[model_type] = name


def architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_of(config_json: dict) -> str:
    names = config_json.get("architectures")
    if not names:
        by_type = _BY_MODEL_TYPE.get(config_json.get("model_type"))
        if by_type is None:
            raise ConfigError("config.json names no known architecture (keys 'architectures', 'model_type')")
        names = [by_type]
    if names[0] not in _ARCHITECTURES:
        raise ConfigError(f"architecture {names[0]!r} is not registered; known: {', '.join(architectures()) or 'none'}")
    return names[0]


def resolve(config_json: dict):
    """config.json contents -> (typed config, ModelSpec)."""
    config_cls, builder = _ARCHITECTURES[architecture_of(config_json)]
    cfg = config_cls.from_dict(config_json)
    return cfg, builder(cfg)


def resolve_folder(folder):
    """Model folder -> (typed config, ModelSpec); honours generation_config.json where the
    configuration class reads it."""
    folder = Path(folder)
    path = folder / "config.json"
    if not path.exists():
        raise ConfigError(f"{folder} holds no config.json")
    raw = json.loads(path.read_text())
    config_cls, builder = _ARCHITECTURES[architecture_of(raw)]
    cfg = config_cls.read(folder) if hasattr(config_cls, "read") else config_cls.from_dict(raw)
    return cfg, builder(cfg)
