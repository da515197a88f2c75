"""The one registry from an architecture's name (config.json `architectures[0]`) to its
configuration class.  A configuration class has `from_dict(dict)`, `to_dict()` and `to_spec()`."""
from __future__ import annotations

import json
from pathlib import Path

from .spec import ConfigError

_ARCHITECTURES: dict[str, type] = {}


def register_architecture(name: str):
    def deco(cls):
        _ARCHITECTURES[name] = cls
        cls.architecture = name
        return cls
    return deco


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_from_dict(d: dict):
    archs = d.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError(f"config.json has no 'architectures' list; known architectures: {known_architectures()}")
    name = archs[0]
    cls = _ARCHITECTURES.get(name)
    if cls is None:
        raise ConfigError(f"unknown architecture {name!r}; known architectures: {known_architectures()}")
    return cls.from_dict(d)


def load_config(folder):
    path = Path(folder) / "config.json"
    if not path.exists():
        raise FileNotFoundError(f"config not found at {path}")
    return config_from_dict(json.loads(path.read_text()))
