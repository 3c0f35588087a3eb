"""One registry from the architecture's name (config.json `architectures[0]`) to its model.

The reference selects only a metadata prefix by `general.architecture` and runs every decoder
through one code path (gguf.go:585, README.md:17-20). Here an entry holds the typed configuration
class and the function that lays the model out from it; adding an architecture is one `register`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .base import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type            # has from_dict(raw, where) and to_json_dict()
    layout: Callable              # config -> engine.layout.ModelLayout


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, layout: Callable, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, layout)


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_for(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"architecture {name!r} is not registered; registered: "
                          f"{', '.join(registered_architectures()) or '(none)'}") from None


def load_config(model_dir):
    """config.json of `model_dir` -> (Architecture, typed config)."""
    raw, where = read_config_json(model_dir)
    archs = raw.get("architectures")
    if not (isinstance(archs, list) and archs and isinstance(archs[0], str)):
        raise ConfigError(f"{where}: 'architectures' must be a list that names the model class")
    arch = architecture_for(archs[0])
    return arch, arch.config_class.from_dict(raw, where)
