"""Reading a model folder's config.json into a typed record.

The reference fills its ModelConfig from GGUF metadata keyed by the architecture's name, with a
default for each optional key (gguf.go:50-61, gguf.go:585-612). Here the source is config.json; the
same defaults apply where the reference has them.
"""
from __future__ import annotations

import json
from pathlib import Path


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model: names the key and what is wrong."""


_MISSING = object()


class KeyReader:
    """Typed access to a config dict; remembers which keys were read, so that the rest can be
    reported."""

    def __init__(self, raw: dict, where: str):
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: top level must be a JSON object")
        self.raw = raw
        self.where = where
        self.seen: set[str] = set()

    def _get(self, key, default):
        self.seen.add(key)
        v = self.raw.get(key, _MISSING)
        if v is _MISSING or v is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key {key!r} is missing")
            return default
        return v

    def integer(self, key, default=_MISSING, minimum=None):
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            raise ConfigError(f"{self.where}: {key!r} must be an integer, found {v!r}")
        v = int(v)
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: {key!r} must be at least {minimum}, found {v}")
        return v

    def number(self, key, default=_MISSING, positive=False):
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: {key!r} must be a number, found {v!r}")
        v = float(v)
        if positive and not v > 0:
            raise ConfigError(f"{self.where}: {key!r} must be positive, found {v}")
        return v

    def boolean(self, key, default=_MISSING):
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: {key!r} must be true or false, found {v!r}")
        return v

    def string(self, key, default=_MISSING, choices=None):
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: {key!r} must be a string, found {v!r}")
        if choices is not None and v not in choices:
            raise ConfigError(f"{self.where}: {key!r} is {v!r}; supported: {', '.join(choices)}")
        return v

    def any(self, key, default=None):
        return self._get(key, default)


def read_config_json(model_dir) -> tuple[dict, str]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    return raw, str(path)
