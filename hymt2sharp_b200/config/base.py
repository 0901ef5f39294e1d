"""Typed reading of config.json: every architecture's configuration class is
built from these helpers, so that a wrong or missing key gives one kind of
error that names the key."""
from __future__ import annotations

import json
import os
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot be used: the message names the key."""


_MISSING = object()


class ConfigReader:
    """Reads keys of one config.json dictionary with types and aliases."""

    def __init__(self, data: dict, source: str = "config.json"):
        if not isinstance(data, dict):
            raise ConfigError(f"{source}: the top level must be an object")
        self.data = data
        self.source = source

    def _find(self, names, default):
        for name in names:
            node: Any = self.data
            ok = True
            for part in name.split("."):
                if isinstance(node, dict) and part in node and node[part] is not None:
                    node = node[part]
                else:
                    ok = False
                    break
            if ok:
                return name, node
        if default is _MISSING:
            raise ConfigError(f"{self.source}: required key '{names[0]}' is missing")
        return names[0], default

    def integer(self, *names, default=_MISSING, minimum=None) -> int:
        name, v = self._find(names, default)
        if v is None:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            raise ConfigError(f"{self.source}: key '{name}' must be an integer, got {v!r}")
        v = int(v)
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.source}: key '{name}' must be >= {minimum}, got {v}")
        return v

    def number(self, *names, default=_MISSING, minimum=None, exclusive_minimum=None) -> float:
        name, v = self._find(names, default)
        if v is None:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.source}: key '{name}' must be a number, got {v!r}")
        v = float(v)
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.source}: key '{name}' must be >= {minimum}, got {v}")
        if exclusive_minimum is not None and v <= exclusive_minimum:
            raise ConfigError(f"{self.source}: key '{name}' must be > {exclusive_minimum}, got {v}")
        return v

    def boolean(self, *names, default=_MISSING) -> bool:
        name, v = self._find(names, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.source}: key '{name}' must be true or false, got {v!r}")
        return v

    def string(self, *names, default=_MISSING) -> str:
        name, v = self._find(names, default)
        if v is not None and not isinstance(v, str):
            raise ConfigError(f"{self.source}: key '{name}' must be a string, got {v!r}")
        return v


def read_config_json(folder_or_file: str) -> dict:
    path = folder_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path) as f:
            return json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None


def architecture_name(data: dict, source: str = "config.json") -> str:
    archs = data.get("architectures")
    if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError(f"{source}: key 'architectures' must be a list with one architecture name")
    return archs[0]
