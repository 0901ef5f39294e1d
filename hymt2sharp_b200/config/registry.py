"""One registry from an architecture's name (config.json "architectures"[0])
to its configuration class and its model builder."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .base import ConfigError, architecture_name, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build_spec: Callable  # config -> engine.spec.ModelSpec
    tensor_shapes: Callable  # config -> {tensor name: (shape, kind)} of a checkpoint


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_spec: Callable, tensor_shapes: Callable) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec, tensor_shapes)


def known_architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture '{name}'; known: {', '.join(sorted(_ARCHITECTURES))}") from None


def load_config(folder_or_file: str):
    """config.json → (Architecture, typed configuration)."""
    data = read_config_json(folder_or_file)
    arch = get_architecture(architecture_name(data, str(folder_or_file)))
    return arch, arch.config_class.from_dict(data, str(folder_or_file))


def _load_builtin() -> None:
    # the built-in architecture registers itself on import
    from ..engine import hunyuan_dense  # noqa: F401
