"""One registry from an architecture's name (config.json `architectures[0]`) to its model.

The reference has a single code path and uses the architecture string only to pick
defaults and the metadata prefix (model.rs:65-71, :89-95).  Here a name maps to an
`Architecture`: how to read its config.json into a typed config, and how to turn that
config into a `ModelSpec` (the list of layers, each assembled from named parts).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .model_config import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]   # config.json dict -> typed config
    build_spec: Callable[[Any], Any]                    # typed config -> parts.spec.ModelSpec


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_spec, *, replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    arch = Architecture(name, parse_config, build_spec)
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {', '.join(sorted(_ARCHITECTURES))}"
        ) from None


def config_from_dict(d: Mapping[str, Any]):
    """Pick the architecture named by the dict and parse it into that architecture's config."""
    archs = d.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError("config.json: 'architectures' must be a non-empty list")
    return get_architecture(str(archs[0])).parse_config(d)


def load_config(model_dir: str):
    return config_from_dict(read_config_json(model_dir))


def load_spec(model_dir: str):
    """(config, ModelSpec) of a model folder: config.json's architecture name picks the
    architecture, which parses the config and builds the spec."""
    d = read_config_json(model_dir)
    archs = d.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError("config.json: 'architectures' must be a non-empty list")
    arch = get_architecture(str(archs[0]))
    config = arch.parse_config(d)
    return config, arch.build_spec(config)


def _ensure_builtin() -> None:
    # The dense decoder registers itself on import.
    from ..models import dense_decoder  # noqa: F401
