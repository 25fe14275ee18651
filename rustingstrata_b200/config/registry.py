"""One registry from an architecture's name to its configuration class and model builder.

The reference resolves ``general.architecture`` with a ``match`` that returns a flag
struct and reports the supported names on a miss (src/config.rs:56-87,268).  Here an
architecture registers (a) the names it answers to (``architectures[0]`` and
``model_type`` of config.json), (b) its typed configuration class, (c) a builder that
turns that configuration into a :class:`~rustingstrata_b200.parts.spec.ModelSpec`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Tuple

from .model_config import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    names: Tuple[str, ...]
    config_class: type
    build_spec: Callable[[Any], Any]


_ARCHS: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_spec: Callable, aliases: Tuple[str, ...] = (),
                          *, replace: bool = False) -> Architecture:
    arch = Architecture(name=name, names=(name,) + tuple(aliases), config_class=config_class, build_spec=build_spec)
    for n in arch.names:
        if n in _ARCHS and not replace:
            raise ValueError(f"architecture name '{n}' is already registered")
    for n in arch.names:
        _ARCHS[n] = arch
    return arch


def unregister_architecture(name: str) -> None:
    arch = _ARCHS.get(name)
    if arch:
        for n in arch.names:
            _ARCHS.pop(n, None)


def registered_architectures():
    return sorted(_ARCHS)


def resolve_architecture(config: Mapping[str, Any], where: str = "config.json") -> Architecture:
    """The architecture a config.json names: ``architectures[0]`` first, then ``model_type``."""
    tried = []
    archs = config.get("architectures")
    if isinstance(archs, (list, tuple)):
        tried += [str(a) for a in archs]
    if config.get("model_type") is not None:
        tried.append(str(config["model_type"]))
    for n in tried:
        if n in _ARCHS:
            return _ARCHS[n]
    if not tried:
        raise ConfigError(f"{where}: neither 'architectures' nor 'model_type' names an architecture "
                          f"(registered: {', '.join(registered_architectures())})")
    raise ConfigError(f"{where}: unsupported architecture {', '.join(repr(t) for t in tried)} "
                      f"(registered: {', '.join(registered_architectures())})")


def load_model_config(model_dir: str):
    """(architecture, typed configuration) of a model folder."""
    raw = read_config_json(model_dir)
    arch = resolve_architecture(raw, where=f"{model_dir}/config.json")
    return arch, arch.config_class.from_dict(raw, where=f"{model_dir}/config.json")
