"""One registry from an architecture's name to its configuration class and builder.

tamnd/fastmlx dispatches on config.json's `model_type` alone through a map of builders
(compute/models/registry.go:26-128) and names the unknown type in its error.  Here the
`architectures` strings are keys too, so "llama" and "LlamaForCausalLM" reach the same
entry.  A new architecture is one `register` call; nothing else in the engine changes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Mapping

from .config.base import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping], ModelConfig]
    build: Callable[[ModelConfig], "object"]      # -> parts.model.Model (unbound weights)


_BY_NAME: dict[str, Architecture] = {}


def register(names, parse_config, build, *, replace: bool = False) -> Architecture:
    """Register an architecture under its model_type and architectures strings."""
    if isinstance(names, str):
        names = [names]
    arch = Architecture(names[0], parse_config, build)
    for n in names:
        if n in _BY_NAME and not replace:
            raise ValueError(f"models: {n!r} is already registered")
        _BY_NAME[n] = arch
    return arch


def unregister(names) -> None:
    if isinstance(names, str):
        names = [names]
    for n in names:
        _BY_NAME.pop(n, None)


def registered_model_types() -> list[str]:
    """Sorted names (compute/models/registry.go:133-140)."""
    return sorted(_BY_NAME)


def resolve(config: Mapping) -> Architecture:
    """The architecture that config.json names: `model_type` first, then each entry of
    `architectures`."""
    mt = config.get("model_type")
    archs = config.get("architectures") or []
    if not mt and not archs:
        raise ConfigError("models: config has no model_type")
    for key in ([mt] if mt else []) + list(archs):
        if key in _BY_NAME:
            return _BY_NAME[key]
    raise ConfigError(f"models: unsupported model_type {mt!r} (architectures {list(archs)!r}); "
                      f"registered: {registered_model_types()}")


def build_model(config: Mapping):
    """config.json dict -> (typed configuration, unbound model)."""
    arch = resolve(config)
    cfg = arch.parse_config(config)
    return cfg, arch.build(cfg)
