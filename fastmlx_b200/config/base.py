"""What every architecture's configuration offers the engine."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Mapping


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine runs."""


@dataclass(frozen=True)
class ModelConfig:
    """Base of the typed configurations.  The engine itself reads only these: the
    vocabulary size (logit width), the longest position (context cap) and the ids that
    end a generation.  Everything else is between a configuration and its builder."""

    @property
    def eos_token_id(self) -> int:  # pragma: no cover - overridden
        return -1

    def to_dict(self) -> dict:  # pragma: no cover - overridden
        raise NotImplementedError


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "rb") as f:
            body = f.read()
    except OSError as e:
        raise ConfigError(f"cannot read {path}: {e.strerror or e}") from None
    return parse_config_json(body)


def parse_config_json(body: bytes | str) -> dict:
    try:
        d = json.loads(body)
    except json.JSONDecodeError as e:
        raise ConfigError(f"decode config: {e}") from None
    if not isinstance(d, Mapping):
        raise ConfigError("decode config: config.json must hold a JSON object")
    return dict(d)
