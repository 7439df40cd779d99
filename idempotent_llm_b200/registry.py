"""The one registry from an architecture's name (config.json ``architectures[0]``)
to its typed configuration and its model.

The reference has a single hard-wired class and a backend alias table that
raises on unknown names (src/detllm/backends.py:17-34); the same
normalise-or-raise behaviour is kept here for architecture names.

An entry holds the configuration class (``from_dict``, ``to_dict``,
``to_model_spec``) and a builder ``(model_spec, weights, runtime) -> model``.
The default builder assembles the generic decoder from registered parts.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, Optional

from .config.specs import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build_model: Optional[Callable] = None  # None: the generic assembly from parts


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_model: Optional[Callable] = None) -> None:
    for attr in ("from_dict", "to_model_spec"):
        if not hasattr(config_class, attr):
            raise TypeError(f"configuration class for {name!r} lacks {attr}()")
    _ARCHITECTURES[name] = Architecture(name, config_class, build_model)


def architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture {name!r}; registered: {sorted(_ARCHITECTURES)}") from None


def registered_architectures():
    return sorted(_ARCHITECTURES)


def read_config(model_dir: str):
    """Read ``model_dir/config.json`` and return (Architecture, typed configuration)."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path} does not exist")
    with open(path) as f:
        raw = json.load(f)
    archs = raw.get("architectures")
    if not archs:
        raise ConfigError(f"{path}: key 'architectures' is missing or empty")
    arch = architecture(archs[0])
    return arch, arch.config_class.from_dict(raw)


def _register_builtin() -> None:
    from .config.qwen3 import ARCHITECTURE, Qwen3Config
    register_architecture(ARCHITECTURE, Qwen3Config)


_register_builtin()
