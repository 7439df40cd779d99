"""Named configurations shipped as config.json files (data, not code): the three Qwen3
sizes the benchmarks quote and two tiny ones that differ in every size and option."""

from __future__ import annotations

import json
import os

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "presets")


def preset_names():
    return sorted(f[:-5] for f in os.listdir(_DIR) if f.endswith(".json"))


def preset_dict(name: str) -> dict:
    path = os.path.join(_DIR, name.lower() + ".json")
    if not os.path.isfile(path):
        raise ValueError(f"unknown preset {name!r}; known: {preset_names()}")
    with open(path) as f:
        return json.load(f)


def preset(name: str, **overrides):
    """The typed configuration of a preset, through the registry like any config.json."""
    from ..registry import architecture
    d = preset_dict(name)
    d.update(overrides)
    return architecture(d["architectures"][0]).config_class.from_dict(d)
