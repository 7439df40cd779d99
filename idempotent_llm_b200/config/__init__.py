"""Typed configurations and the architecture-neutral specs they translate to."""

from .specs import (AttentionSpec, ConfigError, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec,
                    RotarySpec, RunEntry, default_schedule)
from .qwen3 import Qwen3Config

__all__ = ["AttentionSpec", "ConfigError", "GatedMLPSpec", "LayerSpec", "ModelSpec", "NormSpec",
           "RotarySpec", "RunEntry", "default_schedule", "Qwen3Config"]
