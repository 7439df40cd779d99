"""Model assembly, the step function, the generation loop, trace replay."""

from .assembly import CausalLM, cache_needs, declare_weights
from .batch import StepContext
from .engine import Engine
from .generate import GenerationResult, generate, plan_batches

__all__ = ["CausalLM", "cache_needs", "declare_weights", "StepContext", "Engine", "GenerationResult",
           "generate", "plan_batches"]
