"""idempotent_llm_b200: a small, whole, single-GPU model library for the Qwen3 dense
decoder on NVIDIA B200 (sm_100a): configuration and registry, weights by name, layers
from parts, a paged sequence cache, one step function, a generation loop, sampling,
trace replay, and hand-written CUDA kernels in bfloat16 and in true 32-bit."""

from .api import LM, build_model, canonical_dtype, from_random, load
from .config import ConfigError, Qwen3Config
from .registry import read_config, register_architecture, registered_architectures

__all__ = ["LM", "build_model", "canonical_dtype", "from_random", "load", "ConfigError", "Qwen3Config",
           "read_config", "register_architecture", "registered_architectures"]
__version__ = "0.1.0"
