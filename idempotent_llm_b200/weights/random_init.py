"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed.  The reference has no such mode (its benchmark uses
random *ids* on the real checkpoint, scripts/bench.py:25-26); here every tensor
is drawn from a generator seeded by (seed, tensor name), so a tensor's values do
not depend on which other tensors exist or on the order they are made in.
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Sequence

import torch

from .loader import TensorDecl
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def draw(decl: TensorDecl, seed: int, std: float, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, decl.name))
    t = torch.randn(decl.shape, generator=g, dtype=torch.float32, device=device) * std
    if decl.init == "one_plus_normal":
        t = t + 1.0
    elif decl.init != "normal":
        raise ValueError(f"unknown init {decl.init!r} for {decl.name}")
    return t.to(dtype)


def random_weights(decls: Sequence[TensorDecl], seed: int, std: float, dtype=torch.bfloat16,
                   device="cpu") -> Dict[str, torch.Tensor]:
    """In-memory random tensors (used for layer sizes too large to write to disk first)."""
    return {d.name: draw(d, seed, std, dtype, device) for d in decls if not d.optional}


def write_random_model(config, out_dir: str, seed: int = 0, dtype=torch.bfloat16, std=None) -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors`` for a typed configuration."""
    from ..engine.assembly import declare_weights
    spec = config.to_model_spec()
    std = spec.init_std if std is None else std
    os.makedirs(out_dir, exist_ok=True)
    d = config.to_dict()
    d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}.get(dtype, str(dtype))
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(d, f, indent=1)
    tensors = [(decl.name, draw(decl, seed, std, dtype)) for decl in declare_weights(spec) if not decl.optional]
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed, "std": std})
    return out_dir
