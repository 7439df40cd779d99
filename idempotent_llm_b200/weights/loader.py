"""Weights by tensor name.

What a model needs is the list of ``TensorDecl`` its parts declare; what a
folder holds is read from its safetensors header.  The two are compared
before any tensor is moved, and every disagreement (missing, unexpected,
wrong shape) is reported in ONE error.  The reference asserts dtype per tensor
while loading its artifact (src/detllm/model.py:116-119) and names the
checkpoint's tensors in src/detllm/prepare.py:323-384.

Storage policy: bfloat16 stays bfloat16, a tensor stored in 32-bit floating point
stays 32-bit, float16 is widened to 32-bit (exact; narrowing it to bfloat16 here
would drop three bits even on the 32-bit path), integer tables become int32.  The
parts decide afterwards what the compute path needs (matrices in the compute
dtype, norm weights in 32-bit).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsDir


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part needs: checkpoint name, shape, and how random init draws it
    (``normal``: N(0, std); ``one_plus_normal``: 1 + N(0, std), for norm weights)."""

    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    optional: bool = False   # present-or-absent both fine (an lm_head beside tied embeddings)


class WeightError(ValueError):
    """The folder's tensors do not match what the model declares."""

    def __init__(self, where, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = [f"weights in {where} do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {dt}" for n, dt in self.wrong_dtype))
        super().__init__("\n".join(lines))


def storage_dtype(dt: torch.dtype) -> torch.dtype:
    if dt == torch.bfloat16:
        return torch.bfloat16
    if dt in (torch.float16, torch.float32, torch.float64):
        return torch.float32
    return torch.int32


def check_declared(where: str, decls: Sequence[TensorDecl], have: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]]):
    want = {d.name: d for d in decls}
    missing = [n for n, d in want.items() if n not in have and not d.optional]
    unexpected = [n for n in have if n not in want]
    wrong_shape, wrong_dtype = [], []
    for n, d in want.items():
        if n in have:
            dt, shape = have[n]
            if tuple(shape) != tuple(d.shape):
                wrong_shape.append((n, tuple(shape), tuple(d.shape)))
            if not isinstance(dt, torch.dtype) or not dt.is_floating_point:
                wrong_dtype.append((n, dt))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(where, missing, unexpected, wrong_shape, wrong_dtype)


def load_weights(model_dir: str, decls: Sequence[TensorDecl], device) -> Dict[str, torch.Tensor]:
    """Read every declared tensor from ``model_dir`` onto ``device`` (tensor by tensor)."""
    src = SafetensorsDir(model_dir)
    have = {n: src.info(n) for n in src.names()}
    check_declared(model_dir, decls, have)
    for d in decls:
        if d.optional and d.name in have:
            import warnings
            warnings.warn(f"{model_dir}: {d.name} is in the file but the model does not use it "
                          f"(tied embeddings): ignored", stacklevel=2)
    out = {}
    for d in decls:
        if d.name not in have or d.optional:
            continue
        t = src.get(d.name)
        out[d.name] = t.to(device=device, dtype=storage_dtype(t.dtype), copy=True)
    return out
