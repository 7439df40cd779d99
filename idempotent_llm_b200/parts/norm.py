"""RMS norm: ``x / sqrt(mean(x^2) + eps) * weight``, all in 32-bit.

The reference's float form is ``x / sqrt(mean(x^2))`` (tests/test_ops.py:198-199,
scripts/attribute_error.py:48-51) with the weight folded into the consumer
(src/detllm/prepare.py:342-343); its integer runtime clamps instead of adding
eps (src/detllm/ops/di_rmsnorm.py:14, 50).  Here eps is added to the mean
inside the square root and the weight multiplies afterwards.
"""

from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import NORMS, Norm


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    @classmethod
    def declare(cls, spec, prefix):
        return [TensorDecl(prefix + spec.weight, (spec.size,), init="one_plus_normal")]

    def __init__(self, spec, weights, prefix, rt):
        self.spec = spec
        self.rt = rt
        self.weight = weights[prefix + spec.weight].to(torch.float32).contiguous()

    def forward(self, h, delta, ctx, rows=None):
        return self.rt.kernels.add_rmsnorm(h, delta, self.weight, self.spec.eps, rows=rows)

    def emit(self, prog, h, out, rows=False):
        prog.add_rmsnorm(h, self.weight, self.spec.eps, out, self.spec.size, rows=rows)
