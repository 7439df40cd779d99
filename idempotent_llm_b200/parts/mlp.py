"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))``, no bias
(reference: src/detllm/model.py:415-427; float form ``g * sigmoid(g) * u`` in
tests/test_ops.py:240-242 and scripts/attribute_error.py:37-40).  Gate and up
are one matrix here (rows concatenated)."""

from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import FEED_FORWARDS, FeedForward


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    @classmethod
    def declare(cls, spec, prefix):
        p = prefix + "mlp."
        return [TensorDecl(p + "gate_proj.weight", (spec.intermediate, spec.hidden)),
                TensorDecl(p + "up_proj.weight", (spec.intermediate, spec.hidden)),
                TensorDecl(p + "down_proj.weight", (spec.hidden, spec.intermediate))]

    def __init__(self, spec, weights, prefix, rt):
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not built; only 'silu'")
        self.spec = spec
        self.rt = rt
        p = prefix + "mlp."
        self.w_gate_up = torch.cat([weights[p + "gate_proj.weight"].to(rt.dtype),
                                    weights[p + "up_proj.weight"].to(rt.dtype)], dim=0).contiguous()
        self.w_down = weights[p + "down_proj.weight"].to(rt.dtype).contiguous()

    def forward(self, x, ctx):
        K = self.rt.kernels
        gu = K.gemm(x, self.w_gate_up)          # [P, N, 2 * intermediate]
        y = K.swiglu(gu)                        # [N, intermediate]
        return K.gemm(y, self.w_down)           # [P, N, hidden]
