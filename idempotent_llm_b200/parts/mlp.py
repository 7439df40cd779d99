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
    accepts_residual = True

    @classmethod
    def declare(cls, spec, prefix):
        nm = spec.names
        return [TensorDecl(prefix + nm.gate, (spec.intermediate, spec.hidden)),
                TensorDecl(prefix + nm.up, (spec.intermediate, spec.hidden)),
                TensorDecl(prefix + nm.down, (spec.hidden, spec.intermediate))]

    def __init__(self, spec, weights, prefix, rt):
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not built; only 'silu'")
        self.spec = spec
        self.rt = rt
        nm = spec.names
        gate, up = weights[prefix + nm.gate].to(rt.dtype), weights[prefix + nm.up].to(rt.dtype)
        # with the fused kernels the activation is the epilogue of the gate/up product, which wants
        # gate and up rows interleaved in tiles; otherwise the rows are simply concatenated
        if rt.dtype == torch.bfloat16 and (spec.hidden % 8 or spec.intermediate % 8):
            raise ValueError(f"in bfloat16 the widths of a feed-forward must be multiples of 8 (matrix rows start on "
                             f"16-byte borders); got hidden {spec.hidden}, intermediate {spec.intermediate}")
        self.fused = bool(getattr(rt.kernels, "fused", False))
        if self.fused:
            self.w_gate_up = rt.kernels.tile_gate_up(gate, up)
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = weights[prefix + nm.down].to(rt.dtype).contiguous()

    def emit(self, prog, x, h):
        """The calls of ``forward`` on the fused path, adding into the stream ``h``."""
        from ..kernels.program import NotProgrammable
        if not self.fused:
            raise NotProgrammable("the activation as a kernel of its own is called from forward")
        s = self.spec
        y = prog.buffer("feed_forward.y", per_token=2 * s.intermediate)
        prog.gemm_swiglu(x, self.w_gate_up, s.hidden, s.intermediate, y)
        prog.gemm_residual(y, self.w_down, s.intermediate, h)

    def forward(self, x, ctx, residual=None):
        """Returns the delta ``[P, N, hidden]``, or None after adding it into ``residual`` in place."""
        K = self.rt.kernels
        if self.fused:
            y = K.gemm_swiglu(x, self.w_gate_up, self.spec.intermediate)
            if residual is not None:
                K.gemm_residual(y, self.w_down, residual)
                return None
            return K.gemm(y, self.w_down)
        gu = K.gemm(x, self.w_gate_up)          # [P, N, 2 * intermediate]
        y = K.swiglu(gu)                        # [N, intermediate]
        return K.gemm(y, self.w_down)           # [P, N, hidden]
