"""Rotary position encoding: the step's cos/sin table.

``inv_freq_j = theta ** (-2 j / dim)`` in 64-bit, angle = position * inv_freq in
64-bit, cos and sin rounded to 32-bit (reference: src/detllm/ops/rope.py:25-35
builds its table the same way before quantising it; float form in
src/detllm/prepare.py:137-141).  The table is made once per step and shared by
every layer with the same ``(theta, dim)``; the rotation itself is fused into
the mixer's kernel.
"""

from __future__ import annotations

import torch

from .base import POSITIONS, PositionEncoding


@POSITIONS.register("rotary")
class Rotary(PositionEncoding):
    def __init__(self, spec, weights, prefix, rt):
        if spec.dim % 2:
            raise ValueError(f"rotary dimension {spec.dim} must be even")
        self.spec = spec
        self.rt = rt
        j = torch.arange(0, spec.dim // 2, dtype=torch.float64)
        self.inv_freq = (float(spec.theta) ** (-2.0 * j / spec.dim)).to(rt.device)

    def emit(self, prog):
        """The table's two buffers in a step program (made once a step, like ``tables``)."""
        key = ("rotary", float(self.spec.theta), self.spec.dim)
        bufs = prog.shared.get(key)
        if bufs is None:
            per_token = self.spec.dim // 2 * 2 * 4
            bufs = prog.shared[key] = (prog.buffer(f"rotary.{len(prog.shared)}", per_token),
                                       prog.buffer(f"rotary.{len(prog.shared)}.by_dim", per_token))
            prog.rope_table(self.inv_freq, *bufs)
        return bufs

    def tables(self, ctx):
        key = ("rotary", float(self.spec.theta), self.spec.dim)
        t = ctx.memo.get(key)
        if t is None:
            t = self.rt.kernels.rope_table(ctx.positions, self.inv_freq)
            ctx.memo[key] = t
        return t
