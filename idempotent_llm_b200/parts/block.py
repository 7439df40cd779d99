"""Pre-norm residual block: ``h += mixer(norm(h)); h += feed_forward(norm(h))``
(reference: src/detllm/model.py:303-427).  The residual stream stays 32-bit;
each part's output is handed on as a pending delta, which the next norm adds in
the same kernel that norms."""

from __future__ import annotations

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    @classmethod
    def declare(cls, spec, prefix=None):
        p = spec.prefix
        return (NORMS.get(spec.mixer_norm.kind).declare(spec.mixer_norm, p + spec.mixer_norm_prefix)
                + MIXERS.get(spec.mixer.kind).declare(spec.mixer, p)
                + NORMS.get(spec.feed_forward_norm.kind).declare(spec.feed_forward_norm,
                                                                 p + spec.feed_forward_norm_prefix)
                + FEED_FORWARDS.get(spec.feed_forward.kind).declare(spec.feed_forward, p))

    def __init__(self, spec, weights, prefix, rt):
        p = spec.prefix
        self.spec = spec
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, weights, p + spec.mixer_norm_prefix, rt)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, weights, p, rt)
        self.feed_forward_norm = NORMS.get(spec.feed_forward_norm.kind)(
            spec.feed_forward_norm, weights, p + spec.feed_forward_norm_prefix, rt)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, weights, p, rt)

    def emit(self, prog, h, kv, state, writes_cache: bool):
        """The block's calls in a step program; every part must be able to emit its own."""
        from ..kernels.program import NotProgrammable
        parts = (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)
        for part in parts:
            if not hasattr(part, "emit"):
                raise NotProgrammable(f"{type(part).__name__} has no emit")
        x = prog.buffer("block.x", per_token=2 * self.spec.mixer_norm.size)
        self.mixer_norm.emit(prog, h, x)
        self.mixer.emit(prog, x, h, kv, state, writes_cache)
        self.feed_forward_norm.emit(prog, h, x)
        self.feed_forward.emit(prog, x, h)

    def forward(self, h, pending, ctx, kv, state, writes_cache: bool):
        x = self.mixer_norm.forward(h, pending, ctx)
        if getattr(self.mixer, "accepts_residual", False):
            a = self.mixer.forward(x, ctx, kv, state, writes_cache, residual=h)    # None: already added
        else:
            a = self.mixer.forward(x, ctx, kv, state, writes_cache)
        x = self.feed_forward_norm.forward(h, a, ctx)
        if getattr(self.feed_forward, "accepts_residual", False):
            return h, self.feed_forward.forward(x, ctx, residual=h)
        return h, self.feed_forward.forward(x, ctx)
