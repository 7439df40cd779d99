"""From a ModelSpec to (a) the tensors the model declares and (b) the model.

The generic decoder: token embedding, the schedule of blocks, final norm and
head, as the reference's step runs them (src/detllm/model.py:233-286), except
that logits are computed only for the rows that are asked for.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.spec import CacheNeed
from ..config.specs import ModelSpec
from ..parts.base import BLOCKS, MIXERS, NORMS, Runtime
from ..weights.loader import TensorDecl


def declare_weights(spec: ModelSpec) -> List[TensorDecl]:
    decls = [TensorDecl(spec.embed_name, (spec.vocab_size, spec.hidden))]
    for layer in spec.layers:
        decls += BLOCKS.get(layer.kind).declare(layer)
    decls += NORMS.get(spec.final_norm.kind).declare(spec.final_norm, spec.final_norm_prefix)
    # tied: an lm_head in the file is tolerated and ignored; untied: it is required
    decls.append(TensorDecl(spec.head_name, (spec.vocab_size, spec.hidden), optional=spec.tie_embeddings))
    seen = set()
    for d in decls:
        if d.name in seen:
            raise ValueError(f"tensor {d.name} is declared twice")
        seen.add(d.name)
    return decls


def cache_needs(spec: ModelSpec) -> Dict[int, CacheNeed]:
    """cache id -> need, from the mixer of the schedule entry that writes it."""
    needs: Dict[int, CacheNeed] = {}
    for e in spec.schedule:
        need = MIXERS.get(spec.layers[e.layer].mixer.kind).cache_need(spec.layers[e.layer].mixer)
        if e.writes_cache:
            needs[e.cache] = need
    return needs


class CausalLM:
    """Embedding -> blocks in schedule order -> final norm -> head."""

    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.embed = weights[spec.embed_name].to(rt.dtype).contiguous()
        if spec.tie_embeddings:
            self.head = self.embed
        else:
            self.head = weights[spec.head_name].to(rt.dtype).contiguous()
        self.blocks = [BLOCKS.get(layer.kind)(layer, weights, layer.prefix, rt) for layer in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, weights,
                                                          spec.final_norm_prefix, rt)
        self._programs = {}
        self.graph_safe = all(getattr(part, "graph_safe", True) for b in self.blocks
                              for part in vars(b).values())

    def program(self, cache):
        """The model's kernel calls over ``cache`` as a step program (``kernels/program.py``), made once; None
        if a part cannot emit its calls, the kernels hold no programs (32-bit; separate epilogues), or a
        stand-in for the kernels has none."""
        key = id(cache)
        if key not in self._programs:
            self._programs[key] = (cache, self._emit(cache))   # (the cache is kept: its id stays its own)
        return self._programs[key][1]

    def _emit(self, cache):
        K = self.rt.kernels
        if not hasattr(K, "use_programs"):
            return None
        from ..kernels.program import NotProgrammable, StepProgram
        hidden = self.spec.hidden
        try:
            prog = StepProgram(K)
            h = prog.buffer("stream", per_token=4 * hidden)
            prog.embed(self.embed, h)
            for e in self.spec.schedule:
                block = self.blocks[e.layer]
                state = cache.state_of(e.cache)
                if not hasattr(block, "emit") or (state is not None and state.numel()):
                    raise NotProgrammable("a block without emit, or with per-sequence state")
                block.emit(prog, h, cache.view(e.cache), state, e.writes_cache)
            if not hasattr(self.final_norm, "emit"):
                raise NotProgrammable("the final norm has no emit")
            x = prog.buffer("head.x", per_row=2 * hidden)
            self.final_norm.emit(prog, h, x, rows=True)
            logits = prog.buffer("logits")
            prog.gemm_store(x, self.head, hidden, logits, rows=True)
            return prog.finish(logits, self.head.shape[0])
        except NotProgrammable:
            return None

    def forward(self, ctx, cache, want_rows: torch.Tensor) -> torch.Tensor:
        """Run the step's tokens; returns 32-bit logits ``[len(want_rows), vocab]``."""
        K = self.rt.kernels
        if getattr(K, "use_programs", False):
            prog = self.program(cache)
            if prog is not None:
                return prog.run(ctx, want_rows)
        h = K.embed(ctx.tokens, self.embed)
        pending = None
        for e in self.spec.schedule:
            h, pending = self.blocks[e.layer].forward(h, pending, ctx, cache.view(e.cache),
                                                      cache.state_of(e.cache), e.writes_cache)
        x = self.final_norm.forward(h, pending, ctx, rows=want_rows)
        return K.gemm_store(x, self.head)

    def weight_bytes(self) -> int:
        seen, n = set(), 0

        def add(t):
            nonlocal n
            if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                n += t.numel() * t.element_size()

        def walk(o, depth=0):
            if isinstance(o, torch.Tensor):
                add(o)
            elif depth < 4 and hasattr(o, "__dict__"):
                for k, v in vars(o).items():
                    if k in ("rt", "spec"):
                        continue
                    if isinstance(v, (list, tuple)):
                        for i in v:
                            walk(i, depth + 1)
                    else:
                        walk(v, depth + 1)
        walk(self)
        return n
