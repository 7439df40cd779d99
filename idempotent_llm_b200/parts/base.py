"""Interfaces of the parts a layer is put together from, and their registries.

Every part is built from its own spec (sizes and constants as parameters), a
dict of weights by checkpoint name, the name prefix of its tensors, and the
``Runtime`` (device, compute dtype, kernels).  No part sees the model's
configuration.  The registries map a spec's ``kind`` to the implementing class;
registering another class under another kind adds a part without touching
this package.

Interfaces (duck-typed; the base classes document them):

* ``Norm.forward(h, delta, ctx, rows=None) -> x``: ``h`` is the 32-bit residual
  stream ``[N, hidden]``; if ``delta`` (32-bit partial sums ``[P, N, hidden]``) is
  given it is added into ``h`` first, in place, in 32-bit; ``x`` is the normed
  result in the compute dtype.  ``rows`` selects token rows (then ``h`` is left
  untouched and only those rows are returned).
* ``Mixer.forward(x, ctx, kv, state, writes_cache) -> delta`` and
  ``Mixer.cache_need(spec) -> CacheNeed``: ``kv`` is the ``KVView`` of the cache
  entry (or None), ``state`` the per-sequence state tensor ``[max_seqs, ...]`` of
  the entry (or None), indexed with ``ctx.slots``.
* ``FeedForward.forward(x, ctx) -> delta``.
* ``PositionEncoding.tables(ctx)``: whatever its mixer kernels need for the
  step's tokens (computed once per step and shared between layers).
* ``Block.forward(h, pending, ctx, kv, state, writes_cache) -> (h, pending)``:
  ``pending`` is a delta not yet added to ``h``; the next norm adds it.

A mixer or feed-forward whose class sets ``accepts_residual = True`` also takes ``residual=h``
and may add its output into ``h`` itself (fused into its last kernel) and return None.

Optional, beside ``forward``: ``emit``.  A part whose kernel calls never change from step to step may
write them down once in a ``StepProgram`` (``kernels/program.py``), which the library then runs for
every step with one call from the host: ``Norm.emit(prog, h, out, rows=False)``,
``Mixer.emit(prog, x, h, kv, state, writes_cache)`` and ``FeedForward.emit(prog, x, h)`` (both add their
output into the stream ``h``), ``PositionEncoding.emit(prog) -> its table's buffers``,
``Block.emit(prog, h, kv, state, writes_cache)``; buffers are the program's, by index.  ``emit`` must
make exactly the calls ``forward`` makes.  A part without it, or one that raises ``NotProgrammable``,
makes its model run call by call from ``forward``: nothing else changes.

``delta`` is always 32-bit ``[P, N, hidden]``: P partial sums whose total is the
part's output (P is 1 unless a matrix product was split along its inner axis);
the consumer adds them in ascending order.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

import torch

from ..cache.spec import CacheNeed
from ..weights.loader import TensorDecl


@dataclass
class Runtime:
    device: torch.device
    dtype: torch.dtype          # compute/storage dtype of activations, weights and cache
    kernels: object             # idempotent_llm_b200.kernels.Kernels (or a stand-in with its methods)


class Part:
    # False for a part that synchronises with the host inside ``forward`` (reads device values):
    # a model with such a part runs its single-token steps without CUDA graphs.
    graph_safe = True

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        return []


class Norm(Part):
    def forward(self, h, delta, ctx, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    def tables(self, ctx):
        raise NotImplementedError


class Mixer(Part):
    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        return CacheNeed()

    def forward(self, x, ctx, kv, state, writes_cache: bool):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx):
        raise NotImplementedError


class Block(Part):
    def forward(self, h, pending, ctx, kv, state, writes_cache: bool):
        raise NotImplementedError


class _Registry:
    def __init__(self, what: str):
        self.what = what
        self._by_kind: Dict[str, type] = {}

    def register(self, kind: str, cls: type = None):
        if cls is None:                       # decorator form
            def deco(c):
                self._by_kind[kind] = c
                return c
            return deco
        self._by_kind[kind] = cls
        return cls

    def get(self, kind: str) -> type:
        try:
            return self._by_kind[kind]
        except KeyError:
            raise KeyError(f"no {self.what} registered under kind {kind!r}; "
                           f"known: {sorted(self._by_kind)}") from None

    def kinds(self):
        return sorted(self._by_kind)


NORMS = _Registry("norm")
POSITIONS = _Registry("position encoding")
MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
BLOCKS = _Registry("block")
