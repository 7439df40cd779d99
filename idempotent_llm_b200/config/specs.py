"""Architecture-neutral descriptions of a model: what each layer is made of.

An architecture's typed configuration (for instance ``Qwen3Config``) is
translated once into a ``ModelSpec``.  Everything below the registry (parts,
cache, engine, weights) works from these specs only, so no part knows which
model it is in, and another architecture is another translation.

A spec carries every size and constant its part needs.  The ``kind`` field of
a spec is the key under which the implementing class is registered
(``idempotent_llm_b200.parts.registry``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


class ConfigError(ValueError):
    """A configuration that cannot be built (bad value, missing key)."""


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding.

    Angles are ``position * theta ** (-2 j / dim)`` for ``j < dim / 2``, tiled
    twice (not interleaved); pairs are ``(d, d + dim / 2)``
    (reference: src/detllm/ops/rope.py:25-35, 47-55).  ``variant`` names how the
    rotation sits in a head, which the mixer's kernels must have:
    ``"half_whole_head"`` (``dim`` = the head size, pairs half a head apart) is the
    one built; a partial rotation (``dim`` < head size) or interleaved pairs would
    be other variants, refused by name until a kernel has them.
    """

    theta: float
    dim: int
    max_positions: int
    variant: str = "half_whole_head"
    kind: str = "rotary"


@dataclass(frozen=True)
class NormSpec:
    """Root-mean-square norm over the last axis, weight applied afterwards.
    ``weight``: the tensor's name behind the prefix the block gives the norm."""

    size: int
    eps: float
    weight: str = "weight"
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class AttentionNames:
    """Checkpoint names of an attention layer's tensors, behind the layer's prefix.  An architecture's
    configuration sets them; the part has none of its own."""

    q: str
    k: str
    v: str
    o: str
    q_norm: str
    k_norm: str


@dataclass(frozen=True)
class GatedMLPNames:
    """Checkpoint names of a gated feed-forward's matrices, behind the layer's prefix."""

    gate: str
    up: str
    down: str


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention (a *mixer*).

    ``head_dim`` is free of ``hidden / n_heads``.  ``qk_norm`` applies an
    RMS norm over ``head_dim`` with one weight shared by all heads to q and k
    before the position encoding (reference: src/detllm/model.py:200-216).
    ``window`` of W lets a query at position p see keys p-W+1 .. p; ``None``
    means all keys.  ``kv_from_other`` marks a layer that owns no k/v
    projection and reads the cache another layer wrote.
    """

    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    softmax_scale: float
    qk_norm: bool
    qk_norm_eps: float
    position: Optional[RotarySpec]
    names: AttentionNames
    window: Optional[int] = None
    kv_from_other: bool = False
    kind: str = "attention"


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: ``down(act(gate(x)) * up(x))``
    (reference: src/detllm/model.py:415-427, src/detllm/ops/di_swiglu.py:43-45)."""

    hidden: int
    intermediate: int
    names: GatedMLPNames
    activation: str = "silu"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which block arrangement, and the parts inside it.

    ``prefix`` is the weight-name prefix of the layer (``model.layers.3.``);
    ``mixer_norm_prefix`` / ``feed_forward_norm_prefix`` follow it for the two norms'
    tensors.  ``mixer`` and ``feed_forward`` are specs of any registered kind.
    """

    prefix: str
    mixer: object
    feed_forward: object
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    mixer_norm_prefix: str
    feed_forward_norm_prefix: str
    kind: str = "prenorm"


@dataclass(frozen=True)
class RunEntry:
    """One stop in the order in which layers run.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named twice).
    ``cache`` names the cache entry the mixer uses; entries that share a
    number share keys and values.  ``writes_cache`` is False for a mixer that
    only reads what an earlier entry wrote.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[RunEntry, ...]
    final_norm: NormSpec
    tie_embeddings: bool
    max_positions: int
    embed_name: str                     # checkpoint names: set by the architecture's configuration
    final_norm_prefix: str
    head_name: str
    stop_token_ids: Tuple[int, ...] = ()
    init_std: float = 0.02
    extra: dict = field(default_factory=dict, compare=False)

    def __post_init__(self):
        n = len(self.layers)
        seen_writer = set()
        for e in self.schedule:
            if not 0 <= e.layer < n:
                raise ConfigError(f"schedule names layer {e.layer}, model has {n}")
            if e.writes_cache:
                if e.cache in seen_writer:
                    raise ConfigError(f"cache entry {e.cache} is written by two schedule entries")
                seen_writer.add(e.cache)
            elif e.cache not in seen_writer:
                raise ConfigError(f"schedule entry reads cache {e.cache} before anything wrote it")


def default_schedule(n_layers: int) -> Tuple[RunEntry, ...]:
    """Every layer once, in order, each with a cache entry of its own."""
    return tuple(RunEntry(layer=i, cache=i) for i in range(n_layers))
