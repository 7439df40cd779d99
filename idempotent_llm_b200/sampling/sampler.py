"""Choosing the next token from 32-bit logits.

Greedy: the largest logit, the lowest token id among equals -- the reference's
rule (src/detllm/model.py:482-490).  Temperature (the reference has none;
docs/SPEC.md:123 only asks that a sampler be deterministic): the Gumbel-max
form of sampling from softmax(logits / T): ``argmax(logits / T + g_v)`` with
``g_v = -log(-log(u_v))``.  The uniform numbers come from a counter-based
generator keyed by (seed, request, step, token id), so a request's draw does
not depend on which other requests share its batch or on the batch's order.

Generator (all arithmetic modulo 2**64):
    mix(x): x += 0x9E3779B97F4A7C15; x = (x ^ x>>30) * 0xBF58476D1CE4E5B9;
            x = (x ^ x>>27) * 0x94D049BB133111EB; return x ^ x>>31
    row_key = mix(mix(mix(seed) ^ request) ^ step)
    bits_v  = mix(row_key ^ (v * 0xD1342543DE82EF95))
    u_v     = ((bits_v >> 41) + 0.5) / 2**23         (in [2**-24, 1 - 2**-24]: x + 0.5 is exact in
              32-bit only for x < 2**23; with 24 bits the largest x would round up to u = 1)
"""

from __future__ import annotations

from typing import List, Sequence

import torch

_M = (1 << 64) - 1


def mix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M
    return x ^ (x >> 31)


def row_key(seed: int, request: int, step: int) -> int:
    return mix64(mix64(mix64(seed & _M) ^ (request & _M)) ^ (step & _M))


def uniform_from_bits(bits: int) -> float:
    """The uniform number the kernel makes of 64 generator bits, with its 32-bit roundings."""
    import numpy as np
    return float((np.float32(bits >> 41) + np.float32(0.5)) * np.float32(1.0 / 8388608.0))


def _as_i64(x: int) -> int:
    return x - (1 << 64) if x >= (1 << 63) else x


def row_keys(seed: int, request_ids: Sequence[int], steps: Sequence[int]) -> torch.Tensor:
    """The rows' keys as int64 on the host."""
    return torch.tensor([_as_i64(row_key(seed, r, s)) for r, s in zip(request_ids, steps)], dtype=torch.int64)


def sample_tokens(kernels, logits: torch.Tensor, temperature: float, seed: int,
                  request_ids: Sequence[int], steps: Sequence[int]) -> List[int]:
    """One token per row of ``logits`` ``[B, vocab]`` (float32, on the device)."""
    if temperature < 0:
        raise ValueError("temperature must be >= 0")
    B = logits.shape[0]
    if len(request_ids) != B or len(steps) != B:
        raise ValueError("one request id and one step per row")
    keys = None
    if temperature > 0:
        keys = row_keys(seed, request_ids, steps).to(logits.device)
    out = kernels.sample(logits, float(temperature), keys)        # int32 [B] on the device
    return out.tolist()
