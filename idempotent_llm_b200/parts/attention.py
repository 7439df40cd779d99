"""Causal grouped-query attention over the sequence cache (a mixer).

Order of operations as the reference runs them (src/detllm/model.py:303-412):
q/k/v projections without bias; per (token, head) RMS norm over head_dim with
one weight of shape [head_dim] shared by all heads (model.py:200-216); rotary
encoding after the norm; k and v written once into the cache (model.py:338-343);
scores q.k / sqrt(head_dim) of q-head h against kv-head h // group
(model.py:170; ops/fused_attn.py:60); softmax over the allowed keys, masked keys
contributing exactly nothing (ops/di_softmax.py:41-61); context; heads merged
as channel = head * head_dim + d (model.py:170-172); output projection.
The three projections are one matrix here (rows concatenated; no dot product
changes).
"""

from __future__ import annotations

import torch

from ..cache.spec import CacheNeed
from ..weights.loader import TensorDecl
from .base import MIXERS, POSITIONS, Mixer


@MIXERS.register("attention")
class GQAAttention(Mixer):
    accepts_residual = True

    @classmethod
    def declare(cls, spec, prefix):
        nm = spec.names
        q_rows, kv_rows = spec.n_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim
        d = [TensorDecl(prefix + nm.q, (q_rows, spec.hidden))]
        if not spec.kv_from_other:
            d += [TensorDecl(prefix + nm.k, (kv_rows, spec.hidden)),
                  TensorDecl(prefix + nm.v, (kv_rows, spec.hidden))]
        d.append(TensorDecl(prefix + nm.o, (spec.hidden, q_rows)))
        if spec.qk_norm:
            d.append(TensorDecl(prefix + nm.q_norm, (spec.head_dim,), init="one_plus_normal"))
            if not spec.kv_from_other:
                d.append(TensorDecl(prefix + nm.k_norm, (spec.head_dim,), init="one_plus_normal"))
        return d

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        return CacheNeed(kind="window" if spec.window else "full", n_kv_heads=spec.n_kv_heads,
                         head_dim=spec.head_dim, window=spec.window)

    def __init__(self, spec, weights, prefix, rt):
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if rt.dtype == torch.bfloat16 and (spec.hidden % 8 or (spec.n_heads * spec.head_dim) % 8):
            raise ValueError(f"in bfloat16 the widths of an attention layer must be multiples of 8 (matrix rows start "
                             f"on 16-byte borders); got hidden {spec.hidden}, heads x head_dim {spec.n_heads * spec.head_dim}")
        self.spec = spec
        self.rt = rt
        nm = spec.names
        mats = [weights[prefix + nm.q]]
        if not spec.kv_from_other:
            mats += [weights[prefix + nm.k], weights[prefix + nm.v]]
        self.w_qkv = torch.cat([m.to(rt.dtype) for m in mats], dim=0).contiguous()
        self.w_o = weights[prefix + nm.o].to(rt.dtype).contiguous()
        self.q_gamma = self.k_gamma = None
        if spec.qk_norm:
            self.q_gamma = weights[prefix + nm.q_norm].to(torch.float32).contiguous()
            if not spec.kv_from_other:
                self.k_gamma = weights[prefix + nm.k_norm].to(torch.float32).contiguous()
        if spec.kv_from_other and spec.window:
            raise ValueError("a mixer that reads another layer's windowed cache is not built: a prompt's "
                             "own keys are not all in the ring")
        self.position = None
        if spec.position is not None:
            # what this mixer's kernels do with a position encoding's table: rotate pairs half a head apart
            # over the whole head.  Another arrangement is refused by name, not by a shape error later.
            variant = getattr(spec.position, "variant", None)
            if variant != "half_whole_head" or getattr(spec.position, "dim", spec.head_dim) != spec.head_dim:
                raise ValueError(f"attention: position encoding variant {variant!r} over "
                                 f"{getattr(spec.position, 'dim', '?')} of {spec.head_dim} dims is not built; the kernels "
                                 f"rotate pairs (d, d + head_dim / 2) over the whole head ('half_whole_head')")
            self.position = POSITIONS.get(spec.position.kind)(spec.position, weights, prefix, rt)

    def emit(self, prog, x, h, kv, state, writes_cache: bool):
        """The calls of ``forward`` on the fused path without a window, adding into the stream ``h``."""
        from ..kernels.program import NotProgrammable
        s = self.spec
        if writes_cache == s.kv_from_other:
            raise ValueError("a mixer with its own k/v must write its cache entry; one without must not")
        if s.window or kv.ring:
            raise NotProgrammable("a windowed layer reads a prompt's own keys from buffers of the step")
        cs = self.position.emit(prog) if self.position is not None else None
        width = s.n_heads * s.head_dim
        q = prog.buffer("attention.q", per_token=2 * width)
        prog.gemm_qkv(x, self.w_qkv, s.hidden, s.n_heads, 0 if s.kv_from_other else s.n_kv_heads, s.head_dim,
                      self.q_gamma, self.k_gamma, s.qk_norm_eps, cs, q, kv if writes_cache else None)
        o = prog.buffer("attention.o", per_token=2 * width)
        prog.attention(q, kv, s.n_heads, s.softmax_scale, o)
        prog.gemm_residual(o, self.w_o, width, h)

    def forward(self, x, ctx, kv, state, writes_cache: bool, residual=None):
        """Returns the delta ``[P, N, hidden]``, or None after adding it into ``residual`` in place."""
        s, K = self.spec, self.rt.kernels
        if writes_cache == s.kv_from_other:
            raise ValueError("a mixer with its own k/v must write its cache entry; one without must not")
        cs = self.position.tables(ctx) if self.position is not None else None
        fused = bool(getattr(K, "fused", False))
        # A windowed layer's ring cannot hold a whole prompt, so a step of several tokens reads its
        # own keys from packed buffers and writes the ring afterwards.  A single token overwrites
        # position p - ring only, which lies outside its window, so it is written first like any key.
        windowed = kv.ring > 0 and not ctx.single_token
        finish = (s.n_heads, 0 if s.kv_from_other else s.n_kv_heads, s.head_dim, self.q_gamma, self.k_gamma,
                  s.qk_norm_eps, cs, ctx, kv if (writes_cache and not windowed) else None)
        if fused and s.head_dim in K.QKV_FUSED_HEAD_DIMS:
            # norm, rotation and the cache write are the epilogue of the projection
            q, k_new, v_new = K.gemm_qkv(x, self.w_qkv, *finish, keep_new=writes_cache and windowed)
        else:
            qkv = K.gemm(x, self.w_qkv)                                   # [1, N, (n_q [+ 2 n_kv]) * hd]
            q, k_new, v_new = K.qkv_finish(qkv, *finish, keep_new=writes_cache and windowed)
        o = K.attention(q, kv, ctx, k_new, v_new, s.softmax_scale, s.window)  # [N, n_q * hd]
        if writes_cache and windowed:
            K.kv_write_ring(k_new, v_new, kv, ctx)
        if fused and residual is not None:
            K.gemm_residual(o, self.w_o, residual)
            return None
        return K.gemm(o, self.w_o)                                    # [P, N, hidden]
