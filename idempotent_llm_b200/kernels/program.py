"""A step of a model as data, run by one call into the library (``csrc/step_program.cu``).

A model's parts *emit* their kernel calls once (``StepProgram.add_rmsnorm``, ``gemm_qkv``, ...: the calls
``Kernels`` would make, with the same checks on what never changes: weights, sizes, cache entries); a
step then hands the library its packed tokens, the addresses of its buffers and the plan of its
attention tiles, and the library makes the calls.  Buffers are named; a name stands for one region of
the step's workspace, sized by the step's tokens (or wanted rows), so a part says which of its
temporaries may share memory by giving them the same name in every layer.

Only what the fused bfloat16 kernels cover can be emitted; a part that cannot (a window, a head size
without a fused kernel, state of its own) raises ``NotProgrammable`` or has no ``emit`` at all, and its
model runs call by call as before.  The two ways give the same bits (tested): the kernels and their
arguments are the same.

The reference runs its layers from Python and replays single-token steps from a captured graph
(src/detllm/graphed.py:43-73); it has nothing like this for prompts.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Dict, List, Optional, Tuple

import torch

OP_INTS, OP_FLOATS, OP_POINTERS = 10, 2, 6
MAX_BUFFERS, MAX_PLANS = 16, 4

EMBED, ROPE_TABLE, ADD_RMSNORM, GEMM_QKV, ATTENTION, GEMM_RESIDUAL, GEMM_SWIGLU, GEMM_STORE = range(8)


class NotProgrammable(Exception):
    """A part has no call sequence that the library can run by itself."""


class IdmOp(ctypes.Structure):
    _fields_ = [("kind", c_int), ("i", c_int * OP_INTS), ("f", c_float * OP_FLOATS), ("pad", c_int),
                ("p", c_void_p * OP_POINTERS)]


class IdmAttnPlan(ctypes.Structure):
    _fields_ = [("tile_seq", c_void_p), ("tile_start", c_void_p), ("tile_pool", c_void_p), ("scratch", c_void_p),
                ("n_tiles", c_int), ("rows_cap", c_int), ("max_runs", c_int), ("max_parts", c_int),
                ("runs_per_part", c_int), ("run_blocks", c_int)]


class IdmStep(ctypes.Structure):
    _fields_ = [("tokens", c_void_p), ("token_seq", c_void_p), ("positions", c_void_p), ("cu_q", c_void_p),
                ("slots", c_void_p), ("q_start", c_void_p), ("kv_len", c_void_p), ("rows", c_void_p),
                ("buf", c_void_p * MAX_BUFFERS), ("attn", IdmAttnPlan * MAX_PLANS),
                ("n_tokens", c_int), ("n_rows", c_int), ("launches", c_int), ("failed_op", c_int)]


def layout() -> List[int]:
    """Sizes and offsets of the records as this file defines them, in the order of ``idm_program_layout``."""
    return [ctypes.sizeof(IdmOp), IdmOp.i.offset, IdmOp.f.offset, IdmOp.p.offset,
            ctypes.sizeof(IdmAttnPlan), IdmAttnPlan.n_tiles.offset,
            ctypes.sizeof(IdmStep), IdmStep.buf.offset, IdmStep.attn.offset, IdmStep.n_tokens.offset,
            MAX_BUFFERS, MAX_PLANS]


def _align(n: int) -> int:
    return (n + 255) // 256 * 256


class StepProgram:
    def __init__(self, kernels):
        K = kernels
        if K.dtype != torch.bfloat16 or not K.fused or K.attention_impl != "tcgen05":
            raise NotProgrammable("step programs hold the fused bfloat16 kernels only")
        self.K = K
        self._ops: List[IdmOp] = []
        self._buffers: Dict[str, List[int]] = {}      # name -> [index, bytes per token, bytes per wanted row]
        self._plans: List[Tuple[int, int, int]] = []  # (q heads, kv heads, head size) of the attention calls
        self._keep: List[torch.Tensor] = []           # what the calls point at
        self._output: Optional[Tuple[int, int]] = None
        self.shared: Dict = {}                        # what parts make once for the whole program (position tables)
        self._array = None
        self._step = IdmStep()

    # ------------------------------------------------------------------ building
    def buffer(self, name: str, per_token: int = 0, per_row: int = 0) -> int:
        """The index of the step buffer ``name`` with room for that many bytes per token of the step (and per
        wanted row); asked for again, the same buffer, grown to the larger need."""
        b = self._buffers.get(name)
        if b is None:
            if len(self._buffers) == MAX_BUFFERS:
                raise NotProgrammable(f"a step program has {MAX_BUFFERS} buffers at most")
            b = self._buffers[name] = [len(self._buffers), 0, 0]
        b[1], b[2] = max(b[1], int(per_token)), max(b[2], int(per_row))
        return b[0]

    def _ptr(self, t: Optional[torch.Tensor], dtype, what: str) -> Optional[int]:
        if t is None:
            return None
        self.K._need(t, dtype, what)
        self._keep.append(t)
        return t.data_ptr()

    def _op(self, kind: int, ints=(), floats=(), ptrs=()) -> None:
        if self._array is not None:
            raise RuntimeError("the program is finished")
        op = IdmOp()
        op.kind = kind
        for k, v in enumerate(ints):
            op.i[k] = int(v)
        for k, v in enumerate(floats):
            op.f[k] = float(v)
        for k, v in enumerate(ptrs):
            op.p[k] = v
        self._ops.append(op)

    def embed(self, table: torch.Tensor, out: int) -> None:
        """``out`` (32-bit rows of ``table``'s width) <- the rows of the step's tokens."""
        self._op(EMBED, (table.shape[1], out), (), (self._ptr(table, self.K.dtype, "embed table"),))

    def rope_table(self, inv_freq: torch.Tensor, cs: int, by_dim: int) -> None:
        self._op(ROPE_TABLE, (inv_freq.numel(), cs, by_dim), (), (self._ptr(inv_freq, torch.float64, "inv_freq"),))

    def add_rmsnorm(self, h: int, gamma: torch.Tensor, eps: float, out: int, hidden: int, rows: bool = False) -> None:
        """``out`` <- norm of the residual stream ``h`` (of the step's wanted rows only, if ``rows``)."""
        if gamma.numel() != hidden:
            raise ValueError(f"norm weight has {gamma.numel()} elements, rows have {hidden}")
        self._op(ADD_RMSNORM, (hidden, h, out, 1 if rows else 0), (eps,),
                 (self._ptr(gamma, torch.float32, "norm weight"),))

    def _weight(self, w: torch.Tensor, inner: int, what: str) -> int:
        if w.dim() != 2 or w.shape[1] != inner:
            raise ValueError(f"{what}: weight {tuple(w.shape)} does not have rows of {inner}")
        if inner % 8:
            raise ValueError(f"{what}: the inner size {inner} must be a multiple of 8 in bfloat16")
        return self._ptr(w, self.K.dtype, what)

    def gemm_qkv(self, x: int, w: torch.Tensor, inner: int, n_q: int, n_kv: int, hd: int, q_gamma, k_gamma, eps: float,
                 cs: Optional[Tuple[int, int]], q: int, kv) -> None:
        """The fused q/k/v projection of ``x`` [tokens, inner]: q to the buffer ``q``, k and v into the cache
        entry ``kv`` (None: this mixer has no keys of its own); ``cs``: the rotary table's two buffers."""
        K = self.K
        if hd not in K.QKV_FUSED_HEAD_DIMS:
            raise NotProgrammable(f"no fused q/k/v projection for head size {hd}")
        if w.shape[0] != (n_q + 2 * n_kv) * hd:
            raise ValueError(f"gemm_qkv: weight rows {w.shape[0]}, heads {(n_q, n_kv)}, head_dim {hd}")
        for g in (q_gamma, k_gamma):
            if g is not None and g.numel() != hd:
                raise ValueError("q/k norm weight must have head_dim elements")
        if kv is not None:
            if kv.ring:
                raise NotProgrammable("a windowed cache entry is written call by call")
            K._check_kv(kv, n_kv, hd)
            self._keep += [kv.k, kv.v, kv.table]
        self._op(GEMM_QKV,
                 (inner, n_q, n_kv, hd, x, q, cs[0] if cs else -1, cs[1] if cs else -1,
                  kv.table.shape[1] if kv is not None else 0, 0),
                 (eps,),
                 (self._weight(w, inner, "q/k/v weight"), self._ptr(q_gamma, torch.float32, "q norm weight"),
                  self._ptr(k_gamma, torch.float32, "k norm weight"),
                  kv.k.data_ptr() if kv is not None else None, kv.v.data_ptr() if kv is not None else None,
                  kv.table.data_ptr() if kv is not None else None))

    def attention(self, q: int, kv, n_q: int, scale: float, out: int) -> None:
        """``out`` [tokens, n_q * hd] <- causal attention of ``q`` over the cache entry ``kv``."""
        K = self.K
        hd, n_kv = kv.head_dim, kv.n_kv_heads
        if kv.ring or kv.window or not K.lib.idm_attention_tc_supports(hd):
            raise NotProgrammable("only the tensor-core attention (head sizes 64 and 128, no window) is in step programs")
        K._check_kv(kv, n_kv, hd)
        key = (n_q, n_kv, hd)
        if key not in self._plans:
            if len(self._plans) == MAX_PLANS:
                raise NotProgrammable(f"a step program has {MAX_PLANS} arrangements of attention heads at most")
            self._plans.append(key)
        self._keep += [kv.k, kv.v, kv.table]
        self._op(ATTENTION, (kv.k.shape[0], kv.table.shape[1], n_q, n_kv, hd, q, out, self._plans.index(key)),
                 (scale,), (kv.k.data_ptr(), kv.v.data_ptr(), kv.table.data_ptr()))

    def gemm_residual(self, x: int, w: torch.Tensor, inner: int, h: int) -> None:
        """``h`` += ``x`` [tokens, inner] . w^T in 32-bit."""
        self._op(GEMM_RESIDUAL, (w.shape[0], inner, x, h), (), (self._weight(w, inner, "weight"),))

    def gemm_swiglu(self, x: int, w_tiled: torch.Tensor, inner: int, inter: int, out: int) -> None:
        """``out`` [tokens, inter] <- silu(gate) * up of ``x`` . (tiled gate/up rows)^T."""
        if w_tiled.shape[0] != -(-inter // 64) * 128:
            raise ValueError(f"tiled gate/up weight has {w_tiled.shape[0]} rows, expected {-(-inter // 64) * 128}")
        self._op(GEMM_SWIGLU, (inter, inner, x, out), (), (self._weight(w_tiled, inner, "gate/up weight"),))

    def gemm_store(self, x: int, w: torch.Tensor, inner: int, out: int, rows: bool = False) -> None:
        """``out`` <- ``x`` . w^T in 32-bit (``rows``: x holds the step's wanted rows, not its tokens)."""
        self._op(GEMM_STORE, (w.shape[0], inner, x, out, 1 if rows else 0), (), (self._weight(w, inner, "weight"),))

    def finish(self, output: int, output_width: int) -> "StepProgram":
        """No more calls; ``output``: the buffer a step returns (32-bit, one row of ``output_width`` per
        wanted row), which every step gets as a tensor of its own."""
        self._output = (output, output_width)
        self._array = (IdmOp * len(self._ops))(*self._ops)
        self._order = sorted(self._buffers.values())
        return self

    @property
    def n_calls(self) -> int:
        return len(self._ops)

    # ------------------------------------------------------------------ running
    def run(self, ctx, want_rows: torch.Tensor) -> torch.Tensor:
        """The step ``ctx`` through the program; returns what the output buffer holds, ``[wanted rows, width]``."""
        K, st = self.K, self._step
        n, rows = ctx.n_tokens, want_rows.numel()
        K._need(want_rows, torch.int32, "wanted rows")
        out_buf, width = self._output
        out = torch.empty((rows, width), dtype=torch.float32, device=K.device)
        sizes, total = [], 0
        for index, per_token, per_row in self._order:
            if index == out_buf:
                sizes.append(-1)
                continue
            sizes.append(total)
            total += _align(n * per_token + rows * per_row)
        base = K.scratch("step_program", (total + 3) // 4).data_ptr()
        for (index, _, _), at in zip(self._order, sizes):
            st.buf[index] = out.data_ptr() if at < 0 else base + at
        for k, (n_q, n_kv, hd) in enumerate(self._plans):
            plan = K.attention_tc_plan(ctx, n_q, n_kv, hd)
            a = st.attn[k]
            (a.tile_seq, a.tile_start, a.n_tiles, a.rows_cap, a.max_runs, a.scratch, a.tile_pool, a.max_parts,
             a.runs_per_part) = plan
            a.run_blocks = K.attention_run_blocks
        st.tokens, st.token_seq, st.positions = ctx.tokens.data_ptr(), ctx.token_seq.data_ptr(), ctx.positions.data_ptr()
        st.cu_q, st.slots, st.q_start, st.kv_len = (ctx.cu_q.data_ptr(), ctx.slots.data_ptr(), ctx.q_start.data_ptr(),
                                                     ctx.kv_len.data_ptr())
        st.rows = want_rows.data_ptr() if rows else None
        st.n_tokens, st.n_rows = n, rows
        rc = K.lib.idm_run_program(self._array, len(self._ops), ctypes.byref(st), K._stream())
        K.launches += st.launches
        if rc != 0:
            from .ops import KernelError
            raise KernelError(f"{K.lib.idm_last_error().decode()} (call {st.failed_op} of the step program)")
        return out
