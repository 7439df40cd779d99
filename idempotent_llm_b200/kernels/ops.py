"""Python side of the CUDA kernels: shape checks, output allocation, the call.

``Kernels(dtype, device)`` loads the library compiled for that storage dtype
(``float32`` or ``bfloat16``) and exposes one method per kernel.  Every method
checks what the kernel cannot check itself and raises ``KernelError`` with the
library's message when a launch is refused.  There is no CPU path: constructing
``Kernels`` without a CUDA device raises.

Matrix products: the 32-bit library has its own FMA kernel (no tensor cores, no
reduced-precision mode).  In bfloat16 they run on the hand-written tcgen05
kernels of ``csrc/gemm_tcgen05.cu`` (the reference sends every matrix product to
a library, ``torch._int_mm``, src/detllm/backends.py:88-135); ``IDM_GEMM=library``
switches to the GEMM torch wraps, which is kept only to compare against.

Environment switches (all default to the fast path): ``IDM_GEMM``, ``IDM_FUSED``,
``IDM_FUSED_MIN_TOKENS``, ``IDM_FUSED_MAX_SMALL``, ``IDM_PREFILL``, ``IDM_PREFILL_RUN``,
``IDM_PDL``, ``IDM_PDL_ATTN``, ``IDM_DECODE_MMA``.

The entry points are called through ctypes with declared argument types (``SIGNATURES``), so that a
call passes plain integers and floats; the current stream's handle comes from torch without a stream
object being built.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import builder

_DT = {torch.float32: "float32", torch.bfloat16: "bfloat16"}


class KernelError(RuntimeError):
    pass


# the handle of the current stream of a device as an integer, without building a stream object
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


# Every entry point of the libraries: result type and, per argument, p pointer (or stream) / i int /
# f float / q long long, in the order of the C declarations in csrc/ (a test reads the declarations
# and compares).
SIGNATURES = {
    "idm_last_error": (ctypes.c_char_p, ""),
    "idm_dtype_name": (ctypes.c_char_p, ""),
    "idm_page_tokens": (c_int, ""),
    "idm_set_pdl": (None, "i"),
    "idm_embed": (c_int, "pppiip"),
    "idm_add_rmsnorm": (c_int, "ppiqpfppiip"),
    "idm_rope_table": (c_int, "ppppiip"),
    "idm_qkv_finish": (c_int, "piqiiiippfpppppppiipppp"),
    "idm_kv_write_ring": (c_int, "pppppiippppiiip"),
    "idm_swiglu": (c_int, "piqpiiip"),
    "idm_sample_scratch_floats": (c_longlong, "ii"),
    "idm_sample": (c_int, "piifpppp"),
    "idm_decode_advance": (c_int, "pppppppiip"),
    "idm_attention_generic": (c_int, "pppppiipppppppiiiifip"),
    "idm_attention_decode_supports": (c_int, "i"),
    "idm_attention_decode_chunk": (c_int, ""),
    "idm_attention_decode_scratch_floats": (c_longlong, "iiii"),
    "idm_attention_decode": (c_int, "pppppiipppiiiiifip"),
    "idm_attention_decode_static": (c_int, "pppppiippiiiiifip"),
    "idm_attention_prefill_supports": (c_int, "i"),
    "idm_attention_prefill_max_run": (c_int, "qiii"),
    "idm_attention_prefill_scratch_floats": (c_longlong, "iiii"),
    "idm_attention_prefill": (c_int, "ppppipippippppiiiifiipp"),
    "idm_attention_prefill_status": (c_int, ""),
    "idm_gemm_f32": (c_int, "pppiiip"),
    "idm_gemm_bf16_splits": (c_int, "iii"),
    "idm_gemm_bf16_workspace_floats": (c_longlong, "iii"),
    "idm_gemm_set_cluster": (None, "i"),
    "idm_gemm_set_persistent": (None, "i"),
    "idm_gemm_set_many_from": (None, "i"),
    "idm_gemm_bf16": (c_int, "pppiiiip"),
    "idm_gemm_bf16_store": (c_int, "ppppiiiip"),
    "idm_gemm_bf16_residual": (c_int, "ppppiiiip"),
    "idm_gemm_bf16_swiglu": (c_int, "ppppiiiip"),
    "idm_gemm_bf16_qkv": (c_int, "pppiiiiiippfppppppppiipppp"),
    "idm_gemm_status": (c_int, ""),
}


class Kernels:
    def __init__(self, dtype: torch.dtype, device):
        device = torch.device(device)
        if dtype not in _DT:
            raise KernelError(f"no kernels for dtype {dtype}; float32 and bfloat16 exist")
        if device.type != "cuda" or not torch.cuda.is_available():
            raise KernelError("the kernels run on a CUDA device only; there is no CPU path")
        cap = torch.cuda.get_device_capability(device)
        if cap[0] != 10:
            raise KernelError(f"the kernels are compiled for sm_100a; this device is sm_{cap[0]}{cap[1]}")
        self.dtype = dtype
        self.device = device
        self.lib = builder.load(_DT[dtype])
        self.launches = 0                     # kernels of this library launched so far
        self._scratch = {}
        self._device_index = device.index if device.index is not None else 0
        self._retired = []
        L = self.lib
        # argument and result types of every entry point: with them set, plain integers (addresses,
        # sizes), floats and None (a null pointer) go in as they are -- no ctypes object per argument
        kinds = {"p": c_void_p, "i": c_int, "f": c_float, "q": c_longlong}
        for name, (result, args) in SIGNATURES.items():
            fn = getattr(L, name, None)
            if fn is None:
                continue                      # an entry point of the other precision's library
            fn.restype = result
            fn.argtypes = [kinds[a] for a in args]
        # "tcgen05": the hand-written tensor-core kernel; "library": the GEMM torch wraps (kept to
        # compare against)
        self.gemm_impl = os.environ.get("IDM_GEMM", "tcgen05")
        # fused epilogues of the tensor-core product (residual add, SwiGLU, q/k/v finish): parts use
        # them when this is True and fall back to separate kernels otherwise
        self.fused = (dtype == torch.bfloat16 and self.gemm_impl == "tcgen05"
                      and os.environ.get("IDM_FUSED", "1") != "0")
        # Up to 64 tokens the slices of a split inner axis are added inside a thread-block cluster and
        # the epilogue is fused; above 256 tokens nothing is split and the epilogue is fused; between
        # the two the separate kernels, which add the slices with the whole GPU, are quicker than one
        # block per tile doing it -- unless the layer's products are so short that the library does not
        # split them at all (see use_fused).  IDM_FUSED_MIN_TOKENS / IDM_FUSED_MAX_SMALL move the borders.
        self.fused_min_tokens = int(os.environ.get("IDM_FUSED_MIN_TOKENS", "257"))
        if dtype == torch.bfloat16:
            L.idm_gemm_set_many_from(self.fused_min_tokens)
        self.fused_max_small = int(os.environ.get("IDM_FUSED_MAX_SMALL", "64"))
        # "tcgen05": prompts' attention on the tensor cores; "general": the one-warp-per-query kernel
        self.prefill_impl = os.environ.get("IDM_PREFILL", "tcgen05")
        # the most key blocks (of 64) one block of that kernel works through before a tile is cut into
        # runs for several blocks; 0: by the step's size
        self.prefill_run = int(os.environ.get("IDM_PREFILL_RUN", "0"))
        self.page = L.idm_page_tokens()
        self._gemm_plans = {}          # (M, N, K) -> (splits of the inner axis, workspace floats)

    def use_fused(self, n_tokens: int, *weights) -> bool:
        """Whether a part runs its products with fused epilogues at this many tokens: always up to
        ``fused_max_small`` and from ``fused_min_tokens`` on; in between only if none of the part's
        products (``weights``: their ``[N, K]`` matrices) is split over its inner axis."""
        if not self.fused:
            return False
        if n_tokens >= self.fused_min_tokens or n_tokens <= self.fused_max_small:
            return True
        return bool(weights) and all(self._splits(n_tokens, w.shape[0], w.shape[1]) == 1 for w in weights)

    def _splits(self, M: int, N: int, Kd: int) -> int:
        plan = self._gemm_plans.get((M, N, Kd))
        if plan is None:
            P = self.lib.idm_gemm_bf16_splits(M, N, Kd)
            plan = self._gemm_plans[(M, N, Kd)] = (P, self.lib.idm_gemm_bf16_workspace_floats(M, N, P))
        return plan[0]

    # ------------------------------------------------------------------ helpers
    def _stream(self):
        # (the stream object torch builds for current_stream() costs several microseconds per launch)
        if _raw_stream is not None:
            return _raw_stream(self._device_index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def _check(self, rc: int, n_launches: int = 1):
        if rc != 0:
            raise KernelError(self.lib.idm_last_error().decode())
        self.launches += n_launches

    def _need(self, t: torch.Tensor, dtype, what: str):
        if t.dtype != dtype or not t.is_cuda or not t.is_contiguous():
            raise KernelError(f"{what}: expected a contiguous CUDA tensor of {dtype}, got {t.dtype} "
                              f"{'cuda' if t.is_cuda else 'cpu'} contiguous={t.is_contiguous()}")

    def scratch(self, key: str, n_floats: int) -> torch.Tensor:
        """A 32-bit scratch buffer that only grows (its address is stable across steps once large enough)."""
        buf = self._scratch.get(key)
        if buf is None or buf.numel() < n_floats:
            # a captured graph may still point at the old buffer: it is kept, never freed
            self._retired.append(buf)
            # zeros: kernels keep arrival counters in their scratch and leave them at zero
            buf = self._scratch[key] = torch.zeros(max(n_floats, 1), dtype=torch.float32, device=self.device)
        return buf

    # ------------------------------------------------------------------ kernels
    def embed(self, tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        self._need(tokens, torch.int32, "embed tokens")
        self._need(table, self.dtype, "embed table")
        n, hidden = tokens.numel(), table.shape[1]
        h = torch.empty((n, hidden), dtype=torch.float32, device=self.device)
        self._check(self.lib.idm_embed(_p(tokens), _p(table), _p(h),
                                       n, hidden, self._stream()))
        return h

    def add_rmsnorm(self, h, delta, gamma, eps: float, rows=None) -> torch.Tensor:
        self._need(h, torch.float32, "residual stream")
        self._need(gamma, torch.float32, "norm weight")
        n, hidden = h.shape
        if gamma.numel() != hidden:
            raise KernelError(f"norm weight has {gamma.numel()} elements, rows have {hidden}")
        P, stride = 0, 0
        if delta is not None:
            self._need(delta, torch.float32, "delta")
            if delta.dim() != 3 or tuple(delta.shape[1:]) != (n, hidden):
                raise KernelError(f"delta {tuple(delta.shape)} does not match the stream {(n, hidden)}")
            P, stride = delta.shape[0], n * hidden
        if rows is not None:
            self._need(rows, torch.int32, "rows")
        n_out = n if rows is None else rows.numel()
        x = torch.empty((n_out, hidden), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_add_rmsnorm(_p(h), _p(delta), P, stride,
                                             _p(gamma), eps, _p(x),
                                             _p(rows), n_out, hidden, self._stream()))
        return x

    def rope_table(self, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
        self._need(positions, torch.int32, "positions")
        self._need(inv_freq, torch.float64, "inv_freq")
        n, half = positions.numel(), inv_freq.numel()
        cs = torch.empty((n, half, 2), dtype=torch.float32, device=self.device)
        # for steps of many tokens also as [half, n, 2]: the q/k/v product's epilogue of such steps has
        # a thread per token and reads the tokens of one dim side by side
        by_dim = torch.empty((half, n, 2), dtype=torch.float32, device=self.device) if n > 64 else None
        self._check(self.lib.idm_rope_table(_p(positions), _p(inv_freq), _p(cs), _p(by_dim),
                                            n, half, self._stream()))
        cs.by_dim = by_dim
        return cs

    def qkv_finish(self, qkv, n_q, n_kv, hd, q_gamma, k_gamma, eps, cs, ctx, kv, keep_new: bool):
        """Norm + rotation of q and k heads; k, v to the cache entry ``kv`` (if given) and/or to packed
        buffers (``keep_new``).  Returns (q [N, n_q, hd], k_new, v_new)."""
        self._need(qkv, torch.float32, "qkv")
        P, n, width = qkv.shape
        if width != (n_q + 2 * n_kv) * hd:
            raise KernelError(f"qkv rows have {width} elements, expected {(n_q + 2 * n_kv) * hd}")
        if cs is not None and tuple(cs.shape) != (n, hd // 2, 2):
            raise KernelError(f"rotary table {tuple(cs.shape)} does not match {(n, hd // 2, 2)}")
        for gmm in (q_gamma, k_gamma):
            if gmm is not None and gmm.numel() != hd:
                raise KernelError("q/k norm weight must have head_dim elements")
        q = torch.empty((n, n_q, hd), dtype=self.dtype, device=self.device)
        k_new = v_new = None
        if keep_new and n_kv:
            k_new = torch.empty((n, n_kv, hd), dtype=self.dtype, device=self.device)
            v_new = torch.empty((n, n_kv, hd), dtype=self.dtype, device=self.device)
        if kv is not None:
            self._check_kv(kv, n_kv, hd)
        self._check(self.lib.idm_qkv_finish(
            _p(qkv), P, n * width, n, n_q, n_kv, hd,
            _p(q_gamma), _p(k_gamma), eps, _p(cs),
            _p(q), _p(k_new), _p(v_new),
            (_p(kv.k) if kv is not None else None), (_p(kv.v) if kv is not None else None),
            (_p(kv.table) if kv is not None else None),
            (kv.table.shape[1] if kv is not None else 0), (kv.ring if kv is not None else 0),
            _p(ctx.token_seq), _p(ctx.positions), _p(ctx.slots), self._stream()))
        return q, k_new, v_new

    def _check_kv(self, kv, n_kv, hd):
        if kv.k.dtype != self.dtype or kv.k.shape[1:] != (n_kv, self.page, hd) or not kv.k.is_contiguous():
            raise KernelError(f"cache entry {tuple(kv.k.shape)} {kv.k.dtype} does not fit "
                              f"[pages, {n_kv}, {self.page}, {hd}] {self.dtype}")

    def kv_write_ring(self, k_new, v_new, kv, ctx) -> None:
        n, n_kv, hd = k_new.shape
        self._check_kv(kv, n_kv, hd)
        self._check(self.lib.idm_kv_write_ring(
            _p(k_new), _p(v_new), _p(kv.k), _p(kv.v),
            _p(kv.table), kv.table.shape[1], kv.ring, _p(ctx.token_seq),
            _p(ctx.positions), _p(ctx.slots), _p(ctx.kv_len), n,
            n_kv, hd, self._stream()))

    def attention(self, q, kv, ctx, k_new, v_new, scale: float, window) -> torch.Tensor:
        """Causal attention of the step's queries over the cache entry; returns [N, n_q * hd]."""
        self._need(q, self.dtype, "q")
        n, n_q, hd = q.shape
        self._check_kv(kv, kv.n_kv_heads, hd)
        out = torch.empty((n, n_q * hd), dtype=self.dtype, device=self.device)
        w = int(window) if window else 0
        # 32-bit keeps ONE kernel for prompts and single tokens, so its logits are the same bits
        # however a sequence is cut into steps; bfloat16 takes the bandwidth-bound decode kernel
        if (self.dtype != torch.float32 and ctx.single_token and k_new is None
                and self.lib.idm_attention_decode_supports(hd)):
            return self.attention_decode(q, kv, ctx.slots, ctx.kv_len, ctx.max_kv_len, scale, w, out)
        if (self.dtype == torch.bfloat16 and self.prefill_impl == "tcgen05" and not ctx.single_token
                and k_new is None and not w and kv.ring == 0 and self.lib.idm_attention_prefill_supports(hd)):
            return self.attention_prefill(q, kv, ctx, scale, out)
        self._check(self.lib.idm_attention_generic(
            _p(q), _p(out), _p(kv.k), _p(kv.v), _p(kv.table),
            kv.table.shape[1], kv.ring, _p(k_new), _p(v_new),
            _p(ctx.token_seq), _p(ctx.positions), _p(ctx.slots),
            _p(ctx.q_start), _p(ctx.cu_q), n, n_q, kv.n_kv_heads,
            hd, scale, w, self._stream()))
        return out

    def attention_prefill(self, q, kv, ctx, scale: float, out=None) -> torch.Tensor:
        """Causal attention of prompts on the tensor cores (tiles of 128 query tokens x q-heads)."""
        n, n_q, hd = q.shape
        if out is None:
            out = torch.empty((n, n_q * hd), dtype=self.dtype, device=self.device)
        tiles = ctx.memo.get("prefill_tiles")
        if tiles is None:
            # (sequence, first token of the tile); tiles with the most keys first, so that the longest
            # blocks start first
            items = []
            for i, L in enumerate(ctx.host_q_lens):
                for st in range(0, L, 128):
                    items.append((ctx.host_starts[i] + min(st + 127, L - 1), i, st))
            items.sort(key=lambda t: -t[0])
            host = torch.tensor([[i for _, i, _ in items], [st for _, _, st in items]], dtype=torch.int32)
            blocks = [last // 64 + 1 for last, _, _ in items]        # key blocks of each tile
            dev = host.to(self.device)
            tiles = ctx.memo["prefill_tiles"] = (dev, dev[0].data_ptr(), dev[1].data_ptr(), len(items), sum(blocks),
                                                 blocks[0])
        _, tile_seq, tile_start, n_tiles, key_blocks, longest = tiles
        plan = ctx.memo.get(("prefill_runs", n_q, hd, self.prefill_run))
        if plan is None:
            max_run = self.prefill_run or self.lib.idm_attention_prefill_max_run(
                key_blocks * n_q, longest, n_tiles, n_q)
            split = min(4, -(-longest // max_run))
            need = self.lib.idm_attention_prefill_scratch_floats(n_tiles, n_q, hd, split)
            plan = ctx.memo[("prefill_runs", n_q, hd, self.prefill_run)] = (max_run, split, need)
        max_run, split, need = plan
        scratch = self.scratch("attention_prefill", need) if need else None
        self._check(self.lib.idm_attention_prefill(
            _p(q), _p(out), _p(kv.k), _p(kv.v), kv.k.shape[0],
            _p(kv.table), kv.table.shape[1], tile_seq, tile_start, n_tiles, _p(ctx.cu_q), _p(ctx.q_start),
            _p(ctx.kv_len), _p(ctx.slots), n, n_q, kv.n_kv_heads,
            hd, scale, split, max_run, _p(scratch),
            self._stream()))
        return out

    def attention_prefill_status(self) -> int:
        return 0 if self.dtype == torch.float32 else self.lib.idm_attention_prefill_status()

    def attention_generic(self, q, kv, ctx, k_new, v_new, scale: float, window) -> torch.Tensor:
        """The general kernel, whatever the step's shape (tests compare the special kernels with it)."""
        n, n_q, hd = q.shape
        out = torch.empty((n, n_q * hd), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_attention_generic(
            _p(q), _p(out), _p(kv.k), _p(kv.v), _p(kv.table),
            kv.table.shape[1], kv.ring, _p(k_new), _p(v_new),
            _p(ctx.token_seq), _p(ctx.positions), _p(ctx.slots),
            _p(ctx.q_start), _p(ctx.cu_q), n, n_q, kv.n_kv_heads,
            hd, scale, (int(window) if window else 0), self._stream()))
        return out

    def attention_decode(self, q, kv, slots, kv_len, max_kv_len: int, scale: float, window: int,
                         out=None) -> torch.Tensor:
        """One query per sequence against its cached keys (split over chunks of keys, then merged)."""
        n, n_q, hd = q.shape
        if out is None:
            out = torch.empty((n, n_q * hd), dtype=self.dtype, device=self.device)
        n_chunks = -(-max_kv_len // self.lib.idm_attention_decode_chunk())
        need = self.lib.idm_attention_decode_scratch_floats(n, n_q, n_chunks, hd)
        scratch = self.scratch("attention_decode", need)
        self._check(self.lib.idm_attention_decode(
            _p(q), _p(out), _p(kv.k), _p(kv.v), _p(kv.table),
            kv.table.shape[1], kv.ring, _p(slots), _p(kv_len),
            _p(scratch), n, n_q, kv.n_kv_heads, hd, max_kv_len,
            scale, window, self._stream()))
        return out

    def swiglu(self, gu: torch.Tensor, tiled_inter: Optional[int] = None) -> torch.Tensor:
        """``g * sigmoid(g) * u`` of the gate/up product ``[P, N, 2 * inter]`` (gate columns, then up
        columns), or of its tiled form ``[P, N, ceil(inter / 64) * 128]`` when ``tiled_inter`` is given."""
        self._need(gu, torch.float32, "gate-up")
        P, n, width = gu.shape
        if tiled_inter is None:
            if width % 2:
                raise KernelError("gate-up rows must have an even number of elements")
            inter, tiled = width // 2, 0
        else:
            inter, tiled = int(tiled_inter), 1
            if width != -(-inter // 64) * 128:
                raise KernelError(f"tiled gate-up rows have {width} elements, expected {-(-inter // 64) * 128}")
        y = torch.empty((n, inter), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_swiglu(_p(gu), P, n * width, _p(y),
                                        n, inter, tiled, self._stream()))
        return y

    def gemm(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``x [M, K] . w [N, K]^T`` -> 32-bit partial sums ``[P, M, N]`` (their sum over P is the product)."""
        self._need(x, self.dtype, "gemm input")
        self._need(w, self.dtype, "gemm weight")
        M, Kd = x.shape
        N, K2 = w.shape
        if Kd != K2:
            raise KernelError(f"gemm: input rows have {Kd} elements, weight rows {K2}")
        if self.dtype == torch.float32:
            out = torch.empty((1, M, N), dtype=torch.float32, device=self.device)
            self._check(self.lib.idm_gemm_f32(_p(x), _p(w), _p(out), M,
                                              N, Kd, self._stream()))
            return out
        if self.gemm_impl == "library" or Kd % 8 or M == 0:
            return self._gemm_library(x, w)
        P = self.lib.idm_gemm_bf16_splits(M, N, Kd)
        out = torch.empty((P, M, N), dtype=torch.float32, device=self.device)
        self._check(self.lib.idm_gemm_bf16(_p(x), _p(w), _p(out), M, N,
                                           Kd, P, self._stream()))
        return out

    # ---- fused epilogues (bfloat16 only) ------------------------------------------------------------
    def _gemm_shape(self, x, w):
        self._need(x, self.dtype, "gemm input")
        self._need(w, self.dtype, "gemm weight")
        M, Kd = x.shape
        N, K2 = w.shape
        if Kd != K2:
            raise KernelError(f"gemm: input rows have {Kd} elements, weight rows {K2}")
        if Kd % 8:
            raise KernelError(f"gemm: the inner size {Kd} must be a multiple of 8 for the fused kernels")
        P = self._splits(M, N, Kd)
        return M, N, Kd, P, self.scratch("gemm_ws", self._gemm_plans[(M, N, Kd)][1])

    def gemm_store(self, x, w) -> torch.Tensor:
        """``x . w^T`` finished in 32-bit ``[M, N]``."""
        M, N, Kd, P, ws = self._gemm_shape(x, w)
        out = torch.empty((M, N), dtype=torch.float32, device=self.device)
        if M:
            self._check(self.lib.idm_gemm_bf16_store(_p(x), _p(w), _p(out),
                                                     _p(ws), M, N, Kd, P,
                                                     self._stream()))
        return out

    def gemm_residual(self, x, w, h) -> None:
        """``h += x . w^T`` in 32-bit, in place."""
        M, N, Kd, P, ws = self._gemm_shape(x, w)
        self._need(h, torch.float32, "residual stream")
        if tuple(h.shape) != (M, N):
            raise KernelError(f"residual stream {tuple(h.shape)} does not match the product {(M, N)}")
        if M:
            self._check(self.lib.idm_gemm_bf16_residual(_p(x), _p(w), _p(h),
                                                        _p(ws), M, N, Kd, P,
                                                        self._stream()))

    def tile_gate_up(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        """Rows of gate and up alternating (gate row of a feature, then its up row), padded with zero
        rows to whole tiles of 64 features = 128 rows: the layout ``gemm_swiglu`` reads."""
        inter, Kd = gate.shape
        tiles = -(-inter // 64)
        out = torch.zeros((tiles * 64, 2, Kd), dtype=gate.dtype, device=gate.device)
        out[:inter, 0] = gate
        out[:inter, 1] = up
        return out.view(tiles * 128, Kd).contiguous()

    def gemm_swiglu(self, x, w_tiled, inter: int) -> torch.Tensor:
        """``silu(x . gate^T) * (x . up^T)`` in the storage dtype ``[M, inter]``."""
        M, N, Kd, P, ws = self._gemm_shape(x, w_tiled)
        if N != -(-inter // 64) * 128:
            raise KernelError(f"tiled gate/up weight has {N} rows, expected {-(-inter // 64) * 128}")
        y = torch.empty((M, inter), dtype=self.dtype, device=self.device)
        if M:
            self._check(self.lib.idm_gemm_bf16_swiglu(_p(x), _p(w_tiled), _p(y),
                                                      _p(ws), M, inter, Kd, P,
                                                      self._stream()))
        return y

    def gemm_qkv(self, x, w, n_q, n_kv, hd, q_gamma, k_gamma, eps, cs, ctx, kv, keep_new: bool):
        """The fused q/k/v projection with ``qkv_finish`` as its epilogue (128 % hd == 0)."""
        M, N, Kd, P, ws = self._gemm_shape(x, w)
        if N != (n_q + 2 * n_kv) * hd or 128 % hd:
            raise KernelError(f"gemm_qkv: weight rows {N}, heads {(n_q, n_kv)}, head_dim {hd}")
        if cs is not None and tuple(cs.shape) != (M, hd // 2, 2):
            raise KernelError(f"rotary table {tuple(cs.shape)} does not match {(M, hd // 2, 2)}")
        q = torch.empty((M, n_q, hd), dtype=self.dtype, device=self.device)
        k_new = v_new = None
        if keep_new and n_kv:
            k_new = torch.empty((M, n_kv, hd), dtype=self.dtype, device=self.device)
            v_new = torch.empty((M, n_kv, hd), dtype=self.dtype, device=self.device)
        if kv is not None:
            self._check_kv(kv, n_kv, hd)
        if M:
            self._check(self.lib.idm_gemm_bf16_qkv(
                _p(x), _p(w), _p(ws), M, Kd, P, n_q,
                n_kv, hd, _p(q_gamma), _p(k_gamma), eps,
                _p(cs), _p(getattr(cs, "by_dim", None)), _p(q), _p(k_new), _p(v_new),
                (_p(kv.k) if kv is not None else None), (_p(kv.v) if kv is not None else None),
                (_p(kv.table) if kv is not None else None),
                (kv.table.shape[1] if kv is not None else 0), (kv.ring if kv is not None else 0),
                _p(ctx.token_seq), _p(ctx.positions), _p(ctx.slots), self._stream()))
        return q, k_new, v_new

    def gemm_status(self) -> int:
        """0, or 1 if a bounded wait inside the tensor-core GEMM ran out since the last call (synchronises)."""
        return 0 if self.dtype == torch.float32 else self.lib.idm_gemm_status()

    def _gemm_library(self, x, w):
        if M_is_zero(x):
            return torch.empty((1, 0, w.shape[0]), dtype=torch.float32, device=self.device)
        try:
            out = torch.mm(x, w.t(), out_dtype=torch.float32)
        except (TypeError, RuntimeError):
            out = torch.mm(x, w.t()).to(torch.float32)
        return out.unsqueeze(0)

    def sample(self, logits: torch.Tensor, temperature: float, keys: Optional[torch.Tensor]) -> torch.Tensor:
        self._need(logits, torch.float32, "logits")
        B, V = logits.shape
        if keys is not None:
            self._need(keys, torch.int64, "row keys")
            if keys.numel() != B:
                raise KernelError("one key per row")
        out = torch.empty((B,), dtype=torch.int32, device=self.device)
        scratch = self.scratch("sample", self.lib.idm_sample_scratch_floats(B, V))
        self._check(self.lib.idm_sample(_p(logits), B, V, temperature,
                                        _p(keys), _p(out), _p(scratch), self._stream()))
        return out


    def decode_advance(self, tokens, positions, q_start, kv_len, sampled, history, step_counter) -> None:
        """tokens <- sampled; positions, q_start, kv_len += 1; history[step] <- sampled; step += 1."""
        n = tokens.numel()
        self._check(self.lib.idm_decode_advance(
            _p(tokens), _p(positions), _p(q_start), _p(kv_len),
            _p(sampled), _p(history), _p(step_counter), n,
            history.shape[0], self._stream()))


def M_is_zero(x) -> bool:
    return x.shape[0] == 0
