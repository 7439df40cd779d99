"""Python side of the CUDA kernels: shape checks, output allocation, the call.

``Kernels(dtype, device)`` loads the library compiled for that storage dtype
(``float32`` or ``bfloat16``) and exposes one method per kernel.  Every method
checks what the kernel cannot check itself and raises ``KernelError`` with the
library's message when a launch is refused.  There is no CPU path: constructing
``Kernels`` without a CUDA device raises.

Matrix products: the 32-bit library has its own FMA kernel (no tensor cores, no
reduced-precision mode).  In bfloat16 they run on the hand-written tcgen05
kernels of ``csrc/gemm_tcgen05.cu`` (the reference sends every matrix product to
a library, ``torch._int_mm``, src/detllm/backends.py:88-135).  No product is sent
to a library here, and none is split over its inner axis: an element is one chain
of additions whatever the step's size.

Environment switches (all default to the fast path): ``IDM_FUSED=0`` (epilogues as kernels of their
own), ``IDM_ATTENTION=generic`` (the general attention kernel for every step), ``IDM_PDL=0`` (no
programmatic dependent launch), ``IDM_PROGRAM=0`` (every kernel of a step called from Python instead
of one call that runs the step's list of calls).

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
    "idm_attention_tc_supports": (c_int, "i"),
    "idm_attention_tc_heads_per_tile": (c_int, "ii"),
    "idm_attention_tc_scratch_floats": (c_longlong, "iiiiii"),
    "idm_attention_tc": (c_int, "ppppipippippppiiiifiiippiip"),
    "idm_attention_tc_status": (c_int, ""),
    "idm_attention_tc_set_few_rows": (c_int, "i"),
    "idm_gemm_f32": (c_int, "pppiiip"),
    "idm_gemm_set_small": (None, "iii"),
    "idm_gemm_set_small_max": (None, "i"),
    "idm_gemm_set_small_tiles": (None, "i"),
    "idm_gemm_set_wide_tiles": (None, "i"),
    "idm_gemm_set_pair": (None, "ii"),
    "idm_gemm_set_band_mb": (None, "i"),
    "idm_gemm_set_wide_from": (None, "i"),
    "idm_gemm_bf16": (c_int, "pppiiip"),
    "idm_gemm_bf16_residual": (c_int, "pppiiip"),
    "idm_gemm_bf16_swiglu": (c_int, "pppiiip"),
    "idm_gemm_bf16_qkv": (c_int, "ppiiiiippfppppppppiipppp"),
    "idm_gemm_status": (c_int, ""),
    "idm_wait_probe": (c_int, "qipp"),
    "idm_program_layout": (c_int, "p"),
    "idm_run_program": (c_int, "pipp"),
    # only in a library compiled with -DIDM_TRACE (time stamps from inside two kernels: a measuring aid)
    "idm_gemm_trace_read": (c_int, "p"),
    "idm_gemm_block_trace_read": (c_int, "p"),
    "idm_gemm_log_read": (c_int, "pi"),
    "idm_gemm_mma_trace_read": (c_int, "p"),
    "idm_attention_tc_trace_read": (c_int, "p"),
    "idm_attention_item_trace_read": (c_int, "pi"),
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
        self._single_tiles = {}
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
        # fused epilogues of the tensor-core product (residual add, SwiGLU, q/k/v finish): parts use
        # them when this is True and run separate kernels otherwise (IDM_FUSED=0, and the 32-bit library).
        # Which of the two runs never depends on how many tokens a step brings.
        self.fused = dtype == torch.bfloat16 and os.environ.get("IDM_FUSED", "1") != "0"
        # "tcgen05": attention on the tensor cores wherever that kernel has the head size (64, 128) and the
        # layer has no window; "general": the one-warp-per-query kernel everywhere.  Which kernel runs never
        # depends on the step's shape, so prompts and single tokens give the same bits.
        self.attention_impl = os.environ.get("IDM_ATTENTION", "tcgen05")
        # key blocks (of 64) of a run of the tensor-core kernel: each run starts its sums from nothing and
        # the runs are folded in ascending order, so this number is part of the arithmetic's definition
        self.attention_run_blocks = 8
        # prompts: tiles with more key blocks than a fair share are shared by several blocks; the pool holds that
        # many runs' results (of 128 rows x (head_dim + 2) floats)
        self.attention_share_tiles = True
        self.attention_share_scale, self.attention_share_min_runs = 1.0, 2
        self.attention_pool_slots = 4096
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self.page = L.idm_page_tokens()
        # a model whose parts can emit their calls runs a step by one call into the library (program.py);
        # switched off (IDM_PROGRAM=0, or this attribute), every kernel is called from Python: the same bits
        self.use_programs = self.fused and os.environ.get("IDM_PROGRAM", "1") != "0"
        if hasattr(L, "idm_program_layout"):
            from . import program
            seen = (c_int * 16)()
            n = L.idm_program_layout(seen)
            if list(seen[:n]) != program.layout():
                raise KernelError(f"the records of a step program differ between the library {list(seen[:n])} "
                                  f"and the binding {program.layout()}")

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
        """Causal attention of the step's queries over the cache entry; returns [N, n_q * hd].

        One kernel per (dtype, head size, window or not) whatever the step looks like: the 32-bit
        library and windowed layers take the general kernel, bfloat16 with head sizes 64 and 128 the
        tensor-core kernel, for prompts and for single tokens alike."""
        self._need(q, self.dtype, "q")
        n, n_q, hd = q.shape
        self._check_kv(kv, kv.n_kv_heads, hd)
        w = int(window) if window else 0
        if (self.dtype == torch.bfloat16 and self.attention_impl == "tcgen05" and k_new is None and not w
                and kv.ring == 0 and self.lib.idm_attention_tc_supports(hd)):
            return self.attention_tc(q, kv, ctx, scale)
        return self.attention_generic(q, kv, ctx, k_new, v_new, scale, window)

    def attention_tc(self, q, kv, ctx, scale: float, out=None, through_scratch=None, share=None) -> torch.Tensor:
        """Causal attention on the tensor cores: tiles of (128 / gp tokens) x (gp q-heads of one kv-head).

        Steps with few tokens per sequence (at most 32 rows a tile: single tokens above all) give every
        run of key blocks a block of its own, and the runs meet in scratch; other steps let one block
        walk a tile's runs, except that tiles with more key blocks than a fair share of the step's are
        shared by several blocks.  ``through_scratch`` and ``share`` force one way or the other (tests: the
        bits are the same)."""
        n, n_q, hd = q.shape
        if out is None:
            out = torch.empty((n, n_q * hd), dtype=self.dtype, device=self.device)
        (tile_seq, tile_start, n_tiles, rows_cap, max_runs, scratch, tile_pool, max_parts,
         per) = self.attention_tc_plan(ctx, n_q, kv.n_kv_heads, hd, through_scratch, share)
        self._check(self.lib.idm_attention_tc(
            _p(q), _p(out), _p(kv.k), _p(kv.v), kv.k.shape[0],
            _p(kv.table), kv.table.shape[1], tile_seq, tile_start, n_tiles, _p(ctx.cu_q), _p(ctx.q_start),
            _p(ctx.kv_len), _p(ctx.slots), n, n_q, kv.n_kv_heads,
            hd, scale, self.attention_run_blocks, max_runs, rows_cap, scratch, tile_pool, max_parts, per,
            self._stream()))
        return out

    def attention_tc_plan(self, ctx, n_q: int, n_kv: int, hd: int, through_scratch=None, share=None):
        """What the attention launches of one step share, for one arrangement of heads: the list of tiles
        (on the device; made once a step), how the tiles' runs are spread over blocks, and the scratch.
        Returns (tile_seq, tile_start, n_tiles, rows_cap, max_runs, scratch, tile_pool, max_parts,
        runs_per_part) as ``idm_attention_tc`` takes them (addresses as integers or None)."""
        gp = self.lib.idm_attention_tc_heads_per_tile(n_q, n_kv)
        tok = 128 // gp
        R = self.attention_run_blocks
        tiles = ctx.memo.get(("attention_tc_tiles", gp))
        if tiles is None and ctx.single_token:
            # one tile per sequence: the same list for every step of that many sequences (kept, so that a
            # step being captured into a graph copies nothing from the host)
            tiles = self._single_tiles.get((ctx.n_seqs, gp))
            if tiles is None:
                dev = torch.stack([torch.arange(ctx.n_seqs, dtype=torch.int32),
                                   torch.zeros(ctx.n_seqs, dtype=torch.int32)]).to(self.device)
                tiles = self._single_tiles[(ctx.n_seqs, gp)] = (dev, dev[0].data_ptr(), dev[1].data_ptr(), ctx.n_seqs, gp)
        if tiles is None:
            # (sequence, first token of the tile); tiles with the most keys first, so that the longest
            # blocks start first
            items = []
            for i, L in enumerate(ctx.host_q_lens):
                for st in range(0, L, tok):
                    items.append((ctx.host_starts[i] + min(st + tok - 1, L - 1), i, st))
            items.sort(key=lambda t: -t[0])
            rows_cap = min(tok, max(ctx.host_q_lens)) * gp
            # Tiles with more key blocks than a fair share of the step's are shared by several blocks, each
            # walking `per` runs and leaving every run's result in a pool; the last block to arrive folds them
            # in the order of the runs (the same bits as one block walking them all: the runs are the same).
            n_hg = n_q // gp
            blocks_of = [last // self.page + 1 for last, _, _ in items]
            fair = -(-int(sum(blocks_of) * n_hg * self.attention_share_scale) // (2 * self.sm_count))
            per = max(self.attention_share_min_runs, -(-fair // R))   # runs a block walks
            pool, slots_used, max_parts = [], 0, 1
            for nb in blocks_of:
                runs = -(-nb // R)
                if self.attention_share_tiles and rows_cap == 128 and runs > per and slots_used + runs * n_hg <= self.attention_pool_slots:
                    pool.append(slots_used)
                    slots_used += runs * n_hg
                    max_parts = max(max_parts, -(-runs // per))
                else:
                    pool.append(-1)
            host = torch.tensor([[i for _, i, _ in items], [st for _, _, st in items], pool], dtype=torch.int32)
            dev = host.to(self.device)
            plan = (dev[2].data_ptr(), max_parts, per, slots_used) if slots_used else (None, 0, 0, 0)
            tiles = ctx.memo[("attention_tc_tiles", gp)] = (dev, dev[0].data_ptr(), dev[1].data_ptr(), len(items), rows_cap, plan)
        _, tile_seq, tile_start, n_tiles, rows_cap = tiles[:5]
        tile_pool, max_parts, per, pool_slots = tiles[5] if len(tiles) > 5 else (None, 0, 0, 0)
        # an upper bound of the key blocks any tile has (a captured step is replayed at growing lengths)
        longest = -(-ctx.max_kv_len // self.page)
        max_runs = -(-longest // R)
        if through_scratch is None:
            # every run a block of its own where a tile has few rows (single tokens above all): the runs'
            # results are small then.  For whole tiles of a prompt the way through scratch was measured
            # slower (2048 tokens: 88 us against 45 us), although it spreads a long tile over several blocks.
            through_scratch = rows_cap <= 32
        if through_scratch:
            need = self.lib.idm_attention_tc_scratch_floats(n_tiles, n_q, n_kv, hd, max_runs, rows_cap)
            tile_pool, max_parts, per = None, 0, 0
        else:
            if share is False:
                tile_pool, max_parts, per, pool_slots = None, 0, 0, 0
            need = self.lib.idm_attention_tc_scratch_floats(n_tiles, n_q, n_kv, hd, 0, 0) if (max_runs > 1 or pool_slots) else 0
            need += pool_slots * (-(-(128 * (hd + 2)) // 4) * 4)
            max_runs = 0
        scratch = self.scratch("attention_tc", need) if need else None
        return tile_seq, tile_start, n_tiles, rows_cap, max_runs, _p(scratch), tile_pool, max_parts, per

    def attention_tc_few_rows(self, on: bool) -> bool:
        """Whether tiles of at most 16 rows take the kernel made for them (the default) or the one all
        other tiles take; returns the old setting.  Tests compare the two bit for bit."""
        return bool(self.lib.idm_attention_tc_set_few_rows(1 if on else 0))

    def attention_tc_status(self) -> int:
        """Non-zero if a bounded wait inside an attention kernel ran out since the last call (the result
        of that launch is wrong).  The kernels' counters in scratch may then be left standing, so the
        scratch is cleared."""
        if self.dtype == torch.float32:
            return 0
        status = self.lib.idm_attention_tc_status()
        if status and "attention_tc" in self._scratch:
            self._scratch["attention_tc"].zero_()
        return status

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
        """``x [M, K] . w [N, K]^T`` in 32-bit as ``[1, M, N]`` (the leading axis is the one a part's
        delta carries: partial sums that the consumer adds; these kernels never split a sum)."""
        return self.gemm_store(x, w).unsqueeze(0)

    def _gemm_shape(self, x, w):
        self._need(x, self.dtype, "gemm input")
        self._need(w, self.dtype, "gemm weight")
        M, Kd = x.shape
        N, K2 = w.shape
        if Kd != K2:
            raise KernelError(f"gemm: input rows have {Kd} elements, weight rows {K2}")
        if self.dtype == torch.bfloat16 and Kd % 8:
            raise KernelError(f"gemm: the inner size {Kd} must be a multiple of 8 in bfloat16 (rows on 16-byte borders)")
        return M, N, Kd

    def gemm_store(self, x, w) -> torch.Tensor:
        """``x . w^T`` in 32-bit ``[M, N]``."""
        M, N, Kd = self._gemm_shape(x, w)
        out = torch.empty((M, N), dtype=torch.float32, device=self.device)
        if M:
            if self.dtype == torch.float32:
                self._check(self.lib.idm_gemm_f32(_p(x), _p(w), _p(out), M, N, Kd, self._stream()))
            else:
                self._check(self.lib.idm_gemm_bf16(_p(x), _p(w), _p(out), M, N, Kd, self._stream()))
        return out

    def gemm_choices(self, pair: Optional[bool] = None, lanes_up_to_tiles: Optional[int] = None,
                     band_mb: Optional[int] = None) -> None:
        """Which kernel a product of many tokens takes (tests compare them bit for bit; measurements): ``pair``:
        pairs of blocks on a tile where there are tiles enough, or never; ``lanes_up_to_tiles``: up to how many
        tiles of the persistent kernels a step of more than 128 tokens stays on the kernel with the tokens on the
        lanes; ``band_mb``: MB of the weight in a band of the persistent kernels' walk."""
        if self.dtype != torch.bfloat16:
            return
        if pair is not None:
            self.lib.idm_gemm_set_pair(1 if pair else 0, 0)
        if lanes_up_to_tiles is not None:
            self.lib.idm_gemm_set_small_tiles(int(lanes_up_to_tiles))
        if band_mb is not None:
            self.lib.idm_gemm_set_band_mb(int(band_mb))

    # ---- fused epilogues (bfloat16 only) ------------------------------------------------------------
    def gemm_residual(self, x, w, h) -> None:
        """``h += x . w^T`` in 32-bit, in place."""
        M, N, Kd = self._gemm_shape(x, w)
        self._need(h, torch.float32, "residual stream")
        if tuple(h.shape) != (M, N):
            raise KernelError(f"residual stream {tuple(h.shape)} does not match the product {(M, N)}")
        if M:
            self._check(self.lib.idm_gemm_bf16_residual(_p(x), _p(w), _p(h), M, N, Kd, self._stream()))

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
        M, N, Kd = self._gemm_shape(x, w_tiled)
        if N != -(-inter // 64) * 128:
            raise KernelError(f"tiled gate/up weight has {N} rows, expected {-(-inter // 64) * 128}")
        y = torch.empty((M, inter), dtype=self.dtype, device=self.device)
        if M:
            self._check(self.lib.idm_gemm_bf16_swiglu(_p(x), _p(w_tiled), _p(y), M, inter, Kd, self._stream()))
        return y

    QKV_FUSED_HEAD_DIMS = (32, 64, 128)

    def gemm_qkv(self, x, w, n_q, n_kv, hd, q_gamma, k_gamma, eps, cs, ctx, kv, keep_new: bool):
        """The fused q/k/v projection with norm, rotation and cache write as its epilogue
        (head_dim in ``QKV_FUSED_HEAD_DIMS``)."""
        M, N, Kd = self._gemm_shape(x, w)
        if N != (n_q + 2 * n_kv) * hd or hd not in self.QKV_FUSED_HEAD_DIMS:
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
                _p(x), _p(w), M, Kd, n_q,
                n_kv, hd, _p(q_gamma), _p(k_gamma), eps,
                _p(cs), _p(getattr(cs, "by_dim", None)), _p(q), _p(k_new), _p(v_new),
                (_p(kv.k) if kv is not None else None), (_p(kv.v) if kv is not None else None),
                (_p(kv.table) if kv is not None else None),
                (kv.table.shape[1] if kv is not None else 0), (kv.ring if kv is not None else 0),
                _p(ctx.token_seq), _p(ctx.positions), _p(ctx.slots), self._stream()))
        return q, k_new, v_new

    def wait_probe(self, limit_cycles: int, arrive: bool = False):
        """The kernels' bounded wait on a barrier nobody arrives at (or, with ``arrive``, one somebody does):
        returns (ran out, cycles waited, the second role left by the abort flag).  The kernel ends normally
        either way; a wait that ran out shows in ``gemm_status()``."""
        if self.dtype != torch.bfloat16:
            raise KernelError("the wait probe lives in the bfloat16 library")
        out = torch.full((3,), -1, dtype=torch.int32, device=self.device)
        self._check(self.lib.idm_wait_probe(int(limit_cycles), 1 if arrive else 0, _p(out), self._stream()), 1)
        ran_out, cycles, other = out.tolist()
        return bool(ran_out), int(cycles), bool(other)

    def gemm_status(self) -> int:
        """0, or 1 if a bounded wait inside the tensor-core GEMM ran out since the last call (synchronises)."""
        return 0 if self.dtype == torch.float32 else self.lib.idm_gemm_status()

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
