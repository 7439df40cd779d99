"""One kernel alone at a preset's layer sizes, timed with CUDA events (L2 flushed between runs):
``python -m idempotent_llm_b200 kernel-bench --kernel ...``.  A measuring aid beside ``bench.py``; the
summaries under ``profiles/`` name the commands they were made with."""

from __future__ import annotations

import torch


def run(args) -> int:
    """One kernel alone at a preset's layer sizes, timed with CUDA events (L2 flushed between runs)."""
    import math
    from .cache import CacheNeed, SequenceCache
    from .config.presets import preset
    from .kernels import Kernels
    cfg = preset(args.size)
    K = Kernels(torch.bfloat16, "cuda:0")
    # which kernel a product of many tokens takes (defaults: what the library chooses by itself)
    K.gemm_choices(pair=None if getattr(args, "pairs", None) is None else bool(args.pairs),
                   band_mb=getattr(args, "band_mb", None), lanes_up_to_tiles=getattr(args, "lanes_up_to_tiles", None))
    n_q, n_kv, hd, H, I = (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.hidden_size,
                           cfg.intermediate_size)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    g = torch.Generator().manual_seed(0)

    def timed(fn, reps=args.reps):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e-3)
        ts.sort()
        return ts[len(ts) // 2]

    if args.kernel in ("attention_single", "attention_single_mma", "attention_prompt"):
        B = args.batch
        cache = SequenceCache({0: CacheNeed("full", n_kv, hd)}, B * args.capacity, torch.bfloat16, "cuda:0",
                              max_seqs=B, max_seq_len=args.capacity)
        slots = [cache.alloc_slot() for _ in range(B)]
        lens = [int(torch.randint(int(args.context * 0.7), args.context + 1, (1,), generator=g)) for _ in range(B)]
        if args.kernel == "attention_prompt":
            lens = [args.context] * B
        cache.reserve(list(zip(slots, lens))); cache.flush()
        kv = cache.view(0)
        scale = 1.0 / math.sqrt(hd)
        from .engine.batch import context_from_packed, pack_step_host
        if args.kernel != "attention_prompt":
            # one query per sequence at its last position; the grid is sized for the capacity, as a captured step's is
            q = torch.randn(B, n_q, hd, device="cuda").bfloat16()
            packed, n, q_lens = pack_step_host(slots, [L - 1 for L in lens], [[0]] * B)
            ctx = context_from_packed(packed.cuda(), n, slots, q_lens, [L - 1 for L in lens], max_kv_len=args.capacity)
            if args.kernel == "attention_single":
                t = timed(lambda: K.attention_tc(q, kv, ctx, scale))
            else:       # the mma.sync kernel with a fresh sum per page (other bits than prompts get: not on the product path)
                t = timed(lambda: K.attention_decode(q, kv, ctx.slots, ctx.kv_len, args.capacity, scale, 0))
            byt = sum(lens) * n_kv * hd * 2 * 2
            print(f"{args.kernel} {args.size} batch={B} context~{args.context}: {t * 1e6:.1f} us, "
                  f"{byt / 1e6:.1f} MB of keys and values, {byt / t / 1e9:.0f} GB/s")
        else:
            packed, n, q_lens = pack_step_host(slots, [0] * B, [[0] * L for L in lens])
            ctx = context_from_packed(packed.cuda(), n, slots, q_lens, [0] * B)
            q = torch.randn(n, n_q, hd, device="cuda").bfloat16()
            t = timed(lambda: K.attention_tc(q, kv, ctx, scale))
            fl = sum(4 * hd * n_q * L * (L + 1) // 2 for L in lens)
            print(f"attention_prompt {args.size} batch={B} tokens={args.context}: {t * 1e6:.1f} us, "
                  f"{fl / 1e9:.1f} GFLOP (causal), {fl / t / 1e12:.0f} TFLOP/s")
    elif args.kernel == "gemm":
        shapes = {"qkv": ((n_q + 2 * n_kv) * hd, H), "o": (H, n_q * hd), "gate_up": (2 * I, H), "down": (H, I),
                  "lm_head": (cfg.vocab_size, H)}
        for name, (N, Kd) in shapes.items():
            x = torch.randn(args.tokens, Kd, device="cuda").bfloat16()
            w = (torch.randn(N, Kd, device="cuda") * 0.02).bfloat16()
            t = timed(lambda: K.gemm(x, w))
            fl, byt = 2.0 * args.tokens * N * Kd, 2.0 * N * Kd
            print(f"gemm {name} [{args.tokens} x {Kd}] . [{N} x {Kd}]^T: {t * 1e6:.1f} us, {fl / t / 1e12:.1f} TFLOP/s, "
                  f"weights {byt / t / 1e9:.0f} GB/s")
    elif args.kernel == "gemm_fused":
        # the four products of a layer with their fused epilogues, as the parts call them
        from .engine.batch import context_from_packed, pack_step_host
        M = args.tokens
        cache = SequenceCache({0: CacheNeed("full", n_kv, hd)}, -(-M // 64) * 64 + 64, torch.bfloat16, "cuda:0",
                              max_seqs=1, max_seq_len=-(-M // 64) * 64 + 64)
        slot = cache.alloc_slot()
        cache.reserve([(slot, M)]); cache.flush()
        packed, n, q_lens = pack_step_host([slot], [0], [[0] * M])
        ctx = context_from_packed(packed.cuda(), n, [slot], q_lens, [0])
        kv = cache.view(0)
        rnd = lambda *shape: (torch.randn(*shape, device="cuda") * 0.05).bfloat16()
        x, xo, xi = rnd(M, H) * 20, rnd(M, n_q * hd) * 20, rnd(M, I) * 20
        w_qkv, w_o, w_down = rnd((n_q + 2 * n_kv) * hd, H), rnd(H, n_q * hd), rnd(H, I)
        w_gu = K.tile_gate_up(rnd(I, H), rnd(I, H))
        gq = torch.ones(hd, device="cuda"); gk = torch.ones(hd, device="cuda")
        inv = 1e6 ** (-2.0 * torch.arange(0, hd // 2, dtype=torch.float64) / hd)
        cs = K.rope_table(ctx.positions, inv.cuda())
        h = torch.zeros(M, H, device="cuda")
        runs = {"qkv (norm, rotation, cache write)": (lambda: K.gemm_qkv(x, w_qkv, n_q, n_kv, hd, gq, gk, 1e-6, cs, ctx, kv,
                                                                           keep_new=False), (n_q + 2 * n_kv) * hd, H),
                "o (residual add)": (lambda: K.gemm_residual(xo, w_o, h), H, n_q * hd),
                "gate_up (SwiGLU)": (lambda: K.gemm_swiglu(x, w_gu, I), 2 * I, H),
                "down (residual add)": (lambda: K.gemm_residual(xi, w_down, h), H, I)}
        for name, (fn, N, Kd) in runs.items():
            t = timed(fn)
            fl, byt = 2.0 * M * N * Kd, 2.0 * N * Kd
            print(f"gemm {name} [{M} x {Kd}] . [{N} x {Kd}]^T: {t * 1e6:.1f} us, {fl / t / 1e12:.1f} TFLOP/s, "
                  f"weights {byt / t / 1e9:.0f} GB/s")
    elif args.kernel == "step_trace":
        return step_trace(args)
    else:
        raise ValueError(f"unknown kernel {args.kernel!r}")
    return 0


def step_trace(args) -> int:
    """Where a captured single-token step's time goes, from time stamps the kernels take themselves when
    the library is compiled with ``-DIDM_TRACE`` (``IDM_EXTRA_NVCC_FLAGS=-DIDM_TRACE IDM_BUILD_DIR=<a
    folder of its own>``): the last layer's four products and its attention on one clock, and the
    phases of every work item of the attention kernel.  The stamps cost a few percent of the step."""
    import ctypes
    import numpy as np
    from . import from_random
    from .config.presets import preset
    B = args.batch
    lm = from_random(preset(args.size), seed=0, dtype="bfloat16", max_tokens=B * args.capacity, max_seqs=B,
                     max_seq_len=args.capacity)
    eng, L = lm.engine, lm.model.rt.kernels.lib
    if not hasattr(L, "idm_gemm_block_trace_read"):
        raise SystemExit("step_trace needs a library compiled with IDM_EXTRA_NVCC_FLAGS=-DIDM_TRACE")
    for name in ("idm_gemm_block_trace_read", "idm_attention_item_trace_read"):
        getattr(L, name).restype = ctypes.c_int
    L.idm_gemm_block_trace_read.argtypes = [ctypes.c_void_p]
    L.idm_attention_item_trace_read.argtypes = [ctypes.c_void_p, ctypes.c_int]
    g = torch.Generator().manual_seed(0)
    slots = [eng.open() for _ in range(B)]
    cur = []
    for s in slots:
        ids = torch.randint(100, 50000, (args.context,), generator=g).tolist()
        cur.append(eng.sample(eng.step([(s, ids)]), 0.0, 0, [0], [0])[0])
    step = lambda i: eng.step_sample([(s, [t]) for s, t in zip(slots, cur)], 0.0, 0, list(range(B)), [i] * B)[0]
    for i in range(6):
        cur = step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.reps):
        cur = step(10 + i)
    e1.record(); torch.cuda.synchronize()
    print(f"{args.size} batch {B} context {args.context}: {e0.elapsed_time(e1) / args.reps:.3f} ms per step with the stamps in")
    items = np.zeros((512, 4, 8), dtype=np.uint64)
    L.idm_attention_item_trace_read(items.ctypes.data, 1)          # (clear)
    torch.cuda.synchronize()
    cur = step(99)
    torch.cuda.synchronize()
    L.idm_attention_item_trace_read(items.ctypes.data, 0)
    blocks = np.zeros((5, 512, 5), dtype=np.uint64)
    L.idm_gemm_block_trace_read(blocks.ctypes.data)
    items, blocks = items.astype(np.int64), blocks.astype(np.int64)
    # products of the last layer: [kind][block] = wait for the kernel before over, first operands, accumulator ready, done, block started
    # (a residual product counts as kind 1 when its inner axis has more than 32 k-blocks, else 0)
    q = blocks[3][blocks[3][:, 0] > 0]
    t0 = q[:, 0].min()
    pct = lambda v: "/".join(f"{x / 1e3:.1f}" for x in np.percentile(v, [0, 50, 100]))
    print("the last layer, microseconds after its q/k/v product's wait for the kernel before it was over (min/median/max over blocks)")
    for kind, name in ((3, "q/k/v"), (0, "residual product, short inner axis"), (2, "gate/up"), (1, "residual product, long inner axis")):
        x = blocks[kind][blocks[kind][:, 0] > 0]
        if len(x):
            print(f"  {name}: {len(x)} blocks; started {pct(x[:, 4] - t0)}; wait over {pct(x[:, 0] - t0)}; "
                  f"accumulator ready {pct(x[:, 2] - t0)}; done {pct(x[:, 3] - t0)}")
    live = items[:, 0, 6] > 0
    if live.any():
        print(f"  attention (single tokens): {live.sum()} blocks; started {pct(items[live, 0, 6] - t0)}; rehearsal and wait over {pct(items[live, 0, 5] - t0)}")
        for nth in range(4):
            m = live & (items[:, nth, 0] >= items[:, 0, 5]) & (items[:, nth, 4] > 0)   # (stamps older than this launch are left out)
            if not m.any():
                continue
            x = items[m, nth, :5] - t0
            ph = np.diff(x, axis=1)
            print(f"    item {nth} of a block: {m.sum()} blocks; described {pct(x[:, 0])}; scores {pct(ph[:, 0])}; softmax {pct(ph[:, 1])}; "
                  f"context {pct(ph[:, 2])}; result written {pct(ph[:, 3])}; done {pct(x[:, 4])}")
    return 0
