"""The reference arm of ``bench.py``: rishabh135/idempotent_llm ("DetLLM") itself, unmodified, on the
benchmark's configuration.

What runs.  The reference's package lies under ``baseline/_ref/detllm`` exactly as its ``src/detllm``
(pure Python; the offline ``pip install --target baseline/_ref`` fails because its build backend
``uv_build`` is not in the wheelhouse, so the package folder is placed there as that install would
place it).  Its runtime loads an int8 artifact that only ``detllm.prepare`` makes, and that downloads
the checkpoint and a calibration set; there is no network.  So the artifact is synthetic: random
weights of Qwen3-0.6B's layer sizes quantised by ``prepare.py``'s own helpers
(``quant_weight_per_channel``, ``quant_embedding_per_row``, ``fit_gamma_dyadic``,
``fit_dyadic_float(_vec)``, ``ops.rope.build_rope_tables``) with identity smoothing and fixed key/value
ranges -- what its speed depends on (shapes, dtypes, kernels) is the real thing, what its accuracy
depends on is not needed here.  Then its own stock path, as its ``scripts/bench.py:16-63`` drives it for
``--model int-graphed``: ``compile_ops()``, ``IntQwen3(artifact, backend="cuda")``, a prefill
``forward``, ``GraphedDecode(model, cache, lens)``, ``greedy_pick(gd.step(cur))`` per step.

What differs from the other arm, and is said in the printed line: int8 weights and activations (W8A8)
instead of bfloat16; prompts of ONE length (its cache keeps one length for the whole batch,
src/detllm/model.py:67-102), the mean of the other arm's unequal lengths; tied embeddings only.
None of this repository's models, kernels or engine is on this path.
"""

from __future__ import annotations

import json
import math
import os
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:600]}))
    return 0


def build_artifact(out_dir: str, cfg: dict, seed: int = 0) -> None:
    """A synthetic int8 artifact of the reference's format for ``cfg`` (the keys of its config.json)."""
    import torch
    from detllm.ops.rope import build_rope_tables
    from detllm.prepare import (fit_dyadic_float, fit_dyadic_float_vec, fit_gamma_dyadic, quant_embedding_per_row,
                                quant_weight_per_channel)
    from safetensors.torch import save_file
    L, H, NQ, NKV, HD = cfg["n_layers"], cfg["hidden"], cfg["n_q_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    I, V = cfg["intermediate"], cfg["vocab"]
    g = torch.Generator().manual_seed(seed)

    def rn(*s, std):
        return torch.randn(*s, generator=g, dtype=torch.float32).double() * std

    ten, acfg = {}, dict(cfg, layers=[])

    def add(name, Wf, gamma=None):
        w8, m, k = quant_weight_per_channel(Wf * (gamma[None, :] if gamma is not None else 1.0))
        ten[name + ".w8t"] = w8.t().contiguous()
        ten[name + ".m"] = m
        return {"k": k}
    E = rn(V, H, std=0.02)
    ten["embed.e8"], ten["embed.m"], ten["embed.k"] = quant_embedding_per_row(E)
    acfg["head"] = add("head", E, 1 + rn(H, std=0.02))
    del E
    ten["rope.cos"], ten["rope.sin"] = build_rope_tables(HD, cfg["max_pos"], cfg["rope_theta"])
    one = lambda n: torch.ones(n, dtype=torch.int64)
    # ranges of the cached keys (after norm and rotation: a few units) and values (x of unit rms times a
    # random matrix of std 0.02 over `hidden` inputs): generous fixed numbers, the same for every layer
    k_max, v_max = 8.0, 8.0 * 0.02 * math.sqrt(H)
    for i in range(L):
        ap_, Lc = f"layers.{i}.", {}
        ga, gm = 1 + rn(H, std=0.02), 1 + rn(H, std=0.02)
        for nm, shape, gam in (("q", (NQ * HD, H), ga), ("k", (NKV * HD, H), ga), ("v", (NKV * HD, H), ga),
                               ("o", (H, NQ * HD), None), ("gate", (I, H), gm), ("up", (I, H), gm), ("down", (H, I), None)):
            Lc[nm] = add(ap_ + nm, rn(*shape, std=0.02), gam)
        ten[ap_ + "q_norm.m"], Lc["q_norm_k"] = fit_gamma_dyadic(1 + rn(HD, std=0.02))
        ten[ap_ + "k_norm.m"], Lc["k_norm_k"] = fit_gamma_dyadic(1 + rn(HD, std=0.02))
        for nm, n in (("as", H), ("ms", H), ("ds", I), ("os", NQ * HD)):
            ten[ap_ + nm + "_m"] = one(n)
            Lc[nm + "_k"] = 0
        ten[ap_ + "qs_m"] = one(NKV * HD).view(NKV, HD)
        Lc["qs_k"] = 0
        s_kh = torch.full((NKV,), k_max * 1.05 / 127, dtype=torch.float64)
        ten[ap_ + "kq_m"], ten[ap_ + "kq_k"] = fit_dyadic_float_vec(s_kh[:, None].expand(NKV, HD).contiguous())
        ks = [fit_dyadic_float(float(s) / math.sqrt(HD)) for s in s_kh]
        vq = [fit_dyadic_float(v_max * 1.05 / 127) for _ in range(NKV)]
        ten[ap_ + "ks_m"] = torch.tensor([a for a, _ in ks]); ten[ap_ + "ks_k"] = torch.tensor([b for _, b in ks])
        ten[ap_ + "vq_m"] = torch.tensor([a for a, _ in vq]); ten[ap_ + "vq_k"] = torch.tensor([b for _, b in vq])
        acfg["layers"].append(Lc)
    os.makedirs(out_dir, exist_ok=True)
    save_file({k: v.contiguous() for k, v in ten.items()}, os.path.join(out_dir, "model.safetensors"))
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(acfg, f)


def run(args, preset_cfg: dict, prompt_lens, clock_sampler=None) -> int:
    """Prints the reference arm's JSON line (or its ``unavailable`` line) and returns the exit code."""
    if not os.path.isdir(os.path.join(REF, "detllm")):
        return _unavailable("baseline/_ref/detllm is not there: the reference's package was not placed beside this file")
    try:
        import torch
        if not torch.cuda.is_available():
            return _unavailable("no CUDA device")
        sys.path.insert(0, REF)
        cfg = dict(n_layers=preset_cfg["num_hidden_layers"], hidden=preset_cfg["hidden_size"],
                   n_q_heads=preset_cfg["num_attention_heads"], n_kv_heads=preset_cfg["num_key_value_heads"],
                   head_dim=preset_cfg["head_dim"], intermediate=preset_cfg["intermediate_size"],
                   vocab=preset_cfg["vocab_size"], max_pos=int(preset_cfg.get("max_position_embeddings", 40960)),
                   rope_theta=float(preset_cfg.get("rope_theta", 1e6)))
        if not preset_cfg.get("tie_word_embeddings", False):
            return _unavailable("the reference asserts tied embeddings (src/detllm/prepare.py:246); this configuration has an lm_head of its own")
        if cfg["hidden"] > 1024:
            return _unavailable("the reference's integer norm keeps its sums in range for hidden <= 1024 only (src/detllm/ops/di_rmsnorm.py:16-17)")
        batch, steps, warmup = args.batch, args.steps, max(args.warmup, 3)
        prompt_len = int(round(sum(prompt_lens) / len(prompt_lens)))
        t_build = time.perf_counter()
        art = tempfile.mkdtemp(prefix="detllm-artifact-")
        build_artifact(art, cfg)
        t_build = time.perf_counter() - t_build

        from detllm.compile import compile_ops
        compile_ops()
        from detllm.graphed import GraphedDecode
        from detllm.model import IntQwen3
        g = torch.Generator().manual_seed(2)
        V = cfg["vocab"]
        ids = torch.randint(min(100, V - 1), min(50000, V), (batch, prompt_len), generator=g).cuda()
        pos = torch.arange(prompt_len, device="cuda").expand(batch, prompt_len)
        # Its scripts/bench.py runs GraphedDecode with its defaults (one compiled layer graph inside the captured
        # step).  Where this box's torch cannot compile that, the same class is asked, through its own
        # parameter, to capture the step over the per-operator compiled functions instead; what ran is said
        # in the printed line, with the message of what did not.
        attempts = (("GraphedDecode(model, cache, lens): its bench's int-graphed path", {}),
                    ("GraphedDecode(model, cache, lens, layer_compile=False): the step captured over the "
                     "per-operator compiled functions", {"layer_compile": False}))
        failed, mode = [], None
        for mode, kw in attempts:
            t_setup = time.perf_counter()
            try:
                with torch.no_grad():
                    model = IntQwen3(art, backend="cuda")
                    logits, _, _, cache = model.forward(ids, pos)
                    lens = torch.full((batch,), prompt_len, dtype=torch.int64, device="cuda")
                    gd = GraphedDecode(model, cache, lens, **kw)
                    cur = model.greedy_pick(logits[:, -1])
                    del logits
                    for _ in range(warmup):
                        cur = model.greedy_pick(gd.step(cur))
                    torch.cuda.synchronize()
                t_setup = time.perf_counter() - t_setup
                break
            except Exception as e:
                failed.append(f"{mode.split(':')[0]} failed: {type(e).__name__}: {' '.join(str(e).split())[:300]}")
                mode = None
                del e
                model = cache = gd = None
                import gc
                gc.collect()
                torch.cuda.empty_cache()
                torch._dynamo.reset()
        if mode is None:
            return _unavailable("the reference's stock paths failed here: " + " | ".join(failed))
        with torch.no_grad():
            if clock_sampler is not None:
                clock_sampler.start()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                cur = model.greedy_pick(gd.step(cur))
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
            clocks = clock_sampler.stop() if clock_sampler is not None else None
            # end to end: every step's tokens go up from pinned host memory and the chosen ones come back
            host = torch.empty(batch, dtype=torch.int64).pin_memory()
            host.copy_(cur.cpu())
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                dev = host.to("cuda", non_blocking=True)
                host.copy_(model.greedy_pick(gd.step(dev)))          # device -> host: waits for the step
            torch.cuda.synchronize()
            e2e = batch * steps / (time.perf_counter() - t0)
            # its prefill figure: one forward of 2048 tokens after one warm-up, logits at every position
            # (scripts/bench.py:54-63)
            p_tps = p_ms = None
            try:
                pids = torch.randint(min(100, V - 1), min(50000, V), (1, 2048), generator=g).cuda()
                ppos = torch.arange(2048, device="cuda").expand(1, 2048)
                model.forward(pids, ppos)
                torch.cuda.synchronize()
                p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                p0.record()
                model.forward(pids, ppos)
                p1.record()
                torch.cuda.synchronize()
                p_ms = p0.elapsed_time(p1)
                p_tps = 2048 * 1000.0 / p_ms
            except Exception as e:          # the decode figure stands without it
                p_tps, p_ms = None, f"{type(e).__name__}: {e}"[:200]
        out = {
            "metric": "decode tok/s at batch 8 (Qwen3-0.6B layer sizes, random weights, 4096-token cache)",
            "impl": "reference", "value": batch * 1000.0 / ms, "unit": "tok/s", "n_gpus": 1, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 (W8A8, the reference's only arithmetic)", "data": "synthetic: seeded random weights "
            "quantised by the reference's own helpers, uniform-random token ids",
            "same_config": False,
            "differs": "int8 weights and activations instead of bf16; all prompts of one length (the mean of the other "
                       "arm's unequal lengths); artifact synthetic (no calibration)",
            "ran": mode, "did_not_run": failed,
            "config": {"model": args.size, "layers": cfg["n_layers"], "hidden": cfg["hidden"], "q_heads": cfg["n_q_heads"],
                       "kv_heads": cfg["n_kv_heads"], "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate"],
                       "vocab": cfg["vocab"], "tied": True, "global_batch": batch, "seq_len": args.context,
                       "prompt_len": prompt_len, "parallelism": "single GPU",
                       "decode": "the reference's GraphedDecode (whole-step CUDA graph) + greedy_pick"},
            "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": batch * 8, "d2h_bytes_per_step": batch * 8},
            "prefill": {"value": p_tps, "tokens": 2048, "ms": p_ms, "logits": "every position (the reference's forward)"},
            "setup_s": {"artifact": round(t_build, 1), "load_compile_capture": round(t_setup, 1)},
            "clocks": clocks,
        }
        print(json.dumps(out))
        import shutil
        shutil.rmtree(art, ignore_errors=True)
        return 0
    except Exception as e:                      # anything the stock path cannot do on this box
        import traceback
        tb = traceback.extract_tb(e.__traceback__)
        where = f"{os.path.basename(tb[-1].filename)}:{tb[-1].lineno}" if tb else "?"
        return _unavailable(f"the reference's stock path failed here: {type(e).__name__}: {e} (at {where})")
