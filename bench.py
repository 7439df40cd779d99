"""Benchmark of the serving step on one GPU: decode tokens a second at batch 8 with the layer
sizes of Qwen3-0.6B (random weights, cache of 4 096 tokens per sequence, prompts of unequal
lengths), the same through the Python entry point, a prefill of 2 048 tokens, and decode at batch
1 and 64.  Metric definitions follow the reference's scripts/bench.py:28-63 (decode tok/s =
batch * steps / time in steady state with the greedy pick included; prefill tok/s = tokens / time
of one step call after warm-up).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  A "step" is one decode step.  Timed on the device with CUDA events (the median
of several timed regions of --steps steps); every step reads far more than the 126 MB L2 holds (weights
1.2 GB plus the cache), so no flush is needed between iterations.  ``points`` holds decode at batch 1 and
64, a prefill of 512 tokens, and the 8B and 32B layer sizes of the other benchmark configurations (decode
tokens a second with the fraction of the memory roofline, prefill with the fraction of the bfloat16 peak);
``check`` compares bfloat16 with the true 32-bit path at the headline's layer sizes.  ``--impl reference``
runs the unmodified reference (``baseline/reference_arm.py``).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PUBLISHED_A100_DECODE_B8 = 783.3     # the reference's best published batch-8 figure (docs/RESULTS.md:114)


def peaks():
    p = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                m = json.load(f)
            hbm, flops = _number(m.get("hbm_gbs")), _number(m.get("bf16_tflops"))
            if hbm and flops:                      # both or neither: one source for the whole line
                p.update(hbm_gbs=hbm, bf16_tflops=flops, source="measured")
        except (ValueError, OSError, TypeError, AttributeError):
            pass
    return p


def _number(v):
    """A figure of the measured-peaks file: a number, or a record or list that holds one."""
    if isinstance(v, bool) or v is None:
        return None
    if isinstance(v, (int, float)):
        return float(v) if v > 0 else None
    if isinstance(v, dict):
        for key in ("value", "median", "mean", "max"):
            if key in v:
                return _number(v[key])
        return None
    if isinstance(v, (list, tuple)) and v:
        return _number(v[0])
    return None


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v == "Active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}




def prompt_lengths(batch: int, lo: int, hi: int, seed: int):
    """Unequal prompt lengths, uniform in [lo, hi]."""
    import torch
    g = torch.Generator().manual_seed(seed)
    return [int(torch.randint(lo, hi + 1, (1,), generator=g)) for _ in range(batch)]


def headline_lengths(batch: int, context: int, reserve: int, seed: int):
    """The headline's prompts: between half the context and what leaves room for the decode steps."""
    return prompt_lengths(batch, context // 2, context - reserve, seed)


def kv_bytes_per_token(eng) -> int:
    return sum(2 * g_.need.n_kv_heads * g_.need.head_dim * g_.k.element_size() * len(g_.entries)
               for g_ in eng.cache.groups)


def decode_point(lm, lens, steps: int, warmup: int, seed: int, repeats: int = 1, sampler=None):
    """Steady-state decode of a batch with prompts of ``lens`` tokens: ``repeats`` timed regions of ``steps``
    steps each after ``warmup`` steps; the median region counts.  Returns tokens/s, ms per step, the bytes a
    step has to read (every weight once, the cache of the live sequences) and launches per step."""
    import torch
    eng, cfg = lm.engine, lm.config
    V, batch = cfg.vocab_size, len(lens)
    g = torch.Generator().manual_seed(seed + 1)
    slots = [eng.open() for _ in lens]
    first = []
    # prompts go in one sequence at a time: the prefill is set-up here, not what is measured
    for s, n in zip(slots, lens):
        ids = torch.randint(min(100, V - 1), min(50000, V), (n,), generator=g).tolist()
        lg = eng.step([(s, ids)])
        first.append(eng.sample(lg, 0.0, 0, [0], [0])[0])
    total = warmup + repeats * steps
    sess = eng.decode_session(slots, first, total)
    sess.run(warmup)
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
    times = []
    for _ in range(repeats):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        sess.run(steps)
        t1.record()
        torch.cuda.synchronize()
        times.append(t0.elapsed_time(t1) / steps)
    ms = statistics.median(times)
    sess.finish()
    mean_len = sum(l + warmup + repeats * steps / 2 for l in lens)
    bytes_step = lm.model.weight_bytes() + kv_bytes_per_token(eng) * mean_len
    toks = sess.tokens()
    assert toks.shape == (total, batch) and int(toks.min()) >= 0 and int(toks.max()) < V
    for s in slots:
        eng.close(s)
    return {"tps": batch * 1000.0 / ms, "ms": ms, "bytes": bytes_step, "launches": sess.launches_per_step,
            "ms_min": min(times), "ms_max": max(times)}


def e2e_point(lm, lens, steps: int, warmup: int, seed: int):
    """The same decode through the public ``step_sample`` call (what ``generate`` runs per step):
    every step copies its tokens from pinned host memory to the device and reads the chosen tokens
    back."""
    import torch
    eng, cfg = lm.engine, lm.config
    V, batch = cfg.vocab_size, len(lens)
    g = torch.Generator().manual_seed(seed + 1)
    slots = [eng.open() for _ in lens]
    cur = []
    for s, n in zip(slots, lens):
        ids = torch.randint(min(100, V - 1), min(50000, V), (n,), generator=g).tolist()
        cur.append(eng.sample(eng.step([(s, ids)]), 0.0, 0, [0], [0])[0])
    reqs = list(range(batch))

    def one(step):
        nonlocal cur
        cur, _ = eng.step_sample([(s, [t]) for s, t in zip(slots, cur)], 0.0, 0, reqs, [step] * batch)
    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(steps):
        one(warmup + i)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    for s in slots:
        eng.close(s)
    # per step: the packed step (7 ints per sequence, one more, the wanted rows; an even count) goes up,
    # one chosen token per sequence comes back
    return batch * steps / dt, (8 * batch + 1 + 1) // 2 * 2 * 4, batch * 4


def prefill_flops(cfg, lens) -> float:
    """Multiply-adds x 2 of a step that brings whole prompts of ``lens`` tokens: the layers' products, causal
    attention, and the head at each prompt's last position."""
    H, L, V = cfg.hidden_size, cfg.num_hidden_layers, cfg.vocab_size
    qd, kd = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    tokens = sum(lens)
    linear = 2 * tokens * L * (H * (qd + 2 * kd) + qd * H + 3 * H * cfg.intermediate_size)
    attn = sum(L * cfg.num_attention_heads * 4 * cfg.head_dim * t * (t + 1) // 2 for t in lens)
    return linear + attn + 2 * H * V * len(lens)


def prefill_point(lm, lens, warmup: int, iters: int, seed: int):
    """One step that brings whole prompts of ``lens`` tokens (logits at each prompt's last position):
    (tokens/s, ms, flops), the median of ``iters`` runs after ``warmup``."""
    import torch
    eng, cfg = lm.engine, lm.config
    V = cfg.vocab_size
    g = torch.Generator().manual_seed(seed)
    ids = [torch.randint(min(100, V - 1), min(50000, V), (n,), generator=g).tolist() for n in lens]
    times = []
    for i in range(warmup + iters):
        slots = [eng.open() for _ in lens]
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        eng.step(list(zip(slots, ids)))
        t1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(t0.elapsed_time(t1))
        for s in slots:
            eng.close(s)
    ms = statistics.median(times)
    return sum(lens) * 1000.0 / ms, ms, prefill_flops(cfg, lens)


def check_against_32_bit(cfg, seed: int = 0):
    """bfloat16 against the true 32-bit path at the same layer sizes and the same (bfloat16-valued) weights: a
    prompt of 200 tokens, then 8 single tokens; the largest difference of the logits relative to the largest
    logit.  The 32-bit model is built from the bfloat16 weights widened, so only the arithmetic differs."""
    import torch
    from idempotent_llm_b200.api import LM, build_model, canonical_dtype
    from idempotent_llm_b200.engine import declare_weights
    from idempotent_llm_b200.weights.random_init import random_weights
    spec = cfg.to_model_spec()
    g = torch.Generator().manual_seed(9)
    V = cfg.vocab_size
    ids = torch.randint(min(100, V - 1), min(50000, V), (208,), generator=g).tolist()
    out = {}
    for dtype in ("bfloat16", "float32"):
        w = random_weights(declare_weights(spec), seed, spec.init_std, dtype=torch.bfloat16, device="cuda:0")
        lm = LM(build_model(cfg, w, canonical_dtype(dtype), "cuda:0"), cfg, max_tokens=256, max_seqs=1)
        del w
        eng = lm.engine
        slot = eng.open()
        rows = [eng.step([(slot, ids[:200])], [[0, 63, 64, 199]])]
        for t in ids[200:]:
            rows.append(eng.step([(slot, [t])]).clone())
        eng.close(slot)
        out[dtype] = torch.cat(rows).double().cpu()
        del lm, eng
        torch.cuda.empty_cache()
    rel = float((out["bfloat16"] - out["float32"]).abs().max() / out["float32"].abs().max())
    same_pick = int((out["bfloat16"].argmax(-1) == out["float32"].argmax(-1)).sum())
    return {"bf16_vs_f32_max_rel_diff": rel, "rows": out["float32"].shape[0], "same_argmax_rows": same_pick}


# The same configuration (Qwen3-0.6B layer sizes, batch 8, cache of 4096) with the kernels this library had
# before a token's bfloat16 result was made the same bits in every batch and cut: products whose sums were
# split over blocks and clusters, single tokens summed per chunk of 256 keys.  Measured then, on this
# bench; what the cut-invariant arithmetic cost is these against today's figures.
EARLIER_KERNELS = {"decode_tok_s": 6035.2, "ms_per_step": 1.326, "prefill_2048_ms": 3.93}


def check_cuts_bitwise(lm, seed: int = 0):
    """bfloat16 logits of one request: whole in one step, cut into three steps, its last 8 tokens one by one,
    and beside another request in the batch: compared bit for bit."""
    import torch
    eng = lm.engine
    g = torch.Generator().manual_seed(seed + 77)
    V = lm.config.vocab_size
    ids = torch.randint(min(100, V - 1), min(50000, V), (300,), generator=g).tolist()
    other = torch.randint(min(100, V - 1), min(50000, V), (170,), generator=g).tolist()
    want = [0, 130, 291, 292, 299]

    def run(cuts, beside=False):
        a = eng.open()
        b = eng.open() if beside else None
        rows, at = {}, 0
        for n in cuts:
            w = [p - at for p in want if at <= p < at + n]
            entries, wants = [(a, ids[at:at + n])], [w]
            if beside and at == 0:
                entries.append((b, other)); wants.append([])
            out = eng.step(entries, wants)
            for k, p in enumerate(q for q in want if at <= q < at + n):
                rows[p] = out[k].clone()
            at += n
        eng.close(a)
        if b is not None:
            eng.close(b)
        return torch.stack([rows[p] for p in want])

    whole = run([300])
    same = all(torch.equal(whole, other_cut) for other_cut in
               (run([131, 100, 69]), run([292] + [1] * 8), run([300], beside=True)))
    return bool(same)


def reference_arm(args) -> int:
    """The unmodified reference on the same configuration: ``baseline/reference_arm.py``."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    from idempotent_llm_b200.config.presets import preset_dict
    import reference_arm as arm
    lens = headline_lengths(args.batch, args.context, args.repeats * args.steps + max(args.warmup, 3) + 8, 1)
    return arm.run(args, preset_dict(args.size), lens, ClockSampler())


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", default="qwen3-0.6b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (0: all)")
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps; the median counts")
    ap.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64 and the 32-bit check")
    ap.add_argument("--skip-sizes", action="store_true", help="leave out the points at 8B and 32B layer sizes")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not built (this library runs on one device)")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)

    import torch
    import idempotent_llm_b200 as idm
    from idempotent_llm_b200.config.presets import preset, preset_dict

    full_layers = preset_dict(args.size)["num_hidden_layers"]
    cfg = preset(args.size, **({"num_hidden_layers": args.layers, "max_window_layers": args.layers}
                              if args.layers else {}))
    pk = peaks()
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    big = 64 if not args.skip_points else args.batch
    lm = idm.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=max(big, args.batch) * args.context,
                         max_seqs=max(big, args.batch), max_seq_len=args.context)

    reserve = args.repeats * args.steps + args.warmup + 8
    lens = headline_lengths(args.batch, args.context, reserve, 1)
    sampler = ClockSampler()
    head = decode_point(lm, lens, args.steps, args.warmup, 1, args.repeats, sampler)
    clocks = sampler.stop()
    e2e, h2d, d2h = e2e_point(lm, lens, args.steps, args.warmup, 1)
    p_tps, p_ms, p_flops = prefill_point(lm, [2048], 3, 5, 2)
    points = {}
    if not args.skip_points:
        p512 = prefill_point(lm, [512], 3, 5, 5)
        points["prefill_512_tok_s"], points["prefill_512_ms"] = p512[0], p512[1]
        for b, seed in ((1, 3), (64, 4)):
            st = min(args.steps, 64 if b == 1 else 32)
            r = decode_point(lm, headline_lengths(b, args.context, 3 * st + args.warmup + 8, seed), st, args.warmup, seed, 3)
            points[f"decode_b{b}"] = r["tps"]
            points[f"decode_b{b}_hbm_frac"] = r["bytes"] / (r["ms"] * 1e-3) / hbm
    cuts_same = check_cuts_bitwise(lm)
    del lm
    torch.cuda.empty_cache()
    check = None if args.skip_points else check_against_32_bit(cfg)
    if not args.skip_sizes:
        # the other two benchmark configurations: 8B layer sizes at batch 1, 8, 64 with prompts of 128 to 2048
        # tokens, and 32B layer sizes with 8 prompts of 2048; every weight of all layers, random
        steps = min(args.steps, 32)
        c8 = preset("qwen3-8b")
        lm = idm.from_random(c8, seed=0, dtype="bfloat16", max_tokens=64 * 2304, max_seqs=64, max_seq_len=2304)
        for b, seed in ((1, 11), (8, 12), (64, 13)):
            r = decode_point(lm, prompt_lengths(b, 128, 2048, seed), steps, args.warmup, seed, 3)
            points[f"decode_8b_b{b}"] = r["tps"]
            points[f"decode_8b_b{b}_ms"] = r["ms"]
            points[f"decode_8b_b{b}_hbm_frac"] = r["bytes"] / (r["ms"] * 1e-3) / hbm
        t, ms, fl = prefill_point(lm, prompt_lengths(8, 128, 2048, 14), 2, 3, 14)
        points["prefill_8b_8_prompts_tok_s"], points["prefill_8b_8_prompts_frac"] = t, fl / (ms * 1e-3) / tf
        del lm
        torch.cuda.empty_cache()
        c32 = preset("qwen3-32b")
        lm = idm.from_random(c32, seed=0, dtype="bfloat16", max_tokens=8 * 2304, max_seqs=8, max_seq_len=2304)
        r = decode_point(lm, [2048] * 8, steps, args.warmup, 21, 3)
        points["decode_32b_b8"], points["decode_32b_b8_ms"] = r["tps"], r["ms"]
        points["decode_32b_b8_hbm_frac"] = r["bytes"] / (r["ms"] * 1e-3) / hbm
        t, ms, fl = prefill_point(lm, [2048] * 8, 1, 3, 22)
        points["prefill_32b_8x2048_tok_s"], points["prefill_32b_8x2048_frac"] = t, fl / (ms * 1e-3) / tf
        del lm
        torch.cuda.empty_cache()
    tps, ms = head["tps"], head["ms"]
    gbs = head["bytes"] / (ms * 1e-3) / 1e9
    out = {
        "metric": "decode tok/s at batch 8 (Qwen3-0.6B layer sizes, random weights, bf16, 4096-token cache)",
        "value": tps, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": tps / PUBLISHED_A100_DECODE_B8 if args.size == "qwen3-0.6b" and args.batch == 8 else None,
        "dtype": "bf16", "data": "synthetic: seeded random weights and uniform-random token ids",
        "impl": "ours",
        "config": {
            "model": args.size, "layers": cfg.num_hidden_layers, "layers_of_config": full_layers,
            "hidden": cfg.hidden_size, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "tied": cfg.tie_word_embeddings, "global_batch": args.batch, "seq_len": args.context,
            "prompt_len_min": min(lens), "prompt_len_max": max(lens), "prompt_len_mean": sum(lens) / len(lens),
            "parallelism": "single GPU", "l2": "inputs larger than L2 (weights + cache per step)",
            "decode": "CUDA graph per step: model + greedy pick + feedback on device",
            "timed": f"median of {args.repeats} regions of {args.steps} steps",
        },
        "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": head["launches"] * args.steps,
        "prefill": {"value": p_tps, "tokens": 2048, "ms": p_ms, "frac": p_flops / (p_ms * 1e-3) / tf},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / pk["hbm_gbs"], "peaks": pk["source"]},
        "points": points,
        "check": check,
        # a token's bfloat16 logits are the same bits however its sequence was cut and batched (checked on this
        # run: one request whole, in three steps, with its last tokens one by one, beside another request),
        # and what that cost against the kernels before, which split their sums
        "exactness": {"bf16_bitwise_same_across_cuts": cuts_same,
                      "earlier_kernels_decode_tok_s": EARLIER_KERNELS["decode_tok_s"],
                      "earlier_kernels_ms_per_step": EARLIER_KERNELS["ms_per_step"],
                      "earlier_kernels_prefill_2048_ms": EARLIER_KERNELS["prefill_2048_ms"],
                      "decode_now_over_earlier": (tps / EARLIER_KERNELS["decode_tok_s"]
                                                  if args.size == "qwen3-0.6b" and args.batch == 8 and not args.layers else None)},
        "spread": {"ms_per_step_min": head["ms_min"], "ms_per_step_max": head["ms_max"]},
        "clocks": clocks,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
