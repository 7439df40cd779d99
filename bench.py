"""Benchmark of the serving step on one GPU: decode tokens a second at batch 8 with the layer
sizes of Qwen3-0.6B (random weights, cache of 4 096 tokens per sequence, prompts of unequal
lengths), the same through the Python entry point, a prefill of 2 048 tokens, and decode at batch
1 and 64.  Metric definitions follow the reference's scripts/bench.py:28-63 (decode tok/s =
batch * steps / time in steady state with the greedy pick included; prefill tok/s = tokens / time
of one step call after warm-up).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  A "step" is one decode step.  Timed on the device with CUDA events; every
step reads far more than the 126 MB L2 holds (weights 1.2 GB plus the cache), so no flush is needed
between iterations.
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


def prompt_lengths(batch: int, context: int, reserve: int, seed: int):
    """Unequal prompt lengths between half the context and what leaves room for the decode steps."""
    import torch
    g = torch.Generator().manual_seed(seed)
    lo, hi = context // 2, context - reserve
    return [int(torch.randint(lo, hi + 1, (1,), generator=g)) for _ in range(batch)]


def decode_point(lm, batch: int, context: int, steps: int, warmup: int, seed: int, sampler=None):
    """Steady-state decode at ``batch``: returns (tokens/s, ms/step, bytes read per step, launches/step)."""
    import torch
    eng, cfg = lm.engine, lm.config
    V = cfg.vocab_size
    lens = prompt_lengths(batch, context, steps + warmup + 8, seed)
    g = torch.Generator().manual_seed(seed + 1)
    slots = [eng.open() for _ in lens]
    first = []
    # prompts go in one sequence at a time: the prefill is set-up here, not what is measured
    for s, n in zip(slots, lens):
        ids = torch.randint(min(100, V - 1), min(50000, V), (n,), generator=g).tolist()
        lg = eng.step([(s, ids)])
        first.append(eng.sample(lg, 0.0, 0, [0], [0])[0])
    sess = eng.decode_session(slots, first, steps + warmup)
    sess.run(warmup)
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    sess.run(steps)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    sess.finish()
    kv_per_token = sum(2 * g_.need.n_kv_heads * g_.need.head_dim * g_.k.element_size() * len(g_.entries)
                       for g_ in eng.cache.groups)
    mean_len = sum(l + warmup + steps / 2 for l in lens)
    bytes_step = lm.model.weight_bytes() + kv_per_token * mean_len
    launches = sess.launches_per_step
    toks = sess.tokens()
    assert toks.shape == (steps + warmup, batch) and int(toks.min()) >= 0 and int(toks.max()) < V
    for s in slots:
        eng.close(s)
    return batch * 1000.0 / ms, ms, bytes_step, launches, lens


def e2e_point(lm, batch: int, context: int, steps: int, warmup: int, seed: int):
    """The same decode through the public ``step_sample`` call (what ``generate`` runs per step):
    every step copies its tokens from pinned host memory to the device and reads the chosen tokens
    back."""
    import torch
    eng, cfg = lm.engine, lm.config
    V = cfg.vocab_size
    lens = prompt_lengths(batch, context, steps + warmup + 8, seed)
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


def prefill_point(lm, tokens: int, warmup: int, iters: int, seed: int):
    import torch
    eng, cfg = lm.engine, lm.config
    V = cfg.vocab_size
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(min(100, V - 1), min(50000, V), (tokens,), generator=g).tolist()
    times = []
    for i in range(warmup + iters):
        slot = eng.open()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        eng.step([(slot, ids)])
        t1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(t0.elapsed_time(t1))
        eng.close(slot)
    ms = statistics.median(times)
    H, L = cfg.hidden_size, cfg.num_hidden_layers
    qd, kd = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    linear = 2 * tokens * L * (H * (qd + 2 * kd) + qd * H + 3 * H * cfg.intermediate_size)
    attn = L * cfg.num_attention_heads * 4 * cfg.head_dim * tokens * (tokens + 1) // 2
    head = 2 * H * V
    return tokens * 1000.0 / ms, ms, linear + attn + head


def reference_arm():
    """The reference cannot be run here: its runtime loads an int8 artifact that only
    ``detllm.prepare`` makes, and that downloads the checkpoint and a calibration set
    (src/detllm/prepare.py:172, 236-240); there is no network."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "offline install fails (build backend uv_build is not in the wheelhouse), and the reference "
                      "runs only from an artifact that detllm.prepare builds by downloading Qwen/Qwen3-0.6B and "
                      "WikiText2 (prepare.py:172,236-240); no network here"}))
    return 0


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
    ap.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not built (this library runs on one device)")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    import idempotent_llm_b200 as idm
    from idempotent_llm_b200.config.presets import preset, preset_dict

    full_layers = preset_dict(args.size)["num_hidden_layers"]
    cfg = preset(args.size, **({"num_hidden_layers": args.layers, "max_window_layers": args.layers}
                              if args.layers else {}))
    pk = peaks()
    big = 64 if not args.skip_points else args.batch
    lm = idm.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=max(big, args.batch) * args.context,
                         max_seqs=max(big, args.batch), max_seq_len=args.context)
    kern = lm.model.rt.kernels

    sampler = ClockSampler()
    tps, ms, bytes_step, launches, lens = decode_point(lm, args.batch, args.context, args.steps, args.warmup, 1,
                                                       sampler)
    clocks = sampler.stop()
    e2e, h2d, d2h = e2e_point(lm, args.batch, args.context, args.steps, args.warmup, 1)
    p_tps, p_ms, p_flops = prefill_point(lm, 2048, 3, 5, 2)
    points = {}
    if not args.skip_points:
        points["decode_b1"] = decode_point(lm, 1, args.context, min(args.steps, 64), args.warmup, 3)[0]
        points["decode_b64"] = decode_point(lm, 64, args.context, min(args.steps, 32), args.warmup, 4)[0]
    gbs = bytes_step / (ms * 1e-3) / 1e9
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
        },
        "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches * args.steps,
        "prefill": {"value": p_tps, "tokens": 2048, "ms": p_ms,
                    "frac": p_flops / (p_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / pk["hbm_gbs"], "peaks": pk["source"]},
        "points": points,
        "clocks": clocks,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
