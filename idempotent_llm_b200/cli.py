"""Command line, in the manner of the reference's scripts.

``demo``  scripts/demo.py: one fixed prompt, several ways of running it (alone, with 7
          junk co-prompts, prompt fed as prefill + single tokens), a chain hash over the
          logits of every generated step and over the token ids; options ``--config``,
          ``--steps``, ``--artifact``, ``--checkpoint-every`` as there (demo.py:266-278).
``bench`` scripts/bench.py: ``--model``, ``--batch``, ``--prompt-len``, ``--decode-steps``,
          ``--prefill-len`` as there (bench.py:92-100); decode tok/s = batch * steps / time in
          steady state, prefill tok/s = batch * prefill_len / time of one step call.
``generate``  token ids in, token ids out.
``random``    write a model folder with seeded random weights.
``replay``    the trace replay program (also ``bin/trace_run``).
``kernel-bench``  one kernel alone at a preset's layer sizes (the commands under profiles/ use it).

The reference's tokenizer is a library black box (demo.py:82-87); this command line
takes and prints token ids.
"""

from __future__ import annotations

import argparse
import hashlib
import sys
import time
from typing import List

import torch


class HashChain:
    """h_i = sha256(h_{i-1} || bytes_i), as scripts/demo.py:58-71."""

    def __init__(self, every: int = 0, marks=(64, 128, 256, 512)):
        self.h = hashlib.sha256(b"detllm-demo-v1").digest()
        self.steps: List[str] = []
        self.at = {}
        self.every, self.marks = every, marks

    def update(self, data: bytes):
        self.h = hashlib.sha256(self.h + data).digest()
        self.steps.append(self.h.hex()[:16])
        n = len(self.steps)
        if (self.every and n % self.every == 0) or (not self.every and n in self.marks):
            self.at[n] = self.h.hex()[:16]


def _demo_prompt(vocab: int, n: int = 64) -> List[int]:
    g = torch.Generator().manual_seed(18)
    return torch.randint(min(100, vocab - 1), min(50000, vocab), (n,), generator=g).tolist()


def _co_prompts(n: int, vocab: int) -> List[List[int]]:
    """Seeded junk co-prompts, lengths 5-39, ids 100-49 999 (scripts/demo.py:90-94)."""
    g = torch.Generator().manual_seed(1234)
    out = []
    for _ in range(n):
        L = int(torch.randint(5, 40, (1,), generator=g))
        out.append(torch.randint(min(100, vocab - 1), min(50000, vocab), (L,), generator=g).tolist())
    return out


def _run_demo_config(lm, name: str, steps: int, every: int):
    eng = lm.engine
    prompt = _demo_prompt(lm.spec.vocab_size)
    tok_chain, logit_chain = HashChain(every), HashChain(every)
    rows = []

    def on_step(reqs, picked, logits):
        if 0 in reqs:
            i = reqs.index(0)
            rows.append((picked[i], logits[i].detach().cpu()))

    from .engine.generate import generate
    if name == "b1":
        generate(eng, [prompt], steps, on_step=on_step)
    elif name == "b8":
        generate(eng, [prompt] + _co_prompts(7, lm.spec.vocab_size), steps, on_step=on_step)
    elif name == "split":
        half = len(prompt) // 2
        slot = eng.open()
        lg = eng.step([(slot, prompt[:half])])
        for t in prompt[half:]:
            lg = eng.step([(slot, [t])])
        for step in range(steps):
            tok = eng.sample(lg, 0.0, 0, [0], [step])[0]
            rows.append((tok, lg[0].detach().cpu()))
            if step + 1 < steps:
                lg = eng.step([(slot, [tok])])
        eng.close(slot)
    else:
        raise ValueError(f"unknown demo config {name!r}; b1, b8, split")
    for tok, lg in rows:
        tok_chain.update(int(tok).to_bytes(8, "little"))
        logit_chain.update(lg.numpy().astype("<f4").tobytes())
    for c in (tok_chain, logit_chain):
        c.at.setdefault(len(c.steps), c.h.hex()[:16])
    return tok_chain, logit_chain, rows


def cmd_demo(args) -> int:
    from . import api
    with open(f"{args.artifact}/model.safetensors", "rb") as f:
        sha = hashlib.sha256(f.read()).hexdigest()
    print(f"artifact sha256: {sha[:16]}…")
    print(f"hardware: GPU={torch.cuda.get_device_name(0)} | torch {torch.__version__} | dtype {args.dtype}\n")
    lm = api.load(args.artifact, dtype=args.dtype, max_tokens=64 * 8 * (2 + (64 + args.steps) // 64))
    names = [args.config] if args.config else ["b1", "b8", "split"]
    results = {}
    for n in names:
        t0 = time.perf_counter()
        results[n] = _run_demo_config(lm, n, args.steps, args.checkpoint_every or 0)
        tc, lc, _ = results[n]
        print(f"{n:<6} ({args.steps} tokens, {time.perf_counter() - t0:.1f}s)")
        for k in sorted(lc.at):
            print(f"  @{k:<4} tokens {tc.at[k]}   logits {lc.at[k]}")
    ok = True
    base = names[0]
    for n in names[1:]:
        ta, la, ra = results[base]
        tb, lb, rb = results[n]
        tdiv = next((i for i, (x, y) in enumerate(zip(ta.steps, tb.steps)) if x != y), None)
        ldiv = next((i for i, (x, y) in enumerate(zip(la.steps, lb.steps)) if x != y), None)
        worst = max(float((a[1] - b[1]).abs().max()) for a, b in zip(ra, rb))
        print(f"{n} vs {base}: tokens {'identical' if tdiv is None else f'diverge @ {tdiv}'}; logits "
              f"{'bit-identical' if ldiv is None else f'differ from step {ldiv}'} (max |diff| {worst:.3g})")
        if args.dtype == "float32" and ldiv is not None:
            ok = False                      # the 32-bit path promises identical bits across these cuts
    print("\nVERDICT:", "consistent" if ok else "32-BIT DIVERGENCE — this is a bug")
    return 0 if ok else 1


def cmd_bench(args) -> int:
    from . import api
    from .config.presets import preset
    cfg = preset(args.size)
    dtype = {"bf16": "bfloat16", "fp32": "float32"}[args.model]
    ctx = args.prompt_len + args.decode_steps + 16
    lm = api.from_random(cfg, seed=0, dtype=dtype, max_tokens=max(args.batch * (-(-ctx // 64) * 64),
                                                                   -(-args.prefill_len // 64) * 64 * args.batch),
                         max_seqs=args.batch, use_graph=not args.no_graph)
    # --profile-range: the CUDA profiler is switched on around the timed decode steps or the last
    # prompt step only (for `ncu --profile-from-start off`)
    prof = torch.cuda.profiler
    eng = lm.engine
    g = torch.Generator().manual_seed(0)
    V = cfg.vocab_size
    ids = torch.randint(min(100, V - 1), min(50000, V), (args.batch, args.prompt_len), generator=g).tolist()
    slots = [eng.open() for _ in ids]
    lg = eng.step(list(zip(slots, ids)))
    cur = eng.sample(lg, 0.0, 0, list(range(args.batch)), [0] * args.batch)
    for _ in range(10):
        cur = eng.sample(eng.step([(s, [t]) for s, t in zip(slots, cur)]), 0.0, 0, list(range(args.batch)),
                         [0] * args.batch)
    torch.cuda.synchronize()
    if args.profile_range == "decode":
        prof.start()
    t0 = time.perf_counter()
    for _ in range(args.decode_steps):
        cur = eng.sample(eng.step([(s, [t]) for s, t in zip(slots, cur)]), 0.0, 0, list(range(args.batch)),
                         [0] * args.batch)
    torch.cuda.synchronize()
    decode_tps = args.batch * args.decode_steps / (time.perf_counter() - t0)
    if args.profile_range == "decode":
        prof.stop()
    for s in slots:
        eng.close(s)
    pids = torch.randint(min(100, V - 1), min(50000, V), (args.batch, args.prefill_len), generator=g).tolist()
    prefill_tps = 0.0
    for it in range(2):
        slots = [eng.open() for _ in pids]
        torch.cuda.synchronize()
        if args.profile_range == "prefill" and it == 1:
            prof.start()
        t0 = time.perf_counter()
        eng.step(list(zip(slots, pids)))
        torch.cuda.synchronize()
        prefill_tps = args.batch * args.prefill_len / (time.perf_counter() - t0)
        if args.profile_range == "prefill" and it == 1:
            prof.stop()
        for s in slots:
            eng.close(s)
    print(f"{args.model} {args.size} batch={args.batch}: decode {decode_tps:.1f} tok/s, prefill {prefill_tps:.0f} tok/s")
    return 0


def cmd_kernel_bench(args) -> int:
    from .kernel_bench import run
    return run(args)


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def cmd_generate(args) -> int:
    from . import api
    prompts = [_ids(p) for p in args.prompt_ids]
    longest = max(len(p) for p in prompts) + args.max_new
    lm = api.load(args.artifact, dtype=args.dtype, max_tokens=len(prompts) * (-(-longest // 64) * 64))
    stops = _ids(args.stop_ids) if args.stop_ids else (list(lm.spec.stop_token_ids) if args.stop_at_eos else [])
    res = lm.generate_requests(prompts, args.max_new, temperature=args.temperature, seed=args.seed,
                               stop_token_ids=stops)
    for r in res:
        print(f"request {r.request} ({r.finish_reason}): {' '.join(map(str, r.tokens))}")
    return 0


def cmd_random(args) -> int:
    from .config.presets import preset
    from .weights import write_random_model
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    write_random_model(preset(args.size), args.out, seed=args.seed, dtype=dt)
    print(args.out)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="idempotent_llm_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)

    d = sub.add_parser("demo", help="hash chains of one prompt run several ways")
    d.add_argument("--config", help="run one configuration: b1, b8 or split")
    d.add_argument("--steps", type=int, default=512, help="generated tokens for every config (default 512)")
    d.add_argument("--artifact", required=True, help="model folder")
    d.add_argument("--checkpoint-every", type=int, metavar="N")
    d.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    d.set_defaults(fn=cmd_demo)

    b = sub.add_parser("bench", help="decode and prefill throughput with random weights")
    b.add_argument("--model", choices=["bf16", "fp32"], default="bf16")
    b.add_argument("--size", default="qwen3-0.6b")
    b.add_argument("--batch", type=int, default=1)
    b.add_argument("--prompt-len", type=int, default=128)
    b.add_argument("--decode-steps", type=int, default=64)
    b.add_argument("--prefill-len", type=int, default=2048)
    b.add_argument("--no-graph", action="store_true", help="single-token steps launch their kernels one by one")
    b.add_argument("--profile-range", choices=["decode", "prefill"], default=None,
                   help="switch the CUDA profiler on around the timed decode steps or the last prompt step")
    b.set_defaults(fn=cmd_bench)

    g = sub.add_parser("generate", help="token ids in, token ids out")
    g.add_argument("--artifact", required=True)
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--prompt-ids", action="append", required=True, help="'5 17 3' or '5,17,3'; repeatable")
    g.add_argument("--max-new", type=int, default=32)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--stop-at-eos", action="store_true")
    g.add_argument("--stop-ids", default="")
    g.set_defaults(fn=cmd_generate)

    r = sub.add_parser("random", help="write a model folder with seeded random weights")
    r.add_argument("--size", required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.set_defaults(fn=cmd_random)

    k = sub.add_parser("kernel-bench", help="one kernel alone at a preset's layer sizes")
    k.add_argument("--kernel", required=True, choices=["attention_single", "attention_single_mma", "attention_prompt", "gemm", "gemm_fused"])
    k.add_argument("--size", default="qwen3-0.6b")
    k.add_argument("--batch", type=int, default=8)
    k.add_argument("--context", type=int, default=3000)
    k.add_argument("--capacity", type=int, default=4096)
    k.add_argument("--tokens", type=int, default=8)
    k.add_argument("--reps", type=int, default=10)
    k.set_defaults(fn=cmd_kernel_bench)

    p = sub.add_parser("replay", help="trace replay (same as bin/trace_run)", add_help=False)
    p.set_defaults(fn=None)

    if argv is None:
        argv = sys.argv[1:]
    if argv and argv[0] == "replay":
        from .engine.replay import main as replay_main
        return replay_main(argv[1:])
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
