"""Command line, in the manner of the reference's scripts.

``demo``  scripts/demo.py: one fixed prompt, several ways of running it (alone, with 7
          junk co-prompts, prompt fed as prefill + single tokens), a chained digest over the
          logits of every generated step and over the token ids; options ``--config``,
          ``--steps``, ``--artifact``, ``--checkpoint-every`` as there (demo.py:266-278).  Exit 1 if
          any two ways differ in a bit, in either precision.  The reference's fourth way, the same
          model on the CPU as a witness from another device (demo.py:101-164), has no counterpart here
          (there is no CPU path); ``--save-chains`` / ``--against`` compare runs, days and machines
          instead, and the CPU witness of the arithmetic is the plain implementation under ``tests/``.
``bench`` scripts/bench.py: ``--model``, ``--batch``, ``--prompt-len``, ``--decode-steps``,
          ``--prefill-len`` as there (bench.py:92-100); decode tok/s = batch * steps / time in
          steady state, prefill tok/s = batch * prefill_len / time of one step call.
``generate``  token ids in, token ids out.
``random``    write a model folder with seeded random weights.
``replay``    the trace replay program (also ``bin/trace_run``).
``kernel-bench``  one kernel alone at a preset's layer sizes (``kernel_bench.py``).

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


class ChainedDigest:
    """A running SHA-256 over a sequence of records: the state after record i is
    ``sha256(state before || record i)``, starting from a fixed tag.  Two runs agree on their first i
    records exactly if their i-th states agree, so the first state that differs names the first step
    that diverged.  (The reference's demo chains its logits and token ids this way,
    scripts/demo.py:58-71.)"""

    TAG = b"idempotent_llm_b200 chained digest, version 1"

    def __init__(self):
        self._state = hashlib.sha256(self.TAG).digest()
        self.prefixes: List[str] = []          # the first 16 hex digits of every state, in order

    def add(self, record: bytes) -> None:
        self._state = hashlib.sha256(self._state + record).digest()
        self.prefixes.append(self._state.hex()[:16])

    def checkpoints(self, every: int = 0, marks=(64, 128, 256, 512)) -> dict:
        """record count -> state, at every ``every``-th record (or at ``marks``) and at the end."""
        n = len(self.prefixes)
        at = [k for k in range(1, n + 1) if (every and k % every == 0) or (not every and k in marks)]
        return {k: self.prefixes[k - 1] for k in sorted(set(at + ([n] if n else [])))}

    @staticmethod
    def first_difference(a: List[str], b: List[str]):
        """Index of the first record at which two chains differ (a shorter chain differs where it ends), or None."""
        for i, (x, y) in enumerate(zip(a, b)):
            if x != y:
                return i
        return None if len(a) == len(b) else min(len(a), len(b))


def _demo_prompt(vocab: int, n: int = 64) -> List[int]:
    g = torch.Generator().manual_seed(18)
    return torch.randint(min(100, vocab - 1), min(50000, vocab), (n,), generator=g).tolist()


def _co_prompts(n: int, vocab: int) -> List[List[int]]:
    """Junk prompts that share the batch with the demo's prompt: seeded, 5 to 39 tokens long, ids from
    100 up to 49 999 (the numbers of scripts/demo.py:90-94)."""
    g = torch.Generator().manual_seed(1234)
    lo, hi = min(100, vocab - 1), min(50000, vocab)
    lengths = [int(torch.randint(5, 40, (1,), generator=g)) for _ in range(n)]
    return [torch.randint(lo, hi, (L,), generator=g).tolist() for L in lengths]


def _run_demo_config(lm, name: str, steps: int):
    """(token chain, logits chain, [(token, logits)] per generated step) of one way of running the prompt."""
    eng = lm.engine
    prompt = _demo_prompt(lm.spec.vocab_size)
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
    tokens, logits = ChainedDigest(), ChainedDigest()
    for tok, lg in rows:
        tokens.add(int(tok).to_bytes(8, "little"))
        logits.add(lg.numpy().astype("<f4").tobytes())
    return tokens, logits, rows


def cmd_demo(args) -> int:
    import json
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
        results[n] = _run_demo_config(lm, n, args.steps)
        tc, lc, _ = results[n]
        print(f"{n:<6} ({args.steps} tokens, {time.perf_counter() - t0:.1f}s)")
        t_at, l_at = tc.checkpoints(args.checkpoint_every or 0), lc.checkpoints(args.checkpoint_every or 0)
        for k in sorted(l_at):
            print(f"  @{k:<4} tokens {t_at[k]}   logits {l_at[k]}")
    ok = True
    base = names[0]
    for n in names[1:]:
        ta, la, ra = results[base]
        tb, lb, rb = results[n]
        tdiv = ChainedDigest.first_difference(ta.prefixes, tb.prefixes)
        ldiv = ChainedDigest.first_difference(la.prefixes, lb.prefixes)
        worst = max(float((a[1] - b[1]).abs().max()) for a, b in zip(ra, rb))
        print(f"{n} vs {base}: tokens {'identical' if tdiv is None else f'diverge @ {tdiv}'}; logits "
              f"{'bit-identical' if ldiv is None else f'differ from step {ldiv}'} (max |diff| {worst:.3g})")
        if ldiv is not None or tdiv is not None:
            ok = False                      # both precisions promise identical bits across these cuts
    record = {"artifact_sha256": sha, "dtype": args.dtype, "steps": args.steps,
              "chains": {n: {"tokens": results[n][0].prefixes, "logits": results[n][1].prefixes} for n in names}}
    if args.against:
        # the chains of another run -- another process, another day, another machine of the same kind
        with open(args.against) as f:
            other = json.load(f)
        if other.get("artifact_sha256") != sha or other.get("dtype") != args.dtype:
            print(f"{args.against}: made from another artifact or dtype; nothing to compare")
            ok = False
        for n in names:
            theirs = other.get("chains", {}).get(n)
            if theirs is None:
                continue
            ldiv = ChainedDigest.first_difference(record["chains"][n]["logits"][:len(theirs["logits"])],
                                                  theirs["logits"][:len(record["chains"][n]["logits"])])
            print(f"{n} vs {args.against}: logits {'bit-identical' if ldiv is None else f'differ from step {ldiv}'}")
            ok = ok and ldiv is None
    if args.save_chains:
        with open(args.save_chains, "w") as f:
            json.dump(record, f)
    print("\nVERDICT:", "consistent" if ok else "DIVERGENCE — this is a bug")
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
    d.add_argument("--save-chains", metavar="FILE", help="write the chains of this run as JSON")
    d.add_argument("--against", metavar="FILE", help="compare with the chains another run wrote (--save-chains)")
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
    k.add_argument("--kernel", required=True, choices=["attention_single", "attention_single_mma", "attention_prompt", "gemm", "gemm_fused", "step_trace"])
    k.add_argument("--size", default="qwen3-0.6b")
    k.add_argument("--batch", type=int, default=8)
    k.add_argument("--context", type=int, default=3000)
    k.add_argument("--capacity", type=int, default=4096)
    k.add_argument("--tokens", type=int, default=8)
    k.add_argument("--reps", type=int, default=10)
    k.add_argument("--pairs", type=int, choices=[0, 1], default=None,
                   help="products of many tokens: pairs of blocks on a tile where there are tiles enough (1), or never (0)")
    k.add_argument("--band-mb", type=int, default=None,
                   help="products of many tokens: MB of the weight in a band of the tiles' walk (a huge value: no bands)")
    k.add_argument("--lanes-up-to-tiles", type=int, default=None,
                   help="more than 128 tokens stay on the kernel with the tokens on the lanes up to that many persistent tiles")
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
