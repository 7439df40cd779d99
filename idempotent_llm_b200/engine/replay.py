"""Trace replay: given token ids go through the model step by step, logits come out.

Nothing is sampled.  The program drives the same model, step function, cache and
kernels that generation uses.  The reference's nearest relative is the ``split``
configuration of scripts/demo.py:125-155 (a prompt fed as a prefill plus single-token
steps) with its chain hash over each step's logits (scripts/demo.py:58-71); the hash
is kept here as an optional line per step.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: each request's next tokens and the places among them whose logits are
wanted.  ``end``: requests that are finished after this step; their slot and pages are
given back.  For a step that wants something, ``OUT/<step>.f32`` receives the logits
``[wanted, vocab]`` as little-endian float32, in the order of the entries and of
``want``.  After every step ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
from typing import Dict

import numpy as np


class Replayer:
    def __init__(self, lm, out_dir: str, chain_hash: bool = False):
        self.lm = lm
        self.engine = lm.engine
        self.out_dir = out_dir
        self.slots: Dict[str, int] = {}
        self.chain = hashlib.sha256(b"idempotent-llm-b200-replay-v1").digest() if chain_hash else None
        os.makedirs(out_dir, exist_ok=True)

    def run_step(self, rec: dict) -> str:
        step = rec["step"]
        entries = rec.get("entries", [])
        opened = []
        try:
            batch, want = [], []
            for e in entries:
                rid = str(e["id"])
                if rid not in self.slots:
                    self.slots[rid] = self.engine.open()
                    opened.append(rid)
                batch.append((self.slots[rid], [int(t) for t in e["tokens"]]))
                want.append([int(j) for j in e.get("want", [])])
            if batch:
                logits = self.engine.step(batch, want)
                if logits.shape[0]:
                    arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                    arr.tofile(os.path.join(self.out_dir, f"{step}.f32"))
                    if self.chain is not None:
                        self.chain = hashlib.sha256(self.chain + arr.tobytes()).digest()
        except Exception:
            for rid in opened:                       # a refused step leaves no half-open request
                self.engine.close(self.slots.pop(rid))
            raise
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid not in self.slots:
                raise KeyError(f"step {step}: request {rid!r} ends but is not live")
            self.engine.close(self.slots.pop(rid))
        line = f"done {step}"
        if self.chain is not None:
            line += f" {self.chain.hex()[:16]}"
        return line


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--hash", action="store_true", help="append a chain hash of the logits to each 'done' line")
    ap.add_argument("--no-graph", action="store_true", help="do not capture single-token steps in CUDA graphs")
    args = ap.parse_args(argv)

    from .. import api
    lm = api.load(args.model, dtype=args.dtype, max_tokens=args.max_tokens, use_graph=not args.no_graph)
    rp = Replayer(lm, args.out, chain_hash=args.hash)
    for raw in sys.stdin:
        raw = raw.strip()
        if not raw:
            continue
        try:
            rec = json.loads(raw)
        except json.JSONDecodeError as e:
            print(f"trace_run: input line is not JSON: {e}", file=sys.stderr)
            return 2
        print(rp.run_step(rec), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
