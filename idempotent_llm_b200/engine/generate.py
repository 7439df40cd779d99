"""The generation loop above the step function.

The reference's loop (src/detllm/model.py:492-531) prefills a padded batch
once, takes each row's logits at its own last prompt token, then feeds one
token per sequence per step for a fixed number of steps; it accepts
``stop_at_eos`` and ignores it (model.py:495), and every sequence runs to the
end.  Here stop tokens end a sequence (the stop token is kept as its last
token), a finished sequence leaves the batch and gives its slot back at once,
and requests are cut into as many batches, one after another, as the cache
admits.

The loop only needs ``open() -> slot``, ``close(slot)``,
``step(entries, want) -> logits`` and ``sample(logits, temperature, seed,
request_ids, steps) -> list[int]`` from the engine, so its decisions are
testable with a stand-in.  An engine that also has ``step_sample(entries,
temperature, seed, request_ids, steps) -> (tokens, logits)`` is asked for the
two at once when every sequence brings one token; the logits it returns (and
``on_step`` sees) are valid until the engine's next step, so what is kept
(``return_logits``) is copied.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence


@dataclass
class GenerationResult:
    request: int
    prompt_len: int
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""            # "stop" or "length"
    logits: List = field(default_factory=list)   # per generated token, if asked for


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


def plan_batches(prompt_lens: Sequence[int], max_new: int, max_tokens: int, max_seqs: int,
                 page_tokens: int, max_seq_len: Optional[int] = None,
                 batch_size: Optional[int] = None) -> List[List[int]]:
    """Cut requests, in order, into batches that fit the cache at their longest.

    A request may hold ``prompt + max_new - 1`` tokens (the last sampled token
    is never fed back), rounded up to whole pages.  Raises if one request alone
    cannot fit."""
    limit = max_seqs if batch_size is None else min(batch_size, max_seqs)
    if limit <= 0:
        raise ValueError("batch size must be positive")
    batches, cur, used = [], [], 0
    for i, L in enumerate(prompt_lens):
        if L <= 0:
            raise ValueError(f"request {i} has an empty prompt")
        longest = L + max(max_new - 1, 0)
        need = _round_up(longest, page_tokens)
        if need > max_tokens or (max_seq_len is not None and longest > max_seq_len):
            raise ValueError(f"request {i} needs {longest} tokens of cache; the cache holds "
                             f"{max_tokens} in all and {max_seq_len} per sequence")
        if cur and (used + need > max_tokens or len(cur) >= limit):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def generate(engine, prompts: Sequence[Sequence[int]], max_new: int, *, temperature: float = 0.0,
             seed: int = 0, stop_token_ids: Sequence[int] = (), batch_size: Optional[int] = None,
             return_logits: bool = False, max_tokens: Optional[int] = None,
             max_seqs: Optional[int] = None, max_seq_len: Optional[int] = None,
             page_tokens: int = 64, on_step: Optional[Callable] = None) -> List[GenerationResult]:
    """Generate up to ``max_new`` tokens for every prompt.  Results are in request order."""
    if max_new <= 0:
        raise ValueError("max_new must be positive")
    cache = getattr(engine, "cache", None)
    max_tokens = max_tokens if max_tokens is not None else cache.max_tokens
    max_seqs = max_seqs if max_seqs is not None else cache.max_seqs
    max_seq_len = max_seq_len if max_seq_len is not None else getattr(cache, "max_seq_len", None)
    stops = set(int(t) for t in stop_token_ids)
    results = [GenerationResult(request=i, prompt_len=len(p)) for i, p in enumerate(prompts)]
    for batch in plan_batches([len(p) for p in prompts], max_new, max_tokens, max_seqs,
                              page_tokens, max_seq_len, batch_size):
        live = [(r, engine.open()) for r in batch]           # (request, slot)
        try:
            feed = [list(prompts[r]) for r, _ in live]       # this step's tokens per live sequence
            while live:
                entries = [(s, t) for (_, s), t in zip(live, feed)]
                rows, steps = [r for r, _ in live], [len(results[r].tokens) for r, _ in live]
                fused = getattr(engine, "step_sample", None)
                if fused is not None and all(len(t) == 1 for t in feed):
                    picked, logits = fused(entries, temperature, seed, rows, steps)   # one token each
                else:
                    logits = engine.step(entries, [[len(t) - 1] for t in feed])
                    picked = engine.sample(logits, temperature, seed, rows, steps)
                if on_step is not None:
                    on_step([r for r, _ in live], picked, logits)
                nxt_live, nxt_feed = [], []
                for row, ((r, slot), tok) in enumerate(zip(live, picked)):
                    res = results[r]
                    res.tokens.append(int(tok))
                    if return_logits:
                        res.logits.append(logits[row].clone() if hasattr(logits[row], "clone")
                                          else logits[row])
                    if int(tok) in stops:
                        res.finish_reason = "stop"
                    elif len(res.tokens) >= max_new:
                        res.finish_reason = "length"
                    if res.finish_reason:
                        engine.close(slot)
                    else:
                        nxt_live.append((r, slot))
                        nxt_feed.append([int(tok)])
                live, feed = nxt_live, nxt_feed
        finally:
            for _, slot in live:                             # only after an error mid-batch
                engine.close(slot)
    return results
