"""The step function and what it stands on: model, cache, decode graphs.

One ``step`` runs only the tokens it is given, as one packed batch, against
what earlier steps left in the cache, and returns 32-bit logits at the wanted
places.  A batch's sequences start together with unequal lengths (all prompts
in one step), then bring one token each; any other mix of lengths runs too.
The reference's ``forward`` (src/detllm/model.py:220-286) takes a padded
rectangle plus positions and returns logits at every position; its
``GraphedDecode.step`` (src/detllm/graphed.py:111-132) replays one captured
graph per decode step, which ``Engine`` does per batch size.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..cache import CacheError, SequenceCache
from .assembly import CausalLM, cache_needs
from .batch import PackedLayout, StepContext, advance_packed_single, context_from_packed, pack_step_host


class _DecodeGraph:
    """A captured single-token step for a fixed number of sequences; with ``temperature`` given, the
    pick of one token per row from the logits is part of the graph (``keys``: rows draw with keys of
    their own, which come with the step's other inputs)."""

    def __init__(self, engine: "Engine", n_seqs: int, temperature: Optional[float] = None, keys: bool = False):
        self.n = n_seqs
        dev = engine.device
        self.layout = PackedLayout(n_seqs, n_seqs)       # one token per sequence; the wanted rows (one each) behind
        self.packed_size = self.layout.extra_at + n_seqs
        # the rows' 64-bit keys lie behind the packed step on an 8-byte border
        self.keys_at = (self.packed_size + 1) // 2 * 2
        self.size = self.keys_at + (2 * n_seqs if keys else 0)
        self.host = torch.zeros(self.size, dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(self.size, dtype=torch.int32, device=dev)
        self.temperature, self.keys = temperature, keys
        self.graph = None
        self.logits = None
        self.picked = None              # int32 [n_seqs] on the device, if the pick is part of the graph
        self.uploaded = None            # event: the last host->device copy of `host` is done
        self.host_np = self.host.numpy()                 # the same pinned memory
        self.last_slots, self.next_starts = None, None   # the batch of the last run and where it goes on

    def run(self, engine: "Engine", packed: Optional[torch.Tensor], slots, q_lens, starts, keys=None,
            tokens=None) -> torch.Tensor:
        """``packed``: the whole packed step, or None when the step is the last run's batch one token
        further: then only ``tokens`` are new and positions and lengths move on by one in place."""
        if self.uploaded is not None:
            self.uploaded.synchronize()
        if packed is not None:
            self.host[:self.packed_size].copy_(packed)
        else:
            advance_packed_single(self.host_np, self.n, tokens)
        self.last_slots, self.next_starts = slots, [st + 1 for st in starts]
        if self.keys:
            self.host[self.keys_at:].view(torch.int64).copy_(keys)
        self.dev.copy_(self.host, non_blocking=True)
        if self.uploaded is None:
            self.uploaded = torch.cuda.Event()
        self.uploaded.record()
        if self.graph is None:
            ctx = context_from_packed(self.dev, self.n, slots, q_lens, starts,
                                      max_kv_len=engine.cache.max_seq_len)
            rows = self.dev[self.layout.extra_at:self.packed_size]
            dev_keys = self.dev[self.keys_at:].view(torch.int64) if self.keys else None
            K = engine.rt.kernels

            def body():
                ctx.memo.clear()
                self.logits = engine.model.forward(ctx, engine.cache, rows)
                if self.temperature is not None:
                    self.picked = K.sample(self.logits, self.temperature, dev_keys)
            # warm-up outside capture (lazy library state).  Keys and values are written once per position,
            # so running the step again changes nothing there; per-sequence state is read, then written:
            # it is put back, or the replay below would be the step's third run on it
            keep = engine.cache.snapshot_state(slots)
            for _ in range(2):
                body()
            torch.cuda.synchronize()
            engine.cache.restore_state(slots, keep)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=engine._graph_pool):
                body()
            if engine._graph_pool is None:
                engine._graph_pool = g.pool()
            self.graph = g
        self.graph.replay()
        return self.logits


class DecodeSession:
    """Greedy decoding of a fixed batch without the host in the loop: one captured graph holds the
    model's single-token step, the argmax and the feedback of the chosen tokens, so ``run(n)`` is
    ``n`` graph replays back to back (the reference's steady-state decode, scripts/bench.py:28-43:
    ``greedy_pick(gd.step(cur))`` per step, synchronised only at the end).  Pages for all ``n``
    steps are reserved beforehand; reads stay bounded by each sequence's length on the device."""

    def __init__(self, engine: "Engine", slots: Sequence[int], first_tokens: Sequence[int], max_steps: int):
        self.engine, self.slots, self.max_steps = engine, [int(s) for s in slots], max_steps
        cache, dev = engine.cache, engine.device
        B = self.n = len(self.slots)
        self.starts = [cache.length(s) for s in self.slots]
        cache.reserve([(s, st + max_steps) for s, st in zip(self.slots, self.starts)])
        cache.flush()
        full, n, q_lens = pack_step_host(self.slots, self.starts, [[int(t)] for t in first_tokens], extra=range(B))
        self.dev = full.to(dev)
        self.history = torch.zeros((max_steps, B), dtype=torch.int32, device=dev)
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.ctx = context_from_packed(self.dev, B, self.slots, q_lens, self.starts,
                                       max_kv_len=cache.max_seq_len)
        self.layout = PackedLayout(B, B)
        self.rows = self.dev[self.layout.extra_at:]
        self.steps_done = 0
        self.launches_per_step = 0
        backup, keep = self.dev.clone(), cache.snapshot_state(self.slots)
        K = engine.rt.kernels
        for _ in range(2):
            self._one_step()
        torch.cuda.synchronize()
        self.dev.copy_(backup)                    # warm-up moved the positions (and any per-sequence state) on; start again
        cache.restore_state(self.slots, keep)
        self.counter.zero_()
        g = torch.cuda.CUDAGraph()
        before = K.launches
        with torch.cuda.graph(g):                 # a pool of its own: it dies with the session
            self._one_step()
        self.launches_per_step = K.launches - before
        self.graph = g

    def _one_step(self):
        e, K, B = self.engine, self.engine.rt.kernels, self.n
        self.ctx.memo.clear()
        logits = e.model.forward(self.ctx, e.cache, self.rows)
        picked = K.sample(logits, 0.0, None)
        d, lay = self.dev, self.layout
        K.decode_advance(d[lay.tokens], d[lay.positions], d[lay.q_start], d[lay.kv_len], picked,
                         self.history, self.counter)

    def run(self, n_steps: int) -> None:
        if self.steps_done + n_steps > self.max_steps:
            raise ValueError(f"the session was opened for {self.max_steps} steps")
        for _ in range(n_steps):
            self.graph.replay()
        self.steps_done += n_steps

    def tokens(self) -> torch.Tensor:
        """Chosen tokens so far, ``[steps, sequences]`` (device -> host copy; synchronises)."""
        return self.history[:self.steps_done].cpu()

    def finish(self) -> None:
        """Hand the sequences back to the engine's own bookkeeping at their new lengths."""
        torch.cuda.synchronize()
        for s, st in zip(self.slots, self.starts):
            self.engine.cache.set_length(s, st + self.steps_done)


class Engine:
    def __init__(self, model: CausalLM, max_tokens: int, max_seqs: Optional[int] = None,
                 max_seq_len: Optional[int] = None, use_graph: bool = True):
        self.model = model
        self.rt = model.rt
        self.device = model.rt.device
        self.spec = model.spec
        if max_seq_len is None:
            max_seq_len = min(max_tokens, model.spec.max_positions)
        self.cache = SequenceCache(cache_needs(model.spec), max_tokens, model.rt.dtype, self.device,
                                   max_seqs=max_seqs, max_seq_len=max_seq_len)
        self.use_graph = use_graph and self.device.type == "cuda"
        self._graphs: Dict[object, _DecodeGraph] = {}    # by batch size, or (batch size, temperature, keys)
        self._graph_pool = None
        self._pinned: Dict[int, list] = {}
        self.steps_run = 0

    # slots ------------------------------------------------------------------
    def open(self) -> int:
        """Take a slot for a new sequence."""
        return self.cache.alloc_slot()

    def close(self, slot: int) -> None:
        """Give a finished sequence's slot and pages back."""
        self.cache.free_slot(slot)

    # the step function --------------------------------------------------------
    def step(self, entries: Sequence[Tuple[int, Sequence[int]]],
             want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """Run one step.  ``entries``: (slot, this step's tokens) per sequence.
        ``want[i]``: places among sequence i's tokens whose logits are returned
        (default: the last one).  Returns ``[n_wanted, vocab]`` float32 on the
        device, ordered by entry, then by ``want``."""
        if not entries:
            raise ValueError("a step needs at least one sequence")
        slots = [int(s) for s, _ in entries]
        toks = [list(t) for _, t in entries]
        if len(set(slots)) != len(slots):
            raise ValueError("a slot appears twice in one step")
        V = self.spec.vocab_size
        for s, t in zip(slots, toks):
            if not t:
                raise ValueError(f"slot {s} brings no token")
            if min(t) < 0 or max(t) >= V:
                bad = [x for x in t if not 0 <= x < V]
                raise ValueError(f"token id {bad[0]} is outside the vocabulary [0, {V})")
        if want is None:
            want = [[len(t) - 1] for t in toks]
        if len(want) != len(toks):
            raise ValueError("want must have one list per entry")
        rows, off = [], 0
        for t, w in zip(toks, want):
            for j in w:
                if not 0 <= j < len(t):
                    raise ValueError(f"wanted place {j} is outside the entry's {len(t)} tokens")
                rows.append(off + j)
            off += len(t)
        starts = [self.cache.length(s) for s in slots]
        self.cache.reserve([(s, st + len(t)) for s, st, t in zip(slots, starts, toks)])
        single = all(len(t) == 1 for t in toks)
        graphed = single and self.use_graph and getattr(self.model, "graph_safe", True)
        full, n, q_lens = pack_step_host(slots, starts, toks, extra=range(len(slots)) if graphed else rows)
        self.cache.flush()
        if graphed:
            g = self._graphs.get(len(slots))
            if g is None:
                g = self._graphs[len(slots)] = _DecodeGraph(self, len(slots))
            logits = g.run(self, full, slots, q_lens, starts)
            # the graph writes its logits into the same buffer at every replay: hand out a copy
            if rows == list(range(len(slots))):
                logits = logits.clone()
            else:
                logits = logits[torch.tensor(rows, dtype=torch.long, device=self.device)] if rows \
                    else logits[:0].clone()
        else:
            dev = self._upload(full)
            ctx = context_from_packed(dev, n, slots, q_lens, starts)
            logits = self.model.forward(ctx, self.cache, dev[full.numel() - len(rows):])
        for s, st, t in zip(slots, starts, toks):
            self.cache.set_length(s, st + len(t))
        self.steps_run += 1
        return logits

    def step_sample(self, entries: Sequence[Tuple[int, Sequence[int]]], temperature: float, seed: int,
                    request_ids: Sequence[int], steps: Sequence[int]) -> Tuple[List[int], torch.Tensor]:
        """``sample(step(entries), ...)`` for sequences that bring one token each, as one captured
        graph (model and pick) where graphs are in use: the same kernels on the same inputs, so the
        same tokens, without a launch and a copy of the logits in between.  Returns the chosen tokens
        and the logits ``[n, vocab]``, which stay valid until the engine's next step."""
        single = all(len(t) == 1 for _, t in entries)
        if not (single and self.use_graph and getattr(self.model, "graph_safe", True)):
            logits = self.step(entries)
            return self.sample(logits, temperature, seed, request_ids, steps), logits
        from ..sampling.sampler import row_keys
        if temperature < 0:
            raise ValueError("temperature must be >= 0")
        slots = [int(s) for s, _ in entries]
        toks = [[int(t[0])] for _, t in entries]
        n = len(slots)
        if len(set(slots)) != n:
            raise ValueError("a slot appears twice in one step")
        if len(request_ids) != n or len(steps) != n:
            raise ValueError("one request id and one step per row")
        V = self.spec.vocab_size
        for s, t in zip(slots, toks):
            if not 0 <= t[0] < V:
                raise ValueError(f"token id {t[0]} is outside the vocabulary [0, {V})")
        starts = [self.cache.length(s) for s in slots]
        self.cache.reserve([(s, st + 1) for s, st in zip(slots, starts)])
        self.cache.flush()
        keys = row_keys(seed, request_ids, steps) if temperature > 0 else None
        key = (n, float(temperature), keys is not None)
        g = self._graphs.get(key)
        if g is None:
            if len(self._graphs) >= 64:                  # (many temperatures: start over rather than grow)
                self._graphs.clear()
            g = self._graphs[key] = _DecodeGraph(self, n, float(temperature), keys is not None)
        if g.graph is not None and g.last_slots == slots and g.next_starts == starts:
            g.run(self, None, slots, None, starts, keys, tokens=[t[0] for t in toks])   # the same batch, one token on
        else:
            full, _, q_lens = pack_step_host(slots, starts, toks, extra=range(n))
            g.run(self, full, slots, q_lens, starts, keys)
        picked = g.picked.tolist()
        for s, st in zip(slots, starts):
            self.cache.set_length(s, st + 1)
        self.steps_run += 1
        return picked, g.logits

    def _upload(self, host: torch.Tensor) -> torch.Tensor:
        """A step's packed integers to the device through pinned memory.  The copy reads the pinned buffer when
        the GPU gets to it, so a buffer is written again only after the event behind its last copy; two buffers
        per size take turns, so that the host can pack the next step while the GPU is still on this one."""
        if self.device.type != "cuda":
            return host.to(self.device)
        n = host.numel()
        cap = 1 << max(6, (n - 1).bit_length())
        ring = self._pinned.get(cap)
        if ring is None:
            ring = self._pinned[cap] = [0, [], []]               # whose turn, buffers, the events behind their last copies
        turn, bufs, events = ring
        if len(bufs) < 2:
            bufs.append(torch.empty(cap, dtype=torch.int32, pin_memory=True))
            events.append(torch.cuda.Event())
            turn = len(bufs) - 1
        else:
            events[turn].synchronize()                           # the last upload from this buffer is done
        pin = bufs[turn]
        pin[:n].copy_(host)
        dev = pin[:n].to(self.device, non_blocking=True)
        events[turn].record()
        ring[0] = (turn + 1) % 2
        return dev

    def decode_session(self, slots: Sequence[int], first_tokens: Sequence[int], max_steps: int) -> DecodeSession:
        """A device-side greedy decode loop over ``slots`` (see ``DecodeSession``)."""
        return DecodeSession(self, slots, first_tokens, max_steps)

    # sampling -----------------------------------------------------------------
    def sample(self, logits: torch.Tensor, temperature: float, seed: int,
               request_ids: Sequence[int], steps: Sequence[int]) -> List[int]:
        """Pick one token per row of ``logits``; see ``sampling.sampler``."""
        from ..sampling.sampler import sample_tokens
        return sample_tokens(self.rt.kernels, logits, temperature, seed, request_ids, steps)
