"""What one step runs: the packed tokens of a batch and where they sit.

Tokens of all sequences are packed one after another (no padding);
``cu_q[i] .. cu_q[i+1]`` are sequence i's tokens.  The reference pads to a
rectangle and masks (src/detllm/model.py:8-17, 259-266); here padding never
enters the computation.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence

import numpy as np
import torch


@dataclass
class StepContext:
    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor       # int32 [N]  token ids
    token_seq: torch.Tensor    # int32 [N]  index of the token's sequence within this step
    positions: torch.Tensor    # int32 [N]  absolute position of the token in its sequence
    cu_q: torch.Tensor         # int32 [n_seqs + 1]
    slots: torch.Tensor        # int32 [n_seqs]  cache slot of each sequence
    q_start: torch.Tensor      # int32 [n_seqs]  sequence length before this step
    kv_len: torch.Tensor       # int32 [n_seqs]  sequence length after this step
    max_q_len: int
    max_kv_len: int            # an upper bound is enough (sizes grids; kernels read kv_len)
    single_token: bool         # every sequence brings exactly one token
    host_q_lens: List[int]
    host_slots: List[int]
    host_starts: List[int]
    memo: Dict = field(default_factory=dict)   # per-step shared tables (position encodings)


class PackedLayout:
    """Where the arrays of a packed step lie inside its one int32 buffer: for ``n`` tokens of ``n_seq``
    sequences, back to back, tokens[n], token_seq[n], positions[n], cu_q[n_seq + 1], slots[n_seq],
    q_start[n_seq], kv_len[n_seq], then whatever the step appends from ``extra_at`` on (its wanted rows).
    The one definition of that order: packing, the views a step's kernels read, the in-place advance of a
    single-token step and the device-side decode loop all take their offsets from here."""

    def __init__(self, n: int, n_seq: int):
        o = 3 * n
        self.n, self.n_seq = n, n_seq
        self.tokens = slice(0, n)
        self.token_seq = slice(n, 2 * n)
        self.positions = slice(2 * n, o)
        self.cu_q = slice(o, o + n_seq + 1)
        self.slots = slice(o + n_seq + 1, o + 2 * n_seq + 1)
        self.q_start = slice(o + 2 * n_seq + 1, o + 3 * n_seq + 1)
        self.kv_len = slice(o + 3 * n_seq + 1, o + 4 * n_seq + 1)
        self.extra_at = o + 4 * n_seq + 1


def pack_step_host(slots: List[int], starts: List[int], token_lists: List[List[int]],
                   extra: Sequence[int] = ()):
    """Host-side packing: returns one int32 tensor laid out as ``PackedLayout`` says, with ``extra`` (the
    step's wanted rows) behind it, plus N and the sequences' token counts."""
    n_seq = len(slots)
    q_lens = [len(t) for t in token_lists]
    n = sum(q_lens)
    lay = PackedLayout(n, n_seq)
    o = 3 * n
    buf = np.empty(lay.extra_at + len(extra), dtype=np.int32)
    st = np.asarray(starts, dtype=np.int32).reshape(n_seq)
    ql = np.asarray(q_lens, dtype=np.int32).reshape(n_seq)
    if n == n_seq and (n_seq == 0 or min(q_lens) == 1):            # one token each
        buf[0:n] = [t[0] for t in token_lists]
        buf[n:2 * n] = np.arange(n_seq, dtype=np.int32)
        buf[2 * n:o] = st
    elif n:
        buf[0:n] = np.concatenate([np.asarray(t, dtype=np.int64).reshape(-1) for t in token_lists])
        seq_of = np.repeat(np.arange(n_seq, dtype=np.int32), ql)
        first = np.concatenate([[0], np.cumsum(ql)[:-1]]).astype(np.int32)
        buf[n:2 * n] = seq_of
        buf[2 * n:o] = np.arange(n, dtype=np.int32) - first[seq_of] + st[seq_of]
    buf[o] = 0
    buf[o + 1:lay.cu_q.stop] = np.cumsum(ql)
    buf[lay.slots] = slots
    buf[lay.q_start] = st
    buf[lay.kv_len] = st + ql
    if len(extra):
        buf[lay.extra_at:] = extra
    return torch.from_numpy(buf), n, q_lens


def advance_packed_single(buf: np.ndarray, n_seq: int, tokens: Sequence[int]) -> None:
    """In place: the packed step of ``n_seq`` sequences with one token each (``pack_step_host``)
    becomes the step that follows it for the same sequences: ``tokens`` are the new tokens, positions,
    first new positions and lengths move on by one; sequence numbers, ``cu_q``, slots and the wanted
    rows stay."""
    lay = PackedLayout(n_seq, n_seq)
    buf[lay.tokens] = tokens
    buf[lay.positions] += 1
    buf[lay.q_start] += 1
    buf[lay.kv_len] += 1


def context_from_packed(dev_buf: torch.Tensor, n: int, slots: List[int], q_lens: List[int],
                        starts: List[int], max_kv_len=None) -> StepContext:
    n_seq = len(slots)
    lay = PackedLayout(n, n_seq)
    return StepContext(
        n_tokens=n, n_seqs=n_seq,
        tokens=dev_buf[lay.tokens], token_seq=dev_buf[lay.token_seq], positions=dev_buf[lay.positions],
        cu_q=dev_buf[lay.cu_q], slots=dev_buf[lay.slots],
        q_start=dev_buf[lay.q_start],
        kv_len=dev_buf[lay.kv_len],
        max_q_len=max(q_lens) if q_lens else 0,
        max_kv_len=max_kv_len if max_kv_len is not None else max(s + q for s, q in zip(starts, q_lens)),
        single_token=all(q == 1 for q in q_lens),
        host_q_lens=list(q_lens), host_slots=list(slots), host_starts=list(starts))
