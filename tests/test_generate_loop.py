"""The generation loop's decisions, with a stand-in for the engine (CPU)."""

import pytest
import torch

from idempotent_llm_b200.engine.generate import generate, plan_batches
from idempotent_llm_b200.sampling import mix64, row_key
import plain_qwen3 as plain


class FakeEngine:
    """Next token = (last token + 1) % vocab; records every call."""

    def __init__(self, vocab=50, max_slots=4):
        self.vocab, self.free, self.held = vocab, list(range(max_slots)), set()
        self.log, self.closed, self.lengths = [], [], {}

    def open(self):
        s = self.free.pop(0)
        self.held.add(s)
        self.lengths[s] = 0
        return s

    def close(self, slot):
        assert slot in self.held, "slot closed twice or never opened"
        self.held.remove(slot)
        self.free.append(slot)
        self.closed.append(slot)

    def step(self, entries, want):
        assert all(s in self.held for s, _ in entries)
        assert all(w == [len(t) - 1] for (_, t), w in zip(entries, want))
        first = all(self.lengths[s] == 0 for s, _ in entries)
        assert first or all(len(t) == 1 for _, t in entries), "mixed prefill and decode in one step"
        self.log.append([(s, list(t)) for s, t in entries])
        for s, t in entries:
            self.lengths[s] += len(t)
        return torch.stack([torch.nn.functional.one_hot(torch.tensor((t[-1] + 1) % self.vocab), self.vocab).float()
                            for _, t in entries])

    def sample(self, logits, temperature, seed, request_ids, steps):
        self.last_sample = (list(request_ids), list(steps))
        return logits.argmax(-1).tolist()


def run(prompts, max_new, **kw):
    e = FakeEngine(max_slots=kw.pop("max_slots", 4))
    kw.setdefault("max_tokens", 64 * 8)
    kw.setdefault("max_seqs", 4)
    res = generate(e, prompts, max_new, **kw)
    assert not e.held, "a slot was not given back"
    return e, res


def test_unequal_prompts_one_prefill_then_one_token_each():
    e, res = run([[1, 2, 3], [10], [20, 21]], 3)
    assert [r.tokens for r in res] == [[4, 5, 6], [11, 12, 13], [22, 23, 24]]
    assert [len(t) for _, t in e.log[0]] == [3, 1, 2]
    assert all(len(t) == 1 for step in e.log[1:] for _, t in step) and len(e.log) == 3
    assert all(r.finish_reason == "length" for r in res)


def test_stop_token_ends_a_sequence_early_and_frees_its_slot_at_once():
    e, res = run([[1], [5], [30]], 6, stop_token_ids=[7])
    assert res[1].tokens == [6, 7] and res[1].finish_reason == "stop"
    assert res[0].tokens == [2, 3, 4, 5, 6, 7] and res[0].finish_reason == "stop"   # stop wins on the last step
    assert res[2].tokens == [31, 32, 33, 34, 35, 36] and res[2].finish_reason == "length"
    assert [len(step) for step in e.log] == [3, 3, 2, 2, 2, 2]                         # the batch shrinks
    assert e.closed[0] == e.log[0][1][0]                                               # request 1's slot first
    assert e.last_sample == ([0, 2], [5, 5])                                           # request ids and step counts


def test_batches_follow_one_another_and_reuse_slots():
    prompts = [[i] for i in range(10)]
    e, res = run(prompts, 2, max_slots=4, max_seqs=4)
    assert [r.tokens for r in res] == [[i + 1, i + 2] for i in range(10)]
    assert [len(s) for s in e.log] == [4, 4, 4, 4, 2, 2]        # prefill + one decode step per batch
    assert set(s for step in e.log for s, _ in step) <= {0, 1, 2, 3} and len(e.closed) == 10


def test_plan_batches_respects_tokens_pages_and_batch_size():
    assert plan_batches([10, 10, 10], 5, 64 * 2, 8, 64) == [[0, 1], [2]]
    assert plan_batches([60, 3], 6, 64 * 3, 8, 64) == [[0, 1]]          # 60 + 5 = 65 tokens: two pages
    assert plan_batches([60, 3], 6, 64 * 2, 8, 64) == [[0], [1]]
    assert plan_batches([1] * 5, 1, 64 * 100, 8, 64, batch_size=2) == [[0, 1], [2, 3], [4]]
    assert plan_batches([1] * 5, 1, 64 * 100, 3, 64) == [[0, 1, 2], [3, 4]]
    with pytest.raises(ValueError, match="needs"):
        plan_batches([200], 1, 64 * 2, 8, 64)
    with pytest.raises(ValueError, match="needs"):
        plan_batches([100], 30, 64 * 4, 8, 64, max_seq_len=128)
    with pytest.raises(ValueError, match="empty prompt"):
        plan_batches([3, 0], 1, 64 * 4, 8, 64)


def test_slots_come_back_when_a_step_fails():
    class Failing(FakeEngine):
        def step(self, entries, want):
            if len(self.log) == 1:
                raise RuntimeError("boom")
            return super().step(entries, want)
    e = Failing()
    with pytest.raises(RuntimeError, match="boom"):
        generate(e, [[1], [2]], 4, max_tokens=64 * 8, max_seqs=4)
    assert not e.held and sorted(e.closed) == [0, 1]


def test_max_new_must_be_positive():
    with pytest.raises(ValueError):
        run([[1]], 0)


def test_generator_of_the_sampler_is_the_documented_one():
    # the plain implementation restates the generator on its own; both must agree bit for bit
    for x in (0, 1, 2**63, 2**64 - 1, 123456789):
        assert mix64(x) == plain._mix(x)
    assert row_key(7, 3, 11) == plain._mix(plain._mix(plain._mix(7) ^ 3) ^ 11)
    assert row_key(7, 3, 11) != row_key(7, 4, 11) != row_key(7, 3, 12)


def test_the_sampler_s_uniform_number_stays_inside_the_open_interval_in_32_bit():
    """u = ((bits >> 41) + 0.5) / 2**23 with every operation rounded to 32-bit: never 0 and never 1, so
    -log(-log(u)) is finite.  (With 24 bits, x = 2**24 - 1 plus 0.5 rounds up to 2**24: u = 1, the score +inf.)"""
    import math
    import numpy as np
    from idempotent_llm_b200.sampling.sampler import uniform_from_bits
    for k in range(1, 65):
        for bits in ((1 << k) - 1, ((1 << k) - 1) << (64 - k), (1 << 64) - 1, 0):
            u = uniform_from_bits(bits & ((1 << 64) - 1))
            assert 0.0 < u < 1.0, (k, bits, u)
            assert math.isfinite(-math.log(-math.log(u)))
    assert uniform_from_bits((1 << 64) - 1) == 1.0 - 2.0 ** -24 and uniform_from_bits(0) == 2.0 ** -24
    # the 24-bit form the kernel once had does reach 1
    assert float((np.float32((1 << 24) - 1) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)) == 1.0


def test_packed_single_token_step_moved_on_in_place_is_the_next_step_packed_anew():
    """The step function keeps the packed arrays of a batch that goes on by one token and updates them
    in place; that must give what packing the next step from scratch gives."""
    import numpy as np
    from idempotent_llm_b200.engine.batch import advance_packed_single, pack_step_host
    slots, starts = [3, 0, 7, 5], [10, 63, 64, 0]
    first, n, _ = pack_step_host(slots, starts, [[11], [12], [13], [14]], extra=range(4))
    buf = first.numpy().copy()
    for step in range(1, 4):
        tokens = [100 * step + i for i in range(4)]
        advance_packed_single(buf, 4, tokens)
        anew, _, _ = pack_step_host(slots, [s + step for s in starts], [[t] for t in tokens], extra=range(4))
        assert np.array_equal(buf, anew.numpy()), f"step {step}"


class FusedFakeEngine(FakeEngine):
    """The same with the step and the pick in one call for sequences that bring one token each."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.fused_calls, self.plain_calls = 0, 0

    def step(self, entries, want):
        self.plain_calls += 1
        return super().step(entries, want)

    def step_sample(self, entries, temperature, seed, request_ids, steps):
        assert all(len(t) == 1 for _, t in entries), "asked for more than one token per sequence"
        self.fused_calls += 1
        self.plain_calls -= 1
        logits = self.step(entries, [[0]] * len(entries))
        return self.sample(logits, temperature, seed, request_ids, steps), logits


def test_an_engine_that_can_step_and_pick_at_once_is_asked_to_for_single_tokens():
    prompts = [[1, 2, 3], [10], [20, 21]]
    e = FusedFakeEngine(max_slots=4)
    res = generate(e, prompts, 4, stop_token_ids=[12], max_tokens=64 * 8, max_seqs=4, return_logits=True)
    _, want = run(prompts, 4, stop_token_ids=[12], return_logits=True)
    assert [r.tokens for r in res] == [r.tokens for r in want] == [[4, 5, 6, 7], [11, 12], [22, 23, 24, 25]]
    assert [r.finish_reason for r in res] == [r.finish_reason for r in want]
    assert e.plain_calls == 1 and e.fused_calls == 3          # the prompts, then one token each three times
    assert all(torch.equal(a, b) for r, w in zip(res, want) for a, b in zip(r.logits, w.logits))
    assert not e.held
    # request ids and step numbers of the last pick: the two sequences still alive, at their fourth token
    assert e.last_sample == ([0, 2], [3, 3])
