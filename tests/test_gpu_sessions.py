"""Schedules around the step function: the device-side decode loop against generation, the same run ten
times over, captured single-token steps of a mixer that keeps state (GPU)."""

import pytest
import torch

import helpers
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("B", "bfloat16"), ("C", "bfloat16")])
def test_decode_session_gives_the_tokens_generation_gives(model_dirs, name, dtype):
    """``Engine.decode_session`` (model, greedy pick and feedback in one captured graph, the host out of the
    loop) against ``generate`` at temperature 0: the same tokens, over a page border (64) and, with model B,
    past a window's edge (80); the cache's lengths and pages are what the steps made them."""
    import idempotent_llm_b200 as idm
    d = model_dirs(name)
    cfg, _ = plain.read_model(d)
    lm = idm.load(d, dtype=dtype, max_tokens=64 * 24, max_seqs=8)
    eng = lm.engine
    prompts = [helpers.rand_ids(n, cfg["vocab_size"], 500 + n) for n in (5, 61, 30, 100)]
    steps = 70
    toks, _ = lm.generate(prompts, steps)                      # [requests, steps]
    assert eng.cache.slots.n_held == 0 and eng.cache.pages_held() == 0
    slots = [eng.open() for _ in prompts]
    first = eng.sample(eng.step(list(zip(slots, prompts))), 0.0, 0, list(range(len(prompts))), [0] * len(prompts))
    assert first == toks[:, 0].tolist()
    sess = eng.decode_session(slots, first, steps - 1)
    sess.run(10)
    sess.run(steps - 1 - 10)
    got = sess.tokens()                                        # [steps - 1, requests]
    sess.finish()
    assert torch.equal(got.T.long(), toks[:, 1:].long()), "the device-side loop chose other tokens than generation"
    for s, p in zip(slots, prompts):
        assert eng.cache.length(s) == len(p) + steps - 1
    # the sequences go on through the ordinary step function from where the session left them
    more = eng.step([(s, [int(t)]) for s, t in zip(slots, got[-1])])
    whole = torch.stack([plain.forward(*plain.read_model(d), list(p) + toks[i].tolist())[-1] for i, p in enumerate(prompts)])
    assert helpers.rel_err(more, whole) < helpers.TOL[dtype]
    with pytest.raises(ValueError):
        sess.run(1)                                            # opened for steps - 1
    for s in slots:
        eng.close(s)
    assert eng.cache.slots.n_held == 0 and eng.cache.pages_held() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_ten_runs_give_the_same_bits(model_dirs, dtype):
    """The same generation ten times in one process (the reference's run-to-run check,
    tests/test_determinism.py:60-68): tokens and every step's logits, bit for bit."""
    import idempotent_llm_b200 as idm
    d = model_dirs("C")
    cfg, _ = plain.read_model(d)
    lm = idm.load(d, dtype=dtype, max_tokens=64 * 16, max_seqs=4)
    prompts = [helpers.rand_ids(n, cfg["vocab_size"], 600 + n) for n in (7, 70, 3)]
    first_toks, first_logits = lm.generate(prompts, 20)
    first_logits = [l.clone() for l in first_logits]
    for run in range(9):
        toks, logits = lm.generate(prompts, 20)
        assert torch.equal(toks, first_toks), f"run {run + 2}: other tokens"
        for s, (a, b) in enumerate(zip(first_logits, logits)):
            assert torch.equal(a, b), f"run {run + 2}: step {s} differs in bits"
