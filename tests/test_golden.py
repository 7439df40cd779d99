"""The plain implementation against the reference's own integer runtime on a tiny random model
(outputs committed under tests/golden/, made by tests/golden/make_golden.py).  CPU."""

import json
import os

import numpy as np
import torch

import plain_qwen3 as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_plain_implementation_agrees_with_the_reference_integer_runtime():
    cfg, w = plain.read_model(os.path.join(GOLDEN, "tiny_model"))
    ids = json.load(open(os.path.join(GOLDEN, "tokens.json")))["ids"]
    ref_int8 = torch.from_numpy(np.load(os.path.join(GOLDEN, "reference_int8_logits.npy"))).double()
    mine = plain.forward(cfg, w, ids)
    assert mine.shape == ref_int8.shape == (24, 256)
    cos = torch.nn.functional.cosine_similarity(mine, ref_int8, dim=-1)
    # W8A8 integer arithmetic: about 1e-2 relative; a wrong formula (norm/rotation order, pairing,
    # head map, scale) gives cosines far below this
    assert float(cos.min()) > 0.998 and float(cos.mean()) > 0.999
    assert int((mine.argmax(-1) == ref_int8.argmax(-1)).sum()) >= 23


def test_a_wrong_formula_would_show():
    """The check has teeth: rotating before the norm weights, or the interleaved pairing, fails it."""
    cfg, w = plain.read_model(os.path.join(GOLDEN, "tiny_model"))
    ids = json.load(open(os.path.join(GOLDEN, "tokens.json")))["ids"]
    ref_int8 = torch.from_numpy(np.load(os.path.join(GOLDEN, "reference_int8_logits.npy"))).double()
    orig = plain.rope

    def interleaved(x, positions, theta):                 # pairs (2j, 2j+1): not what the reference does
        hd = x.shape[-1]
        j = torch.arange(0, hd // 2, dtype=torch.float64)
        ang = torch.outer(positions.double(), theta ** (-2.0 * j / hd))
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        a, b = x[..., 0::2], x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2], out[..., 1::2] = a * c - b * s, b * c + a * s
        return out
    plain.rope = interleaved
    try:
        wrong = plain.forward(cfg, w, ids)
    finally:
        plain.rope = orig
    cos = torch.nn.functional.cosine_similarity(wrong, ref_int8, dim=-1)
    assert float(cos.min()) < 0.99
