"""Whole models at the layer sizes of the benchmarks (fewer layers, the same widths): the 0.6B sizes with
their whole vocabulary, and the 8B sizes (inner axes of 4096 and 12288) with a smaller vocabulary, which
only shortens the head.  bfloat16 against 32-bit against the plain implementation, and both engines
against themselves bit for bit across whole prompts, single tokens and unequal batches (GPU)."""

import pytest
import torch

import helpers
import plain_qwen3 as plain
from test_gpu_model import _run_batches

pytestmark = pytest.mark.gpu

SIZES = {
    "0.6b-widths": dict(helpers._BASE, num_hidden_layers=2, hidden_size=1024, num_attention_heads=16,
                        num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=151936,
                        rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                        max_position_embeddings=40960, initializer_range=0.02),
    "8b-widths": dict(helpers._BASE, num_hidden_layers=1, hidden_size=4096, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=8192,
                      rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                      max_position_embeddings=40960, initializer_range=0.02),
}


@pytest.mark.parametrize("name", list(SIZES))
def test_real_layer_sizes_in_both_precisions(tmp_path_factory, name):
    import idempotent_llm_b200 as idm
    d = helpers.make_model_dir(SIZES[name], str(tmp_path_factory.mktemp(name)), seed=7)
    cfg, w = plain.read_model(d)
    V = cfg["vocab_size"]
    n, tail = 332, 32
    ids = helpers.rand_ids(n, V, 311)
    rows = [0, 1, 63, 64, 127, 128, 255, 256, n - tail - 1] + list(range(n - tail, n))
    ref = plain.forward(cfg, w, ids, rows=rows)
    lens, tails = [300, 70, 9, 131], [32, 5, 0, 3]
    reqs = [ids[:300]] + [helpers.rand_ids(m, V, 320 + i) for i, m in enumerate(lens[1:])]
    out = {}
    for dtype in ("float32", "bfloat16"):
        lm = idm.load(d, dtype=dtype, max_tokens=64 * 16, max_seqs=4)
        eng = lm.engine
        slot = eng.open()
        got = [eng.step([(slot, ids[:n - tail])], [rows[:9]])]
        for t in ids[n - tail:]:
            got.append(eng.step([(slot, [t])]).clone())
        eng.close(slot)
        got = torch.cat(got)
        err = (got.double().cpu() - ref).abs().amax(dim=1) / ref.abs().max()
        bad = (err >= helpers.TOL[dtype]).nonzero()
        assert bad.numel() == 0, f"{dtype}: first wrong row {int(bad[0])} (position {rows[int(bad[0])]}), error {float(err.max()):.3g}"
        out[dtype] = got
        # the same requests whole and in an unequal batch whose members leave early: the same bits
        whole = []
        for r in reqs:
            s_ = eng.open()
            whole.append(eng.step([(s_, r)], [list(range(len(r)))]).clone())
            eng.close(s_)
        for a, b in zip(whole, _run_batches(eng, reqs, [4], tails)):
            assert torch.equal(a, b), f"{dtype}: a request's logits depend on how its tokens were cut"
        assert torch.equal(whole[0][rows[:8]], got[:8]), f"{dtype}: a prompt's rows depend on its length"
        assert eng.cache.slots.n_held == 0 and eng.cache.pages_held() == 0
        del lm, eng
        torch.cuda.empty_cache()
    rel = float((out["bfloat16"] - out["float32"]).abs().max() / out["float32"].abs().max())
    assert rel < helpers.TOL["bfloat16"], f"bfloat16 against 32-bit: {rel:.3g}"
