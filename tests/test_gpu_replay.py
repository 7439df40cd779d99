"""bin/trace_run, as a user runs it: the same requests whole, with the last 32 tokens one by one,
and in batches of unequal lengths whose shorter requests end earlier, one batch after another so
that slots and pages are used again; compared with the plain implementation (GPU)."""

import pytest
import torch

import helpers
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


def _trace(reqs, tails, batch_sizes):
    """Steps for: every request alone and whole; then prefix + last 32 one by one; then batches."""
    steps, expect = [], []          # expect[i] = list of (request, position) rows of step i
    n = 0

    def add(entries, end, rows):
        nonlocal n
        steps.append({"step": n, "entries": entries, "end": end})
        expect.append(rows)
        n += 1
    for r, ids in enumerate(reqs):
        add([{"id": f"w{r}", "tokens": ids, "want": list(range(len(ids)))}], [f"w{r}"],
            [(r, p) for p in range(len(ids))])
    for r, ids in enumerate(reqs):
        if len(ids) <= 32:
            continue
        pre = len(ids) - 32
        add([{"id": f"s{r}", "tokens": ids[:pre], "want": [pre - 1]}], [], [(r, pre - 1)])
        for k in range(32):
            add([{"id": f"s{r}", "tokens": [ids[pre + k]], "want": [0]}], [f"s{r}"] if k == 31 else [],
                [(r, pre + k)])
    it = iter(range(len(reqs)))
    for bs in batch_sizes:
        batch = [next(it) for _ in range(bs)]
        cut = {r: len(reqs[r]) - tails[r] for r in batch}
        add([{"id": f"b{r}", "tokens": reqs[r][:cut[r]], "want": list(range(cut[r]))} for r in batch],
            [f"b{r}" for r in batch if tails[r] == 0], [(r, p) for r in batch for p in range(cut[r])])
        k = 0
        live = [r for r in batch if tails[r] > 0]
        while live:
            add([{"id": f"b{r}", "tokens": [reqs[r][cut[r] + k]], "want": [0] if (r + k) % 3 else []} for r in live],
                [f"b{r}" for r in live if tails[r] == k + 1],
                [(r, cut[r] + k) for r in live if (r + k) % 3])
            k += 1
            live = [r for r in live if tails[r] > k]
    return steps, expect


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16"),
                                        ("C", "bfloat16")])
def test_replay_whole_split_and_batched(model_dirs, tmp_path, name, dtype):
    d = model_dirs(name)
    cfg, w = plain.read_model(d)
    lens = [5, 90, 2, 200, 33, 64, 1, 130]
    tails = [3, 32, 1, 40, 0, 5, 0, 9]
    reqs = [helpers.rand_ids(n, cfg["vocab_size"], 200 + i) for i, n in enumerate(lens)]
    steps, expect = _trace(reqs, tails, [3, 3, 2])
    # the most that is live at once: the largest batch, each request rounded up to 64
    most = max(sum(-(-lens[r] // 64) * 64 for r in b) for b in ([0, 1, 2], [3, 4, 5], [6, 7]))
    got = helpers.run_trace(d, dtype, steps, str(tmp_path / "out"), max_tokens=most)
    refs = [plain.forward(cfg, w, ids) for ids in reqs]
    scale = [float(r.abs().max()) for r in refs]
    # the three ways of cutting the same requests give the same bits at every (request, position), in both precisions
    seen = {}
    for s, rows in zip(steps, expect):
        for i, (r, p) in enumerate(rows):
            first = seen.setdefault((r, p), (s["step"], got[s["step"]][i]))
            assert torch.equal(first[1], got[s["step"]][i]), (
                f"request {r} position {p}: step {s['step']} ({[e['id'] for e in s['entries']]}) and step {first[0]} differ in bits")
    for s, rows in zip(steps, expect):
        if not rows:
            assert s["step"] not in got
            continue
        lg = got[s["step"]]
        assert lg.shape[0] == len(rows)
        for i, (r, p) in enumerate(rows):
            err = float((lg[i].double() - refs[r][p]).abs().max()) / scale[r]
            assert err < helpers.TOL[dtype], (f"step {s['step']} ({[e['id'] for e in s['entries']]}): request {r} "
                                             f"position {p} of {lens[r]}: error {err:.3g}")


def test_replay_refuses_what_does_not_fit(model_dirs, tmp_path):
    import json, os, subprocess, sys
    d = model_dirs("A")
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1] * 65, "want": []}], "end": []}]
    p = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "bin", "trace_run"), "--model", d, "--dtype",
                        "float32", "--out", str(tmp_path), "--max-tokens", "64"],
                       input=json.dumps(steps[0]) + "\n", capture_output=True, text=True, timeout=300)
    assert p.returncode != 0 and "exceeds" in p.stderr and "done 0" not in p.stdout
