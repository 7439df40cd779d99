"""The command line as a user runs it, on a tiny model (GPU): ``random`` writes a folder, ``generate``
gives the plain implementation's greedy tokens in 32-bit, ``demo`` finds its three ways of running one
prompt bit-identical in both precisions and can compare with the chains of another run."""

import json
import os
import subprocess
import sys

import pytest

import helpers
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


def _cli(*args, ok=True):
    p = subprocess.run([sys.executable, "-m", "idempotent_llm_b200", *args], cwd=helpers.ROOT, capture_output=True,
                       text=True, timeout=600)
    if ok:
        assert p.returncode == 0, f"{args}: exit {p.returncode}\n{p.stdout[-2000:]}\n{p.stderr[-3000:]}"
    return p


def test_random_generate_and_demo(tmp_path):
    d = str(tmp_path / "tiny-b")
    _cli("random", "--size", "tiny-b", "--out", d, "--seed", "11")
    assert os.path.isfile(os.path.join(d, "config.json")) and os.path.isfile(os.path.join(d, "model.safetensors"))
    cfg, w = plain.read_model(d)
    prompts = [helpers.rand_ids(9, cfg["vocab_size"], 700), helpers.rand_ids(3, cfg["vocab_size"], 701)]
    p = _cli("generate", "--artifact", d, "--dtype", "float32", "--max-new", "6",
             *[a for ids in prompts for a in ("--prompt-ids", " ".join(map(str, ids)))])
    lines = [l for l in p.stdout.splitlines() if l.startswith("request ")]
    assert len(lines) == 2
    for i, ids in enumerate(prompts):
        want = plain.generate(cfg, w, ids, 6)[0]
        got = [int(t) for t in lines[i].split(":")[1].split()]
        assert got == want, f"request {i}: {got} instead of {want}"
    chains = str(tmp_path / "chains.json")
    for dtype in ("float32", "bfloat16"):
        p = _cli("demo", "--artifact", d, "--steps", "16", "--dtype", dtype, "--checkpoint-every", "8",
                 "--save-chains", chains + dtype)
        assert "b8 vs b1: tokens identical; logits bit-identical" in p.stdout, p.stdout
        assert "split vs b1: tokens identical; logits bit-identical" in p.stdout, p.stdout
        assert "VERDICT: consistent" in p.stdout
        # another process, the same chains
        p = _cli("demo", "--artifact", d, "--steps", "16", "--dtype", dtype, "--config", "b8", "--against", chains + dtype)
        assert f"b8 vs {chains + dtype}: logits bit-identical" in p.stdout
    # chains of the other precision are not this run's: exit 1
    p = _cli("demo", "--artifact", d, "--steps", "16", "--dtype", "float32", "--config", "b1", "--against", chains + "bfloat16", ok=False)
    assert p.returncode == 1 and "nothing to compare" in p.stdout
    with open(chains + "float32") as f:
        rec = json.load(f)
    assert set(rec["chains"]) == {"b1", "b8", "split"} and len(rec["chains"]["b1"]["logits"]) == 16
