"""Small configurations and utilities of the tests."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_BASE = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", attention_bias=False, hidden_act="silu")

# Tiny configurations that differ in every size and option: head counts and groups, sizes that
# are no power of two, layers, vocabulary, eps, theta, tied or not, window.
TINY = {
    # BASELINE "Tiny Qwen3 A"
    "A": dict(_BASE, num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, max_position_embeddings=2048, eos_token_id=255, initializer_range=0.02),
    # BASELINE "Tiny Qwen3 B", plus a window of 80 keys on layers >= 1
    "B": dict(_BASE, num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=3,
              head_dim=32, intermediate_size=224, vocab_size=320, rope_theta=1000000.0, rms_norm_eps=1e-5,
              tie_word_embeddings=False, max_position_embeddings=4096, eos_token_id=[318, 319],
              initializer_range=0.05, use_sliding_window=True, sliding_window=80, max_window_layers=1),
    # head_dim 128 (the benchmark's head size), group of 4, odd vocabulary and widths
    "C": dict(_BASE, num_hidden_layers=2, hidden_size=160, num_attention_heads=8, num_key_value_heads=2,
              head_dim=128, intermediate_size=288, vocab_size=1000, rope_theta=500000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, max_position_embeddings=8192, eos_token_id=999, initializer_range=0.04),
    # head_dim 48 (a multiple of 16 that is no power of two), no grouping, prime-ish sizes
    "D": dict(_BASE, num_hidden_layers=1, hidden_size=80, num_attention_heads=5, num_key_value_heads=5,
              head_dim=48, intermediate_size=136, vocab_size=131, rope_theta=20000.0, rms_norm_eps=1e-4,
              tie_word_embeddings=False, max_position_embeddings=1024, initializer_range=0.05),
}


def make_model_dir(cfg: dict, out_dir: str, seed: int = 1, dtype=torch.bfloat16, sharp: float = 1.0) -> str:
    """A model folder with seeded random weights.  ``sharp`` > 1 scales every q_norm weight, which
    sharpens attention so that single far keys carry real weight (random weights alone give
    near-uniform attention, which hides a dropped or misplaced key)."""
    from idempotent_llm_b200.config import Qwen3Config
    from idempotent_llm_b200.weights import write_random_model, write_safetensors, SafetensorsFile
    write_random_model(Qwen3Config.from_dict(cfg), out_dir, seed=seed, dtype=dtype)
    if sharp != 1.0:
        path = os.path.join(out_dir, "model.safetensors")
        f = SafetensorsFile(path)
        tensors = []
        for n in f.names():
            t = f.get(n).clone()
            if n.endswith("q_norm.weight"):
                t = (t.float() * sharp).to(t.dtype)
            tensors.append((n, t))
        del f
        write_safetensors(path, tensors)
    return out_dir


def rand_ids(n: int, vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


# Tolerances against the 64-bit plain implementation, fixed before any measurement:
# 32-bit arithmetic with sums of a few hundred terms; bfloat16 rounds activations (8 bits of
# mantissa) a handful of times per layer.
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def run_trace(model_dir: str, dtype: str, steps: list, out_dir: str, max_tokens: int, timeout: int = 600,
              extra=()):
    """Run bin/trace_run on a list of step records; returns {step: tensor [wanted, vocab]}."""
    import numpy as np
    with open(os.path.join(model_dir, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    inp = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype",
                        dtype, "--out", out_dir, "--max-tokens", str(max_tokens), *extra],
                       input=inp, capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0, f"trace_run failed ({p.returncode}):\n{p.stdout[-2000:]}\n{p.stderr[-4000:]}"
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert [l.split()[1] for l in done] == [str(s["step"]) for s in steps], p.stdout[-2000:]
    out = {}
    for s in steps:
        n = sum(len(e.get("want", [])) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if n:
            out[s["step"]] = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(n, vocab).copy())
        else:
            assert not os.path.exists(path)
    return out
