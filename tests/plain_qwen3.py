"""A plain, slow implementation of the Qwen3 dense decoder: whole sequences, no cache,
one function per part, 64-bit floats on the CPU.  It shares no code with the package:
it parses config.json and reads the safetensors file on its own.

It rests on the reference's formulas (the reference has no float model of its own: its
float rows call the transformers library as a black box, src/detllm/prepare.py:236-240,
scripts/demo.py:172-176).  Each function cites where the reference spells its part out.
``tests/golden/`` holds a cross-check of this file against the reference's own integer
runtime on a tiny random model.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- reading
def read_model(model_dir: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors = {k: v.to(F64) for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, tensors


def rope_theta(cfg: dict) -> float:
    # src/detllm/prepare.py:32-35
    if cfg.get("rope_theta") is not None:
        return float(cfg["rope_theta"])
    if isinstance(cfg.get("rope_parameters"), dict):
        return float(cfg["rope_parameters"]["rope_theta"])
    return 10000.0


def layer_window(cfg: dict, i: int) -> Optional[int]:
    # not read by the reference; a layer i >= max_window_layers sees the last sliding_window keys
    if cfg.get("use_sliding_window") and i >= cfg.get("max_window_layers", cfg["num_hidden_layers"]):
        return int(cfg["sliding_window"])
    return None


# ------------------------------------------------------------------------------- parts
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight over the last axis.
    Float form without eps: tests/test_ops.py:198-199, scripts/attribute_error.py:48-51;
    weight after normalisation: deep-dive/README.md:443-462."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x [T, heads, hd]; pairs (d, d + hd/2), angles tiled twice.
    src/detllm/ops/rope.py:25-35, 47-55; float form tests/test_ops.py:281-288,
    src/detllm/prepare.py:137-141, 181-188 (cos/sin rounded to 32-bit there)."""
    hd = x.shape[-1]
    j = torch.arange(0, hd // 2, dtype=F64)
    inv_freq = theta ** (-2.0 * j / hd)
    ang = torch.outer(positions.to(F64), inv_freq)
    ang = torch.cat([ang, ang], dim=-1)
    cos, sin = torch.cos(ang).float().to(x.dtype), torch.sin(ang).float().to(x.dtype)
    rot = torch.cat([-x[..., hd // 2:], x[..., : hd // 2]], dim=-1)
    return x * cos[:, None, :] + rot * sin[:, None, :]


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: Optional[int] = None, q_positions=None) -> torch.Tensor:
    """q [Tq, n_q, hd], k/v [Tk, n_kv, hd]; q-head h uses kv-head h // group
    (src/detllm/model.py:170, ops/fused_attn.py:60); query at position p sees keys j <= p
    (src/detllm/model.py:259-266), and j > p - window under a window; softmax over the
    allowed keys, others exactly 0 (src/detllm/ops/di_softmax.py:41-61; float form
    scripts/attribute_error.py:29-34); scale 1/sqrt(hd) (src/detllm/prepare.py:338)."""
    Tq, n_q, hd = q.shape
    Tk, n_kv, _ = k.shape
    g = n_q // n_kv
    qp = torch.arange(Tk - Tq, Tk) if q_positions is None else q_positions
    kp = torch.arange(Tk)
    allowed = kp[None, :] <= qp[:, None]
    if window:
        allowed &= kp[None, :] > qp[:, None] - window
    out = torch.zeros(Tq, n_q, hd, dtype=q.dtype)
    for h in range(n_q):
        s = (q[:, h, :] @ k[:, h // g, :].T) * scale
        s = torch.where(allowed, s, torch.full_like(s, -float("inf")))
        p = torch.softmax(s, dim=-1)
        p = torch.where(allowed, p, torch.zeros_like(p))
        out[:, h, :] = p @ v[:, h // g, :]
    return out


def attention_block(x, w, prefix, cfg, positions, window, kv=None):
    """Steps (2)-(12) of the attention half, src/detllm/model.py:303-412.
    ``kv``: keys/values another layer produced (then this layer projects q only)."""
    n_q, n_kv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // n_q
    eps, theta = cfg.get("rms_norm_eps", 1e-6), rope_theta(cfg)
    T = x.shape[0]
    p = prefix + "self_attn."
    q = (x @ w[p + "q_proj.weight"].T).view(T, n_q, hd)
    q = rope(rmsnorm(q, w[p + "q_norm.weight"], eps), positions, theta)   # norm, then rotation: model.py:208-215
    if kv is None:
        k = (x @ w[p + "k_proj.weight"].T).view(T, n_kv, hd)
        v = (x @ w[p + "v_proj.weight"].T).view(T, n_kv, hd)
        k = rope(rmsnorm(k, w[p + "k_norm.weight"], eps), positions, theta)
    else:
        k, v = kv
    ctx = attention(q, k, v, 1.0 / math.sqrt(hd), window)
    return ctx.reshape(T, n_q * hd) @ w[p + "o_proj.weight"].T, (k, v)


def mlp_block(x, w, prefix):
    """down(gate * sigmoid(gate) * up): src/detllm/model.py:415-427, ops/di_swiglu.py:43-45,
    float form tests/test_ops.py:240-242."""
    p = prefix + "mlp."
    g = x @ w[p + "gate_proj.weight"].T
    u = x @ w[p + "up_proj.weight"].T
    return (g * torch.sigmoid(g) * u) @ w[p + "down_proj.weight"].T


def embed(ids: torch.Tensor, w) -> torch.Tensor:
    """A pure lookup, no scaling: src/detllm/model.py:246-249."""
    return w["model.embed_tokens.weight"][ids]


def head(x, w, cfg):
    """Final norm, then the tied embedding or an own lm_head: src/detllm/model.py:284-286,
    src/detllm/prepare.py:329-331."""
    x = rmsnorm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    W = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return x @ W.T


# ------------------------------------------------------------------------------- model
def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int],
            schedule: Optional[List[Tuple[int, int, bool]]] = None, dtype=F64, rows=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (or of its positions ``rows`` only: the head of a large
    vocabulary is most of the work).  ``schedule``: (layer, cache id, writes) per stop; default every layer
    once (pre-norm residual order of src/detllm/model.py:288-428)."""
    w = {k: v.to(dtype) for k, v in w.items()}
    ids = torch.as_tensor(list(ids), dtype=torch.long)
    T = ids.numel()
    positions = torch.arange(T)
    eps = cfg.get("rms_norm_eps", 1e-6)
    if schedule is None:
        schedule = [(i, i, True) for i in range(cfg["num_hidden_layers"])]
    h = embed(ids, w)
    kvs = {}
    for layer, cache_id, writes in schedule:
        p = f"model.layers.{layer}."
        x = rmsnorm(h, w[p + "input_layernorm.weight"], eps)
        a, kv = attention_block(x, w, p, cfg, positions, layer_window(cfg, layer),
                                kv=None if writes else kvs[cache_id])
        if writes:
            kvs[cache_id] = kv
        h = h + a
        x = rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + mlp_block(x, w, p)
    return head(h if rows is None else h[list(rows)], w, cfg)


# ---------------------------------------------------------------------------- sampling
_M = (1 << 64) - 1


def _mix(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M
    return x ^ (x >> 31)


def gumbel_scores(logits: torch.Tensor, temperature: float, seed: int, request: int, step: int) -> torch.Tensor:
    """logits / T + Gumbel noise from the counter-based generator the sampler documents."""
    key = _mix(_mix(_mix(seed & _M) ^ (request & _M)) ^ (step & _M))
    V = logits.numel()
    u = torch.empty(V, dtype=F64)
    for v in range(V):
        bits = _mix(key ^ ((v * 0xD1342543DE82EF95) & _M))
        u[v] = ((bits >> 41) + 0.5) / 8388608.0
    return logits.to(F64) / temperature - torch.log(-torch.log(u))


def pick(logits: torch.Tensor, temperature: float = 0.0, seed: int = 0, request: int = 0, step: int = 0) -> int:
    """Largest score, lowest token id among equals (src/detllm/model.py:482-490)."""
    s = logits.to(F64) if temperature == 0 else gumbel_scores(logits, temperature, seed, request, step)
    return int((s == s.max()).nonzero()[0, 0])


def generate(cfg, w, prompt: Sequence[int], max_new: int, temperature: float = 0.0, seed: int = 0,
             request: int = 0, stop: Sequence[int] = (), dtype=F64):
    """Greedy or sampled continuation by re-running the whole sequence each step."""
    seq, out, step_logits = list(prompt), [], []
    for step in range(max_new):
        lg = forward(cfg, w, seq, dtype=dtype)[-1]
        tok = pick(lg, temperature, seed, request, step)
        out.append(tok)
        step_logits.append(lg)
        if tok in stop:
            break
        seq.append(tok)
    return out, step_logits
