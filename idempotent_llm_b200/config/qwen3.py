"""Typed configuration of the Qwen3 dense decoder, read from its config.json.

Keys and their meaning follow what the reference reads from the checkpoint's
configuration (src/detllm/prepare.py:32-35, 244-259, 301-303): model_type,
tie_word_embeddings, num_hidden_layers, hidden_size, num_attention_heads,
num_key_value_heads, head_dim, intermediate_size, vocab_size,
max_position_embeddings, eos_token_id and rope_theta (plain or inside
rope_parameters).  The reference drops the norms' eps (src/detllm/ops/
di_rmsnorm.py:14, 50) and refuses untied embeddings (prepare.py:246); here
rms_norm_eps is read and added to the mean inside the square root, and an
untied lm_head is its own matrix.  The window keys (use_sliding_window,
sliding_window, max_window_layers) are never read by the reference; here a
layer whose index is >= max_window_layers attends to the last
``sliding_window`` keys when use_sliding_window is true.
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, asdict
from typing import Optional, Tuple

from .specs import (AttentionNames, AttentionSpec, ConfigError, GatedMLPNames, GatedMLPSpec, LayerSpec, ModelSpec,
                    NormSpec, RotarySpec, default_schedule)

ARCHITECTURE = "Qwen3ForCausalLM"

# The checkpoint's tensor names, as the reference's offline pass walks them (src/detllm/prepare.py:323-384):
# behind "model.layers.{i}." for the layers' tensors.
ATTENTION_NAMES = AttentionNames(q="self_attn.q_proj.weight", k="self_attn.k_proj.weight", v="self_attn.v_proj.weight",
                                 o="self_attn.o_proj.weight", q_norm="self_attn.q_norm.weight",
                                 k_norm="self_attn.k_norm.weight")
MLP_NAMES = GatedMLPNames(gate="mlp.gate_proj.weight", up="mlp.up_proj.weight", down="mlp.down_proj.weight")


def _need(d: dict, key: str):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    return d[key]


@dataclass(frozen=True)
class Qwen3Config:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    eos_token_id: Optional[Tuple[int, ...]]
    use_sliding_window: bool
    sliding_window: Optional[int]
    max_window_layers: int
    initializer_range: float
    torch_dtype: str
    architecture: str = ARCHITECTURE

    # ------------------------------------------------------------------ read
    @classmethod
    def from_dict(cls, d: dict) -> "Qwen3Config":
        archs = d.get("architectures") or []
        if ARCHITECTURE not in archs:
            raise ConfigError(f"config.json: architectures={archs!r}, expected [{ARCHITECTURE!r}]")
        if d.get("model_type", "qwen3") != "qwen3":
            raise ConfigError(f"config.json: model_type={d.get('model_type')!r}, expected 'qwen3'")
        if d.get("attention_bias", False):
            raise ConfigError("config.json: attention_bias=true is not part of this architecture "
                              "(the reference reads no bias: src/detllm/prepare.py:312-321)")
        if d.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"config.json: hidden_act={d.get('hidden_act')!r}, only 'silu' exists here")
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError("config.json: rope_scaling is set; only plain rotary angles are built")
        hidden = int(_need(d, "hidden_size"))
        n_q = int(_need(d, "num_attention_heads"))
        n_kv = int(d.get("num_key_value_heads") or n_q)
        if "head_dim" in d and d["head_dim"] is not None:
            hd = int(d["head_dim"])
        else:
            if hidden % n_q:
                raise ConfigError("config.json: head_dim absent and hidden_size is no multiple of num_attention_heads")
            hd = hidden // n_q
        if "rope_theta" in d and d["rope_theta"] is not None:
            theta = float(d["rope_theta"])
        elif isinstance(d.get("rope_parameters"), dict) and "rope_theta" in d["rope_parameters"]:
            theta = float(d["rope_parameters"]["rope_theta"])
        else:
            theta = 10000.0
        eos = d.get("eos_token_id")
        if eos is not None:
            eos = tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        n_layers = int(_need(d, "num_hidden_layers"))
        window = d.get("sliding_window")
        cfg = cls(
            num_hidden_layers=n_layers,
            hidden_size=hidden,
            num_attention_heads=n_q,
            num_key_value_heads=n_kv,
            head_dim=hd,
            intermediate_size=int(_need(d, "intermediate_size")),
            vocab_size=int(_need(d, "vocab_size")),
            rope_theta=theta,
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            max_position_embeddings=int(d.get("max_position_embeddings", 40960)),
            eos_token_id=eos,
            use_sliding_window=bool(d.get("use_sliding_window", False)),
            sliding_window=None if window is None else int(window),
            max_window_layers=int(d.get("max_window_layers", n_layers)),
            initializer_range=float(d.get("initializer_range", 0.02)),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_dir(cls, model_dir: str) -> "Qwen3Config":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def validate(self) -> None:
        pos = ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
               "head_dim", "intermediate_size", "vocab_size", "max_position_embeddings")
        for k in pos:
            if getattr(self, k) <= 0:
                raise ConfigError(f"config.json: {k} must be positive, got {getattr(self, k)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"config.json: num_attention_heads={self.num_attention_heads} is no multiple "
                              f"of num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim={self.head_dim} must be even for rotary pairs")
        if not self.rms_norm_eps >= 0:
            raise ConfigError("config.json: rms_norm_eps must be >= 0")
        if self.rope_theta <= 0:
            raise ConfigError("config.json: rope_theta must be positive")
        if self.use_sliding_window and (self.sliding_window is None or self.sliding_window <= 0):
            raise ConfigError("config.json: use_sliding_window=true needs a positive sliding_window")

    # ----------------------------------------------------------------- write
    def to_dict(self) -> dict:
        d = asdict(self)
        d.pop("architecture")
        d["architectures"] = [ARCHITECTURE]
        d["model_type"] = "qwen3"
        d["attention_bias"] = False
        d["hidden_act"] = "silu"
        d["rope_scaling"] = None
        if self.eos_token_id is None:
            d["eos_token_id"] = None
        elif len(self.eos_token_id) == 1:
            d["eos_token_id"] = self.eos_token_id[0]
        else:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    # ------------------------------------------------------------ translation
    def window_of_layer(self, i: int) -> Optional[int]:
        if self.use_sliding_window and i >= self.max_window_layers:
            return self.sliding_window
        return None

    def to_model_spec(self) -> ModelSpec:
        rot = RotarySpec(theta=self.rope_theta, dim=self.head_dim,
                         max_positions=self.max_position_embeddings)
        layers = []
        for i in range(self.num_hidden_layers):
            mixer = AttentionSpec(
                hidden=self.hidden_size, n_heads=self.num_attention_heads,
                n_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                softmax_scale=1.0 / math.sqrt(self.head_dim),  # src/detllm/prepare.py:338
                qk_norm=True, qk_norm_eps=self.rms_norm_eps, position=rot, names=ATTENTION_NAMES,
                window=self.window_of_layer(i))
            ff = GatedMLPSpec(hidden=self.hidden_size, intermediate=self.intermediate_size, names=MLP_NAMES)
            norm = NormSpec(size=self.hidden_size, eps=self.rms_norm_eps)
            layers.append(LayerSpec(prefix=f"model.layers.{i}.", mixer=mixer, feed_forward=ff,
                                    mixer_norm=norm, feed_forward_norm=norm,
                                    mixer_norm_prefix="input_layernorm.",
                                    feed_forward_norm_prefix="post_attention_layernorm."))
        return ModelSpec(
            embed_name="model.embed_tokens.weight", final_norm_prefix="model.norm.", head_name="lm_head.weight",
            architecture=ARCHITECTURE, vocab_size=self.vocab_size, hidden=self.hidden_size,
            layers=tuple(layers), schedule=default_schedule(self.num_hidden_layers),
            final_norm=NormSpec(size=self.hidden_size, eps=self.rms_norm_eps),
            tie_embeddings=self.tie_word_embeddings,
            max_positions=self.max_position_embeddings,
            stop_token_ids=self.eos_token_id or (),
            init_std=self.initializer_range)
