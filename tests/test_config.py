"""Configuration, registry and presets (CPU)."""

import json

import pytest

import helpers
from idempotent_llm_b200.config import ConfigError, Qwen3Config, RunEntry, default_schedule
from idempotent_llm_b200.config.presets import preset, preset_names
from idempotent_llm_b200.config.specs import ModelSpec
from idempotent_llm_b200 import registry


def test_reads_every_key_of_both_tiny_configs():
    a, b = Qwen3Config.from_dict(helpers.TINY["A"]), Qwen3Config.from_dict(helpers.TINY["B"])
    for k in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
              "intermediate_size", "vocab_size", "rope_theta", "rms_norm_eps", "tie_word_embeddings"):
        assert getattr(a, k) == helpers.TINY["A"][k]
        assert getattr(b, k) == helpers.TINY["B"][k]
        assert getattr(a, k) != getattr(b, k), f"the tiny configurations share {k}"
    assert a.eos_token_id == (255,) and b.eos_token_id == (318, 319)
    assert b.num_attention_heads * b.head_dim != b.hidden_size


def test_spec_carries_sizes_per_layer_and_window():
    spec = Qwen3Config.from_dict(helpers.TINY["B"]).to_model_spec()
    assert [l.mixer.window for l in spec.layers] == [None, 80, 80]
    assert spec.layers[0].mixer.head_dim == 32 and spec.layers[0].feed_forward.intermediate == 224
    assert spec.final_norm.eps == 1e-5 and not spec.tie_embeddings
    assert spec.schedule == default_schedule(3)
    assert abs(spec.layers[0].mixer.softmax_scale - 32 ** -0.5) < 1e-12


def test_defaults_and_rope_parameters():
    d = dict(helpers.TINY["A"])
    d.pop("head_dim"); d.pop("rope_theta"); d.pop("num_key_value_heads")
    d["rope_parameters"] = {"rope_theta": 12345.0}
    c = Qwen3Config.from_dict(d)
    assert c.head_dim == 64 // 4 and c.rope_theta == 12345.0 and c.num_key_value_heads == 4


@pytest.mark.parametrize("change, word", [
    ({"architectures": ["LlamaForCausalLM"]}, "architectures"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"use_sliding_window": True}, "sliding_window"),
    ({"hidden_size": None}, "hidden_size"),
])
def test_bad_configs_raise(change, word):
    d = dict(helpers.TINY["A"]); d.update(change)
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(d)


def test_round_trip_through_config_json(tmp_path):
    c = Qwen3Config.from_dict(helpers.TINY["B"])
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    arch, c2 = registry.read_config(str(tmp_path))
    assert arch.name == "Qwen3ForCausalLM" and c2 == c


def test_registry_unknown_and_missing(tmp_path):
    with pytest.raises(ConfigError, match="unknown architecture"):
        registry.architecture("NopeForCausalLM")
    with pytest.raises(ConfigError, match="does not exist"):
        registry.read_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{}")
    with pytest.raises(ConfigError, match="architectures"):
        registry.read_config(str(tmp_path))


def test_schedule_validation():
    spec = Qwen3Config.from_dict(helpers.TINY["A"]).to_model_spec()
    kw = {f: getattr(spec, f) for f in ("architecture", "vocab_size", "hidden", "layers", "final_norm",
                                        "tie_embeddings", "max_positions", "embed_name", "final_norm_prefix", "head_name")}
    ModelSpec(schedule=(RunEntry(0, 0), RunEntry(1, 1), RunEntry(1, 2)), **kw)          # a layer named twice
    with pytest.raises(ConfigError, match="written by two"):
        ModelSpec(schedule=(RunEntry(0, 0), RunEntry(1, 0)), **kw)
    with pytest.raises(ConfigError, match="before anything wrote"):
        ModelSpec(schedule=(RunEntry(0, 0, writes_cache=False),), **kw)
    with pytest.raises(ConfigError, match="names layer"):
        ModelSpec(schedule=(RunEntry(5, 0),), **kw)


def test_presets_match_the_quoted_sizes():
    assert {"qwen3-0.6b", "qwen3-8b", "qwen3-32b", "tiny-a", "tiny-b"} <= set(preset_names())
    c = preset("qwen3-0.6b")
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
            c.intermediate_size, c.vocab_size, c.tie_word_embeddings) == (28, 1024, 16, 8, 128, 3072, 151936, True)
    c = preset("qwen3-32b")
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.intermediate_size) == (64, 5120, 64, 25600)
