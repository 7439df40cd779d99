"""Safetensors reading/writing, loading by name and its one error, random weights (CPU)."""

import json
import os

import pytest
import torch

import helpers
from idempotent_llm_b200.config import Qwen3Config
from idempotent_llm_b200.engine import declare_weights
from idempotent_llm_b200.weights import (SafetensorsFile, WeightError, load_weights, write_random_model,
                                         write_safetensors)
from idempotent_llm_b200.weights.safetensors_io import SafetensorsError


def _folder(tmp_path, name="A", dtype=torch.bfloat16, seed=1):
    return helpers.make_model_dir(helpers.TINY[name], str(tmp_path), seed=seed, dtype=dtype)


def _rewrite(d, edit):
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.get(n).clone() for n in f.names()}
    del f
    edit(tensors)
    write_safetensors(path, list(tensors.items()))


def test_own_reader_agrees_with_the_safetensors_library(tmp_path):
    from safetensors.torch import load_file, save_file
    d = _folder(tmp_path)
    lib = load_file(os.path.join(d, "model.safetensors"))
    own = SafetensorsFile(os.path.join(d, "model.safetensors"))
    assert sorted(lib) == sorted(own.names())
    for n in lib:
        assert torch.equal(lib[n], own.get(n)) and lib[n].dtype == own.get(n).dtype
    save_file({"x": torch.arange(6, dtype=torch.int64).view(2, 3), "y": torch.ones(3)}, str(tmp_path / "o.safetensors"))
    o = SafetensorsFile(str(tmp_path / "o.safetensors"))
    assert o.info("x") == (torch.int64, (2, 3)) and o.get("x").tolist() == [[0, 1, 2], [3, 4, 5]]


def test_names_shapes_and_dtypes_of_a_random_folder(tmp_path):
    d = _folder(tmp_path, "B")
    cfg = Qwen3Config.from_dict(helpers.TINY["B"])
    w = load_weights(d, declare_weights(cfg.to_model_spec()), "cpu")
    assert w["model.layers.2.self_attn.q_proj.weight"].shape == (6 * 32, 96)
    assert w["model.layers.0.self_attn.k_norm.weight"].shape == (32,)
    assert w["model.layers.1.mlp.down_proj.weight"].shape == (96, 224)
    assert w["lm_head.weight"].shape == (320, 96)
    assert all(t.dtype == torch.bfloat16 for t in w.values())
    assert abs(float(w["model.norm.weight"].float().mean()) - 1.0) < 0.05           # 1 + N(0, std)
    assert abs(float(w["model.embed_tokens.weight"].float().std()) - 0.05) < 0.005   # N(0, std)
    assert json.load(open(os.path.join(d, "config.json")))["vocab_size"] == 320


def test_seed_decides_the_weights(tmp_path):
    a = SafetensorsFile(os.path.join(_folder(tmp_path / "a", seed=1), "model.safetensors"))
    b = SafetensorsFile(os.path.join(_folder(tmp_path / "b", seed=1), "model.safetensors"))
    c = SafetensorsFile(os.path.join(_folder(tmp_path / "c", seed=2), "model.safetensors"))
    n = "model.layers.1.mlp.up_proj.weight"
    assert torch.equal(a.get(n), b.get(n)) and not torch.equal(a.get(n), c.get(n))


def test_32_bit_storage_stays_32_bit_and_integers_become_int32(tmp_path):
    from idempotent_llm_b200.weights import storage_dtype
    d = _folder(tmp_path, dtype=torch.float32)
    cfg = Qwen3Config.from_dict(helpers.TINY["A"])
    w = load_weights(d, declare_weights(cfg.to_model_spec()), "cpu")
    assert all(t.dtype == torch.float32 for t in w.values())
    # float16 is widened, not narrowed to bfloat16: the 32-bit path must see the stored values exactly
    assert storage_dtype(torch.float16) == torch.float32 and storage_dtype(torch.bfloat16) == torch.bfloat16
    assert storage_dtype(torch.int64) == torch.int32
    assert storage_dtype(torch.uint8) == torch.int32 and storage_dtype(torch.float32) == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = _folder(tmp_path)

    def edit(t):
        del t["model.layers.0.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
        t["model.layers.1.self_attn.q_norm.weight"] = torch.ones(17, dtype=torch.bfloat16)
    _rewrite(d, edit)
    cfg = Qwen3Config.from_dict(helpers.TINY["A"])
    with pytest.raises(WeightError) as e:
        load_weights(d, declare_weights(cfg.to_model_spec()), "cpu")
    err = e.value
    assert sorted(err.missing) == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert [(n, got, want) for n, got, want in err.wrong_shape] == [
        ("model.layers.1.self_attn.q_norm.weight", (17,), (16,))]
    msg = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (1)", "is [17], expected [16]"):
        assert word in msg


def test_tied_model_tolerates_an_lm_head_and_untied_requires_it(tmp_path):
    d = _folder(tmp_path / "a", "A")
    _rewrite(d, lambda t: t.__setitem__("lm_head.weight", t["model.embed_tokens.weight"].clone()))
    cfg = Qwen3Config.from_dict(helpers.TINY["A"])
    with pytest.warns(UserWarning, match="lm_head.weight is in the file but the model does not use it"):
        w = load_weights(d, declare_weights(cfg.to_model_spec()), "cpu")
    assert "lm_head.weight" not in w
    d = _folder(tmp_path / "b", "B")
    _rewrite(d, lambda t: t.pop("lm_head.weight"))
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_weights(d, declare_weights(Qwen3Config.from_dict(helpers.TINY["B"]).to_model_spec()), "cpu")


def test_integer_tensor_under_a_weight_name_is_refused(tmp_path):
    d = _folder(tmp_path)
    _rewrite(d, lambda t: t.__setitem__("model.norm.weight", torch.ones(64, dtype=torch.int32)))
    with pytest.raises(WeightError, match="wrong dtype"):
        load_weights(d, declare_weights(Qwen3Config.from_dict(helpers.TINY["A"]).to_model_spec()), "cpu")


def test_float16_is_kept_exactly_and_unknown_dtypes_matter_only_where_declared(tmp_path):
    import struct
    d = _folder(tmp_path, dtype=torch.float32)
    cfg = Qwen3Config.from_dict(helpers.TINY["A"])
    half = {}
    _rewrite(d, lambda t: [half.__setitem__(n, t[n].to(torch.float16)) or t.__setitem__(n, t[n].to(torch.float16)) for n in list(t)])
    w = load_weights(d, declare_weights(cfg.to_model_spec()), "cpu")
    assert all(t.dtype == torch.float32 for t in w.values())
    assert all(torch.equal(w[n], half[n].float()) for n in w)
    # a tensor of a dtype this reader does not know: harmless while nobody declares it ...
    path = os.path.join(d, "model.safetensors")
    raw = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    end = max(e["data_offsets"][1] for k, e in header.items() if k != "__metadata__")
    header["extra.scale"] = {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [end, end + 4]}
    hb = json.dumps(header).encode()
    open(path, "wb").write(struct.pack("<Q", len(hb)) + hb + raw[8 + hlen:] + b"\0\0\0\0")
    f = SafetensorsFile(path)
    assert f.info("extra.scale") == ("F8_E4M3", (4,))
    with pytest.raises(SafetensorsError, match="unsupported dtype F8_E4M3"):
        f.get("extra.scale")
    del f
    with pytest.raises(WeightError, match="unexpected \\(1\\): extra.scale"):
        load_weights(d, declare_weights(cfg.to_model_spec()), "cpu")
    # ... and a wrong dtype, named, where a declared tensor has it
    header["model.norm.weight"]["dtype"] = "F8_E4M3"
    del header["extra.scale"]
    hb = json.dumps(header).encode()
    open(path, "wb").write(struct.pack("<Q", len(hb)) + hb + raw[8 + hlen:])
    with pytest.raises(WeightError, match="wrong dtype \\(1\\): model.norm.weight is F8_E4M3"):
        load_weights(d, declare_weights(cfg.to_model_spec()), "cpu")
    # offsets that run backwards or start before the data
    header["model.norm.weight"]["dtype"] = "F16"
    header["model.norm.weight"]["data_offsets"] = [-128, 0]
    hb = json.dumps(header).encode()
    open(path, "wb").write(struct.pack("<Q", len(hb)) + hb + raw[8 + hlen:])
    with pytest.raises(SafetensorsError, match="outside the file"):
        SafetensorsFile(path)


def test_broken_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x05\x00")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    with pytest.raises(SafetensorsError, match="neither"):
        from idempotent_llm_b200.weights import SafetensorsDir
        SafetensorsDir(str(tmp_path / "nothing"))


def test_sharded_folder(tmp_path):
    from idempotent_llm_b200.weights import SafetensorsDir
    d = _folder(tmp_path)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    names = f.names()
    half = len(names) // 2
    write_safetensors(os.path.join(d, "s1.safetensors"), [(n, f.get(n).clone()) for n in names[:half]])
    write_safetensors(os.path.join(d, "s2.safetensors"), [(n, f.get(n).clone()) for n in names[half:]])
    ref = {n: f.get(n).clone() for n in names}
    del f
    os.remove(os.path.join(d, "model.safetensors"))
    wm = {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}
    json.dump({"weight_map": wm}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    sd = SafetensorsDir(d)
    assert sorted(sd.names()) == sorted(names)
    assert all(torch.equal(sd.get(n), ref[n]) for n in names)
