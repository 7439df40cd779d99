"""Cross-check of tests/plain_qwen3.py against the reference's own model code, once, on a tiny
random model; the outputs are committed beside this script.

The reference has no float model of its own (its float rows call the transformers library), but
its integer runtime ``detllm.model.IntQwen3`` runs on the CPU from an artifact.  ``detllm.prepare``
cannot make one offline (it downloads the checkpoint and a calibration set), so this script builds
a synthetic int8 artifact from seeded random float weights with prepare.py's own helpers
(quant_weight_per_channel, quant_embedding_per_row, fit_gamma_dyadic, fit_dyadic_float(_vec),
ops.rope.build_rope_tables), identity smoothing, and key/value ranges taken from a float pass.
The float weights go into a model folder in the library's own format; the reference's integer
logits, scaled back to floats, go into ``reference_int8_logits.npy``.

    python tests/golden/make_golden.py --reference-src /path/to/reference/src

What the comparison can show: W8A8 integer arithmetic agrees with the float formulas to about
1e-2, so a wrong order of q/k norm and rotation, a wrong pairing of rotated dims, a wrong GQA head
map or a missing 1/sqrt(head_dim) would show (cosine far below 0.99); rounding-level details do not.
The reference drops the norms' eps and needs tied embeddings, so the tiny model has eps = 1e-12 and
tied embeddings.
"""

import argparse
import json
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
L, H, NQ, NKV, HD, I, V, THETA, MAXPOS, T = 2, 64, 4, 2, 16, 128, 256, 10000.0, 64, 24
G = NQ // NKV


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-src", required=True, help="the reference's src/ folder (holds detllm/)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference_src)
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from detllm.model import IntQwen3
    from detllm.ops.rope import build_rope_tables
    from detllm.prepare import (fit_dyadic_float, fit_dyadic_float_vec, fit_gamma_dyadic, quant_embedding_per_row,
                                quant_weight_per_channel)
    from safetensors.torch import save_file

    g = torch.Generator().manual_seed(0)

    def rn(*s, std):
        # values exactly representable in bfloat16, so that the folder and the artifact see the same weights
        return (torch.randn(*s, generator=g, dtype=torch.float64) * std).to(torch.bfloat16).to(torch.float64)

    W = {"model.embed_tokens.weight": rn(V, H, std=0.5), "model.norm.weight": 1 + rn(H, std=0.02)}
    for i in range(L):
        p = f"model.layers.{i}."
        W[p + "self_attn.q_proj.weight"] = rn(NQ * HD, H, std=0.1)
        W[p + "self_attn.k_proj.weight"] = rn(NKV * HD, H, std=0.1)
        W[p + "self_attn.v_proj.weight"] = rn(NKV * HD, H, std=0.1)
        W[p + "self_attn.o_proj.weight"] = rn(H, NQ * HD, std=0.1)
        W[p + "mlp.gate_proj.weight"] = rn(I, H, std=0.1)
        W[p + "mlp.up_proj.weight"] = rn(I, H, std=0.1)
        W[p + "mlp.down_proj.weight"] = rn(H, I, std=0.1)
        W[p + "input_layernorm.weight"] = 1 + rn(H, std=0.02)
        W[p + "post_attention_layernorm.weight"] = 1 + rn(H, std=0.02)
        W[p + "self_attn.q_norm.weight"] = 1 + rn(HD, std=0.02)
        W[p + "self_attn.k_norm.weight"] = 1 + rn(HD, std=0.02)
    ids = torch.randint(0, V, (T,), generator=g)

    # the model folder in the library's format
    folder = os.path.join(HERE, "tiny_model")
    os.makedirs(folder, exist_ok=True)
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=L, hidden_size=H,
               num_attention_heads=NQ, num_key_value_heads=NKV, head_dim=HD, intermediate_size=I, vocab_size=V,
               rope_theta=THETA, rms_norm_eps=1e-12, tie_word_embeddings=True, max_position_embeddings=MAXPOS,
               attention_bias=False, hidden_act="silu", torch_dtype="bfloat16")
    json.dump(cfg, open(os.path.join(folder, "config.json"), "w"), indent=1)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in W.items()}, os.path.join(folder, "model.safetensors"))

    # key/value ranges for the static cache scales: a float pass with the plain implementation's parts
    sys.path.insert(0, os.path.dirname(HERE))
    import plain_qwen3 as plain
    pos = torch.arange(T)
    h = plain.embed(ids, W)
    stats = []
    for i in range(L):
        p = f"model.layers.{i}."
        x = plain.rmsnorm(h, W[p + "input_layernorm.weight"], 1e-12)
        a, (k, v) = plain.attention_block(x, W, p, cfg, pos, None)
        stats.append((k.abs().amax(0), v.abs().amax((0, 2))))
        h = h + a
        h = h + plain.mlp_block(plain.rmsnorm(h, W[p + "post_attention_layernorm.weight"], 1e-12), W, p)

    # the synthetic artifact, through the reference's own quantisation helpers
    ten, acfg = {}, dict(n_layers=L, hidden=H, n_q_heads=NQ, n_kv_heads=NKV, head_dim=HD, intermediate=I, vocab=V,
                         layers=[])

    def add(name, Wf, gamma=None):
        w8, m, k = quant_weight_per_channel(Wf * (gamma[None, :] if gamma is not None else 1.0))
        ten[name + ".w8t"] = w8.t().contiguous()
        ten[name + ".m"] = m
        return {"k": k}
    E = W["model.embed_tokens.weight"]
    ten["embed.e8"], ten["embed.m"], ten["embed.k"] = quant_embedding_per_row(E)
    acfg["head"] = add("head", E, W["model.norm.weight"])
    ten["rope.cos"], ten["rope.sin"] = build_rope_tables(HD, MAXPOS, THETA)
    one = lambda n: torch.ones(n, dtype=torch.int64)
    for i in range(L):
        p, ap_, Lc = f"model.layers.{i}.", f"layers.{i}.", {}
        ga, gm = W[p + "input_layernorm.weight"], W[p + "post_attention_layernorm.weight"]
        for nm, key, gam in (("q", "self_attn.q_proj", ga), ("k", "self_attn.k_proj", ga), ("v", "self_attn.v_proj", ga),
                             ("o", "self_attn.o_proj", None), ("gate", "mlp.gate_proj", gm), ("up", "mlp.up_proj", gm),
                             ("down", "mlp.down_proj", None)):
            Lc[nm] = add(ap_ + nm, W[p + key + ".weight"], gam)
        ten[ap_ + "q_norm.m"], Lc["q_norm_k"] = fit_gamma_dyadic(W[p + "self_attn.q_norm.weight"])
        ten[ap_ + "k_norm.m"], Lc["k_norm_k"] = fit_gamma_dyadic(W[p + "self_attn.k_norm.weight"])
        for nm, n in (("as", H), ("ms", H), ("ds", I), ("os", NQ * HD)):
            ten[ap_ + nm + "_m"] = one(n)
            Lc[nm + "_k"] = 0
        ten[ap_ + "qs_m"] = one(NKV * HD).view(NKV, HD)
        Lc["qs_k"] = 0
        kmax, vmax = stats[i]
        s_kh = kmax.amax(1) * 1.05 / 127
        ten[ap_ + "kq_m"], ten[ap_ + "kq_k"] = fit_dyadic_float_vec(s_kh[:, None].expand(NKV, HD).contiguous())
        ks = [fit_dyadic_float(float(s) / math.sqrt(HD)) for s in s_kh]
        vq = [fit_dyadic_float(float(x) * 1.05 / 127) for x in vmax]
        ten[ap_ + "ks_m"] = torch.tensor([a for a, _ in ks]); ten[ap_ + "ks_k"] = torch.tensor([b for _, b in ks])
        ten[ap_ + "vq_m"] = torch.tensor([a for a, _ in vq]); ten[ap_ + "vq_k"] = torch.tensor([b for _, b in vq])
        acfg["layers"].append(Lc)
    import tempfile
    art = tempfile.mkdtemp()
    save_file({k: v.contiguous() for k, v in ten.items()}, os.path.join(art, "model.safetensors"))
    json.dump(acfg, open(os.path.join(art, "config.json"), "w"))

    m = IntQwen3(art, backend="cpu")
    lg, xm, xk, _ = m.forward(ids[None], torch.arange(T)[None], guard=True)
    val = lg[0].double() * m.head_m.double() * xm[0].double() * torch.pow(2.0, -(xk[0].double() + m.head_k))
    np.save(os.path.join(HERE, "reference_int8_logits.npy"), val.numpy().astype(np.float32))
    json.dump({"ids": ids.tolist()}, open(os.path.join(HERE, "tokens.json"), "w"))
    ref = plain.forward(cfg, W, ids.tolist())
    cos = torch.nn.functional.cosine_similarity(val, ref, dim=-1)
    print("reference int8 runtime vs plain implementation: cosine min %.5f mean %.5f; argmax agree %d/%d"
          % (cos.min(), cos.mean(), int((val.argmax(-1) == ref.argmax(-1)).sum()), T))


if __name__ == "__main__":
    main()
