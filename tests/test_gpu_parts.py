"""Each part alone against the plain implementation's function for it; a schedule that names a
layer twice and shares a cache; and toy parts -- a mixer with state of its own, a feed-forward that
routes, another position encoding -- that are registered, built and stepped from this file alone (GPU)."""

from dataclasses import dataclass

import pytest
import torch

import helpers
import plain_qwen3 as plain
from idempotent_llm_b200.cache import CacheNeed, SequenceCache
from idempotent_llm_b200.config import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec, Qwen3Config,
                                        RotarySpec, RunEntry)
from idempotent_llm_b200.config.qwen3 import ATTENTION_NAMES, MLP_NAMES
from idempotent_llm_b200.config.specs import AttentionNames, GatedMLPNames
from idempotent_llm_b200.engine import CausalLM, Engine, cache_needs, declare_weights
from idempotent_llm_b200.engine.batch import context_from_packed, pack_step_host
from idempotent_llm_b200.parts import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, FeedForward, Mixer,
                                       PositionEncoding, Runtime)
from idempotent_llm_b200.weights import TensorDecl, random_weights

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


def _rt(dtype):
    from idempotent_llm_b200.kernels import Kernels
    dev = torch.device("cuda:0")
    return Runtime(device=dev, dtype=DT[dtype], kernels=Kernels(DT[dtype], dev))


def _ctx(slots, starts, lens):
    packed, n, q_lens = pack_step_host(slots, starts, [[0] * L for L in lens])
    return context_from_packed(packed.cuda(), n, slots, q_lens, starts)


def _w64(w):
    return {k: v.double().cpu() for k, v in w.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    rt = _rt(dtype)
    spec = NormSpec(size=100, eps=3e-4)
    cls = NORMS.get(spec.kind)
    assert [(d.name, d.shape, d.init) for d in cls.declare(spec, "n.")] == [("n.weight", (100,), "one_plus_normal")]
    w = random_weights(cls.declare(spec, "n."), 1, 0.3, dtype=DT[dtype], device="cuda")
    part = cls(spec, w, "n.", rt)
    h = torch.randn(9, 100, device="cuda")
    x = part.forward(h, None, None)
    assert x.dtype == DT[dtype]
    assert helpers.rel_err(x, plain.rmsnorm(h.double().cpu(), _w64(w)["n.weight"], 3e-4)) < helpers.TOL[dtype]


def test_rotary_part_is_shared_per_step():
    rt = _rt("float32")
    spec = RotarySpec(theta=7e4, dim=24, max_positions=4096)
    part = POSITIONS.get(spec.kind)(spec, {}, "", rt)
    ctx = _ctx([0, 1], [100, 3000], [3, 2])
    t = part.tables(ctx)
    assert part.tables(ctx) is t and t.shape == (5, 12, 2)
    x = torch.randn(5, 1, 24, dtype=F64)
    want = plain.rope(x, ctx.positions.cpu(), 7e4)
    c, s = t[..., 0].double().cpu()[:, None, :], t[..., 1].double().cpu()[:, None, :]
    got = torch.cat([x[..., :12] * c - x[..., 12:] * s, x[..., 12:] * c + x[..., :12] * s], -1)
    assert (got - want).abs().max() < 1e-12


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [None, 40])
def test_attention_part_prompt_then_single_tokens(dtype, window):
    rt = _rt(dtype)
    cfg = dict(num_attention_heads=6, num_key_value_heads=2, head_dim=32, hidden_size=72, rms_norm_eps=1e-5,
               rope_theta=3e4)
    spec = AttentionSpec(hidden=72, n_heads=6, n_kv_heads=2, head_dim=32, softmax_scale=32 ** -0.5, qk_norm=True,
                         qk_norm_eps=1e-5, position=RotarySpec(3e4, 32, 4096), names=ATTENTION_NAMES, window=window)
    cls = MIXERS.get(spec.kind)
    w = random_weights(cls.declare(spec, "L."), 2, 0.2, dtype=DT[dtype], device="cuda")
    assert cls.cache_need(spec) == CacheNeed("window" if window else "full", 2, 32, window=window)
    part = cls(spec, w, "L.", rt)
    cache = SequenceCache({0: cls.cache_need(spec)}, 64 * 8, DT[dtype], "cuda:0", max_seqs=2)
    slot = cache.alloc_slot()
    T, pre = 150, 140
    x = (torch.randn(T, 72, generator=torch.Generator().manual_seed(3)) * 1.5).to(DT[dtype])
    ref, _ = plain.attention_block(x.double(), _w64(w), "L.", cfg, torch.arange(T), window)
    outs = []
    for lo, hi in [(0, pre)] + [(i, i + 1) for i in range(pre, T)]:
        cache.reserve([(slot, hi)]); cache.flush()
        ctx = _ctx([slot], [lo], [hi - lo])
        outs.append(part.forward(x[lo:hi].contiguous().cuda(), ctx, cache.view(0), None, True).sum(0))
        cache.set_length(slot, hi)
    assert helpers.rel_err(torch.cat(outs), ref) < helpers.TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(dtype):
    rt = _rt(dtype)
    spec = GatedMLPSpec(hidden=72, intermediate=200, names=MLP_NAMES)
    cls = FEED_FORWARDS.get(spec.kind)
    w = random_weights(cls.declare(spec, "L."), 4, 0.2, dtype=DT[dtype], device="cuda")
    part = cls(spec, w, "L.", rt)
    x = torch.randn(11, 72).to(DT[dtype])
    got = part.forward(x.cuda(), None).sum(0)
    assert got.dtype == torch.float32
    assert helpers.rel_err(got, plain.mlp_block(x.double(), _w64(w), "L.")) < helpers.TOL[dtype]


def test_unknown_kinds_and_bad_parts_are_refused():
    with pytest.raises(KeyError, match="no mixer registered"):
        MIXERS.get("nope")
    with pytest.raises(ValueError, match="activation"):
        FEED_FORWARDS.get("gated_mlp")(GatedMLPSpec(8, 8, names=MLP_NAMES, activation="gelu"), {}, "", None)
    # a position encoding whose rotation sits otherwise in the head is refused by name, before any shape meets a kernel
    for pos in (RotarySpec(1e4, 16, 512), RotarySpec(1e4, 32, 512, variant="interleaved")):
        bad = AttentionSpec(hidden=64, n_heads=2, n_kv_heads=2, head_dim=32, softmax_scale=0.2, qk_norm=False,
                            qk_norm_eps=1e-6, position=pos, names=ATTENTION_NAMES)
        with pytest.raises(ValueError, match="half_whole_head"):
            MIXERS.get("attention")(bad, {ATTENTION_NAMES.q: torch.zeros(64, 64), ATTENTION_NAMES.k: torch.zeros(64, 64),
                                          ATTENTION_NAMES.v: torch.zeros(64, 64), ATTENTION_NAMES.o: torch.zeros(64, 64)},
                                    "", Runtime(device=torch.device("cpu"), dtype=torch.float32, kernels=None))


def _custom_schedule_spec(schedule):
    base = Qwen3Config.from_dict(helpers.TINY["A"]).to_model_spec()
    layers = list(base.layers)
    if any(not e.writes_cache for e in schedule):
        # a third layer without k/v of its own that reads layer 1's cache
        m = layers[1].mixer
        reader = AttentionSpec(**{**m.__dict__, "kv_from_other": True})
        layers.append(LayerSpec(prefix="model.layers.2.", mixer=reader, feed_forward=layers[1].feed_forward,
                                mixer_norm=layers[1].mixer_norm, feed_forward_norm=layers[1].feed_forward_norm,
                                mixer_norm_prefix=layers[1].mixer_norm_prefix,
                                feed_forward_norm_prefix=layers[1].feed_forward_norm_prefix))
    kw = {f: getattr(base, f) for f in ("architecture", "vocab_size", "hidden", "final_norm", "tie_embeddings",
                                        "max_positions", "embed_name", "final_norm_prefix", "head_name")}
    return ModelSpec(layers=tuple(layers), schedule=tuple(schedule), **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_named_twice_and_a_layer_reading_anothers_cache(dtype):
    rt = _rt(dtype)
    schedule = [RunEntry(0, 0), RunEntry(1, 1), RunEntry(1, 2), RunEntry(2, 1, writes_cache=False)]
    spec = _custom_schedule_spec(schedule)
    decls = declare_weights(spec)
    assert "model.layers.2.self_attn.k_proj.weight" not in {d.name for d in decls}
    w = random_weights(decls, 5, 0.05, dtype=DT[dtype], device="cuda")
    model = CausalLM(spec, w, rt)
    assert sorted(cache_needs(spec)) == [0, 1, 2]
    eng = Engine(model, 64 * 8, max_seqs=2)
    ids = helpers.rand_ids(80, 256, 6)
    w64 = _w64(w)
    # the reader layer has no k/v of its own: the plain forward borrows layer 1's tensors for names it never uses
    cfg = dict(helpers.TINY["A"], num_hidden_layers=3)
    ref = plain.forward(cfg, w64, ids, schedule=[(0, 0, True), (1, 1, True), (1, 2, True), (2, 1, False)])
    slot = eng.open()
    got = [eng.step([(slot, ids[:70])], [list(range(70))])] + [eng.step([(slot, [t])]).clone() for t in ids[70:]]
    eng.close(slot)
    assert helpers.rel_err(torch.cat(got), ref) < helpers.TOL[dtype]


# ------------------------------------------------------------------ a toy mixer with state
@dataclass(frozen=True)
class ToyDecaySpec:
    hidden: int
    decay: float
    kind: str = "toy_decay"


class ToyDecayMixer(Mixer):
    """s_t = decay * s_{t-1} + x_t per sequence (state of fixed size, kept in the cache's state
    region); output = s_t . W^T.  Plain torch on the device: a toy, not a kernel."""

    graph_safe = False          # reads cu_q and slots on the host

    @classmethod
    def declare(cls, spec, prefix):
        return [TensorDecl(prefix + "toy.weight", (spec.hidden, spec.hidden))]

    @classmethod
    def cache_need(cls, spec):
        return CacheNeed(kind="none", state_shape=(spec.hidden,), state_dtype=torch.float32)

    def __init__(self, spec, weights, prefix, rt):
        self.spec, self.rt = spec, rt
        self.w = weights[prefix + "toy.weight"].float()

    def forward(self, x, ctx, kv, state, writes_cache):
        assert kv is None and state is not None
        out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        cu = ctx.cu_q.tolist()
        for i, slot in enumerate(ctx.slots.tolist()):
            s = state[slot]
            for t in range(cu[i], cu[i + 1]):
                s = self.spec.decay * s + x[t].float()
                out[t] = s @ self.w.T
            state[slot] = s
        return out.unsqueeze(0)


class ToyDecayMixerOnDevice(ToyDecayMixer):
    """The same mixer with its single-token step written without a look at the host, so that the engine may
    capture such steps in a graph.  Its state is read, then written: a step that runs twice shows."""

    graph_safe = True

    def forward(self, x, ctx, kv, state, writes_cache):
        if not ctx.single_token:
            return super().forward(x, ctx, kv, state, writes_cache)
        idx = ctx.slots.long()
        s = self.spec.decay * state.index_select(0, idx) + x.float()
        state.index_copy_(0, idx, s)
        return (s @ self.w.T).unsqueeze(0)


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int = 97
    hidden_size: int = 48
    decay: float = 0.75

    @classmethod
    def from_dict(cls, d):
        return cls(**{k: d[k] for k in ("vocab_size", "hidden_size", "decay") if k in d})

    def to_model_spec(self):
        # every tensor name is this toy architecture's own: the product's parts take them from the specs
        norm = NormSpec(self.hidden_size, 1e-5, weight="scale")
        ff = GatedMLPSpec(self.hidden_size, 64, names=TOY_MLP_NAMES)
        attn = AttentionSpec(hidden=self.hidden_size, n_heads=3, n_kv_heads=1, head_dim=16, softmax_scale=0.25,
                             qk_norm=True, qk_norm_eps=1e-5, position=RotarySpec(1e4, 16, 512), names=TOY_ATTN_NAMES)
        layer = lambda i, mixer: LayerSpec(f"blk{i}.", mixer, ff, norm, norm, mixer_norm_prefix="ln_a.",
                                           feed_forward_norm_prefix="ln_b.")
        layers = (layer(0, ToyDecaySpec(self.hidden_size, self.decay)), layer(1, attn),
                  layer(2, ToyDecaySpec(self.hidden_size, self.decay)))
        return ModelSpec(architecture="ToyForCausalLM", vocab_size=self.vocab_size, hidden=self.hidden_size,
                         layers=layers, schedule=tuple(RunEntry(i, i) for i in range(3)),
                         final_norm=norm, tie_embeddings=True, max_positions=512,
                         embed_name="tok.table", final_norm_prefix="ln_out.", head_name="out.table")


TOY_ATTN_NAMES = AttentionNames(q="att.wq", k="att.wk", v="att.wv", o="att.wo", q_norm="att.q_scale", k_norm="att.k_scale")
TOY_MLP_NAMES = GatedMLPNames(gate="ff.w_gate", up="ff.w_up", down="ff.w_down")


def _as_plain_names(w, p):
    """The toy layer's attention and feed-forward tensors under the names the plain functions look up."""
    out = dict(w)
    for theirs, ours in ((ATTENTION_NAMES, TOY_ATTN_NAMES), (MLP_NAMES, TOY_MLP_NAMES)):
        for f in theirs.__dataclass_fields__:
            if p + getattr(ours, f) in w:
                out[p + getattr(theirs, f)] = w[p + getattr(ours, f)]
    return out


def _toy_plain(w, ids, cfg: ToyConfig):
    ids = torch.as_tensor(ids)
    T = ids.numel()
    h = w["tok.table"][ids]
    acfg = dict(num_attention_heads=3, num_key_value_heads=1, head_dim=16, hidden_size=cfg.hidden_size,
                rms_norm_eps=1e-5, rope_theta=1e4)
    for i in range(3):
        p = f"blk{i}."
        x = plain.rmsnorm(h, w[p + "ln_a.scale"], 1e-5)
        if i == 1:
            a, _ = plain.attention_block(x, _as_plain_names(w, p), p, acfg, torch.arange(T), None)
        else:
            s, rows = torch.zeros(cfg.hidden_size, dtype=F64), []
            for t in range(T):
                s = cfg.decay * s + x[t]
                rows.append(s @ w[p + "toy.weight"].T)
            a = torch.stack(rows)
        h = h + a
        h = h + plain.mlp_block(plain.rmsnorm(h, w[p + "ln_b.scale"], 1e-5), _as_plain_names(w, p), p)
    return plain.rmsnorm(h, w["ln_out.scale"], 1e-5) @ w["tok.table"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_its_own_state_is_registered_built_and_stepped(tmp_path, dtype):
    import json
    import idempotent_llm_b200 as idm
    from idempotent_llm_b200.weights import write_safetensors
    MIXERS.register("toy_decay", ToyDecayMixer)
    idm.register_architecture("ToyForCausalLM", ToyConfig)
    cfg = ToyConfig()
    spec = cfg.to_model_spec()
    w = random_weights(declare_weights(spec), 7, 0.2, dtype=torch.bfloat16)
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["ToyForCausalLM"], "vocab_size": 97,
                                                      "hidden_size": 48, "decay": 0.75}))
    write_safetensors(str(tmp_path / "model.safetensors"), list(w.items()))
    lm = idm.load(str(tmp_path), dtype=dtype, max_tokens=64 * 6, max_seqs=3)       # through the registry
    eng = lm.engine
    assert set(eng.cache.state) == {0, 2} and len(eng.cache.groups) == 1
    w64 = _w64(w)
    reqs = [helpers.rand_ids(n, 97, 8 + n) for n in (9, 30, 4)]
    refs = [_toy_plain(w64, r, cfg) for r in reqs]
    tol = helpers.TOL[dtype]
    # whole
    for r, ref in zip(reqs, refs):
        s = eng.open()
        assert helpers.rel_err(eng.step([(s, r)], [list(range(len(r)))]), ref) < tol
        eng.close(s)
    # a batch of unequal lengths, then one token each; slots (and their state) are used again
    for _ in range(2):
        slots = [eng.open() for _ in reqs]
        cut = [len(r) - 3 for r in reqs]
        lg = eng.step([(s, r[:c]) for s, r, c in zip(slots, reqs, cut)], [list(range(c)) for c in cut])
        assert helpers.rel_err(lg, torch.cat([ref[:c] for ref, c in zip(refs, cut)])) < tol
        for k in range(3):
            lg = eng.step([(s, [r[c + k]]) for s, r, c in zip(slots, reqs, cut)])
            assert helpers.rel_err(lg, torch.stack([ref[c + k] for ref, c in zip(refs, cut)])) < tol
        for s in slots:
            eng.close(s)
    toks, _ = lm.generate(reqs, 4)
    assert toks.shape == (3, 4) and int(toks.min()) >= 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_steps_advance_a_mixer_s_state_once(tmp_path, dtype):
    """Single-token steps of a model whose mixer keeps per-sequence state, captured in graphs (the first such
    step of a batch size also warms up and captures) and launched one by one: the same bits, and both right.
    Also through the device-side decode loop."""
    import json
    import idempotent_llm_b200 as idm
    from idempotent_llm_b200.weights import write_safetensors
    MIXERS.register("toy_decay", ToyDecayMixerOnDevice)
    try:
        idm.register_architecture("ToyForCausalLM", ToyConfig)
        cfg = ToyConfig()
        w = random_weights(declare_weights(cfg.to_model_spec()), 7, 0.2, dtype=torch.bfloat16)
        (tmp_path / "config.json").write_text(json.dumps({"architectures": ["ToyForCausalLM"], "vocab_size": 97,
                                                          "hidden_size": 48, "decay": 0.75}))
        write_safetensors(str(tmp_path / "model.safetensors"), list(w.items()))
        reqs = [helpers.rand_ids(n, 97, 40 + n) for n in (9, 30, 7)]
        refs = [_toy_plain(_w64(w), r, cfg) for r in reqs]
        outs = {}
        for graph in (True, False):
            lm = idm.load(str(tmp_path), dtype=dtype, max_tokens=64 * 6, max_seqs=3, use_graph=graph)
            eng = lm.engine
            assert lm.model.graph_safe
            slots = [eng.open() for _ in reqs]
            cut = [len(r) - 5 for r in reqs]
            eng.step([(s_, r[:c]) for s_, r, c in zip(slots, reqs, cut)])
            got = []
            for k in range(5):
                got.append(eng.step([(s_, [r[c + k]]) for s_, r, c in zip(slots, reqs, cut)]).clone())
                ref = torch.stack([ref_[c + k] for ref_, c in zip(refs, cut)])
                assert helpers.rel_err(got[-1], ref) < helpers.TOL[dtype], f"graph={graph}: single-token step {k}"
            outs[graph] = torch.stack(got)
            # the device-side loop from here: its first step also warms up and captures
            first = [int(t) for t in got[-1].argmax(-1)]
            state_before = {cid: st.clone() for cid, st in eng.cache.state.items()}
            sess = eng.decode_session(slots, first, 3)
            for cid, st in eng.cache.state.items():
                assert torch.equal(st, state_before[cid]), "opening the session moved the state on"
            sess.run(3)
            chosen = sess.tokens()
            sess.finish()
            for i, r in enumerate(reqs):
                seq = list(r)
                for k in range(3):
                    seq.append(first[i] if k == 0 else int(chosen[k - 1, i]))
                    lgt = _toy_plain(_w64(w), seq, cfg)[-1]
                    assert float(lgt.max() - lgt[int(chosen[k, i])]) <= helpers.TOL[dtype] * float(lgt.abs().max())
            for s_ in slots:
                eng.close(s_)
        assert torch.equal(outs[True], outs[False]), "captured and plain single-token steps differ"
    finally:
        MIXERS.register("toy_decay", ToyDecayMixer)


# ------------------------------------- a toy feed-forward with routing and a toy position encoding
@dataclass(frozen=True)
class ToyRoutedSpec:
    hidden: int
    n_experts: int
    kind: str = "toy_routed"


class ToyRoutedFeedForward(FeedForward):
    """Each token goes to the expert with the largest router probability; output = p_top * (W_expert . x).
    Router logits, softmax and the product in 32-bit; plain torch on the device without a host
    synchronisation, so single-token steps with this part still run as captured graphs."""

    @classmethod
    def declare(cls, spec, prefix):
        return [TensorDecl(prefix + "router.weight", (spec.n_experts, spec.hidden)),
                TensorDecl(prefix + "experts.weight", (spec.n_experts, spec.hidden, spec.hidden))]

    def __init__(self, spec, weights, prefix, rt):
        self.router = weights[prefix + "router.weight"].float()
        self.experts = weights[prefix + "experts.weight"].float()

    def forward(self, x, ctx):
        x = x.float()
        p = torch.softmax(x @ self.router.T * 4.0, dim=-1)
        top = p.argmax(dim=-1)
        y = torch.bmm(self.experts[top], x.unsqueeze(-1)).squeeze(-1) * p.gather(-1, top[:, None])
        return y.unsqueeze(0)


@dataclass(frozen=True)
class ToyScaledRotarySpec:
    theta: float
    dim: int
    factor: float
    variant: str = "half_whole_head"       # (the table the attention kernels rotate with: pairs half a head apart)
    kind: str = "toy_scaled_rotary"


class ToyScaledRotary(PositionEncoding):
    """Rotation by position / factor: another position encoding behind the same ``tables(ctx)``."""

    def __init__(self, spec, weights, prefix, rt):
        j = torch.arange(0, spec.dim // 2, dtype=torch.float64)
        self.spec, self.rt = spec, rt
        self.inv_freq = (float(spec.theta) ** (-2.0 * j / spec.dim) / spec.factor).to(rt.device)

    def tables(self, ctx):
        key = ("toy_scaled_rotary", self.spec)
        if key not in ctx.memo:
            ctx.memo[key] = self.rt.kernels.rope_table(ctx.positions, self.inv_freq)
        return ctx.memo[key]


@dataclass(frozen=True)
class ToyRoutedConfig:
    vocab_size: int = 83
    hidden_size: int = 40
    n_experts: int = 3
    factor: float = 4.0

    @classmethod
    def from_dict(cls, d):
        return cls(**{k: d[k] for k in ("vocab_size", "hidden_size", "n_experts", "factor") if k in d})

    def to_model_spec(self):
        norm = NormSpec(self.hidden_size, 1e-5)
        attn = lambda pos: AttentionSpec(hidden=self.hidden_size, n_heads=2, n_kv_heads=2, head_dim=16, softmax_scale=0.25,
                                         qk_norm=True, qk_norm_eps=1e-5, position=pos, names=ATTENTION_NAMES)
        pre = dict(mixer_norm_prefix="input_layernorm.", feed_forward_norm_prefix="post_attention_layernorm.")
        layers = (LayerSpec("model.layers.0.", attn(ToyScaledRotarySpec(1e4, 16, self.factor)),
                            ToyRoutedSpec(self.hidden_size, self.n_experts), norm, norm, **pre),
                  LayerSpec("model.layers.1.", attn(RotarySpec(1e4, 16, 512)),
                            GatedMLPSpec(self.hidden_size, 56, names=MLP_NAMES), norm, norm, **pre))
        return ModelSpec(architecture="ToyRoutedForCausalLM", vocab_size=self.vocab_size, hidden=self.hidden_size,
                         layers=layers, schedule=tuple(RunEntry(i, i) for i in range(2)),
                         final_norm=norm, tie_embeddings=True, max_positions=512,
                         embed_name="model.embed_tokens.weight", final_norm_prefix="model.norm.", head_name="lm_head.weight")


def _toy_routed_plain(w, ids, cfg: ToyRoutedConfig):
    """Returns the logits and the smallest gap between the two largest router probabilities."""
    ids = torch.as_tensor(ids)
    T = ids.numel()
    h = w["model.embed_tokens.weight"][ids]
    acfg = dict(num_attention_heads=2, num_key_value_heads=2, head_dim=16, hidden_size=cfg.hidden_size,
                rms_norm_eps=1e-5, rope_theta=1e4)
    gap = 1.0
    for i in range(2):
        p = f"model.layers.{i}."
        x = plain.rmsnorm(h, w[p + "input_layernorm.weight"], 1e-5)
        pos = torch.arange(T, dtype=F64) / (cfg.factor if i == 0 else 1.0)
        a, _ = plain.attention_block(x, w, p, acfg, pos, None)
        h = h + a
        x = plain.rmsnorm(h, w[p + "post_attention_layernorm.weight"], 1e-5)
        if i == 0:
            pr = torch.softmax(x @ w[p + "router.weight"].T * 4.0, dim=-1)
            two = pr.topk(2, dim=-1).values
            gap = min(gap, float((two[:, 0] - two[:, 1]).min()))
            top = pr.argmax(-1)
            h = h + torch.stack([w[p + "experts.weight"][top[t]] @ x[t] * pr[t, top[t]] for t in range(T)])
        else:
            h = h + plain.mlp_block(x, w, p)
    return plain.rmsnorm(h, w["model.norm.weight"], 1e-5) @ w["model.embed_tokens.weight"].T, gap


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_feed_forward_with_routing_and_toy_position_encoding(tmp_path, dtype):
    """A feed-forward that routes and a position encoding of another kind, both defined here, are
    registered, loaded through the registry and stepped (prompts, unequal batches, single tokens in
    captured graphs) against a plain computation -- with no change to the library's files."""
    import json
    import idempotent_llm_b200 as idm
    from idempotent_llm_b200.weights import write_safetensors
    FEED_FORWARDS.register("toy_routed", ToyRoutedFeedForward)
    POSITIONS.register("toy_scaled_rotary", ToyScaledRotary)
    idm.register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig)
    cfg = ToyRoutedConfig()
    spec = cfg.to_model_spec()
    reqs = [helpers.rand_ids(n, cfg.vocab_size, 40 + n) for n in (11, 37, 5)]
    # weights whose routing is decisive for these requests: a token near a tie could go to another
    # expert in reduced precision, which is no fault of the engine
    for seed in range(40):
        w = random_weights(declare_weights(spec), seed, 0.2, dtype=torch.bfloat16)
        w64 = _w64(w)
        refs, gaps = zip(*[_toy_routed_plain(w64, r, cfg) for r in reqs])
        if min(gaps) > 0.08:
            break
    else:
        pytest.fail("no seed gives decisive routing")
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["ToyRoutedForCausalLM"], "vocab_size": cfg.vocab_size,
                                                      "hidden_size": cfg.hidden_size}))
    write_safetensors(str(tmp_path / "model.safetensors"), list(w.items()))
    lm = idm.load(str(tmp_path), dtype=dtype, max_tokens=64 * 6, max_seqs=3)
    eng = lm.engine
    assert lm.model.graph_safe, "nothing in this model synchronises with the host"
    tol = helpers.TOL[dtype]
    for r, ref in zip(reqs, refs):
        s = eng.open()
        assert helpers.rel_err(eng.step([(s, r)], [list(range(len(r)))]), ref) < tol
        eng.close(s)
    for _ in range(2):
        slots = [eng.open() for _ in reqs]
        cut = [len(r) - 3 for r in reqs]
        lg = eng.step([(s, r[:c]) for s, r, c in zip(slots, reqs, cut)], [list(range(c)) for c in cut])
        assert helpers.rel_err(lg, torch.cat([ref[:c] for ref, c in zip(refs, cut)])) < tol
        for k in range(3):
            lg = eng.step([(s, [r[c + k]]) for s, r, c in zip(slots, reqs, cut)])
            assert helpers.rel_err(lg, torch.stack([ref[c + k] for ref, c in zip(refs, cut)])) < tol
        for s in slots:
            eng.close(s)
    assert eng._graphs, "the single-token steps ran as captured graphs"
