"""Each kernel alone against a plain 64-bit PyTorch restatement of its formula, at sizes other
than the tiny models' (GPU).  Attention inputs are built so that faults show: one far key is
made to stand out, keys outside the allowed range carry NaN."""

import math

import pytest
import torch

import helpers
from idempotent_llm_b200.cache import CacheNeed, SequenceCache
from idempotent_llm_b200.engine.batch import context_from_packed, pack_step_host

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# one rounding to the storage dtype plus 32-bit arithmetic
KTOL = {"float32": 3e-6, "bfloat16": 6e-3}


@pytest.fixture(scope="module")
def kernels():
    from idempotent_llm_b200.kernels import Kernels
    made = {}

    def get(dtype):
        if dtype not in made:
            made[dtype] = Kernels(DT[dtype], "cuda:0")
        return made[dtype]
    return get


def _randn(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(kernels, dtype):
    K = kernels(dtype)
    table = _randn(1003, 72, seed=1).to(DT[dtype]).cuda()
    ids = torch.tensor([0, 1002, 5, 5, 77], dtype=torch.int32).cuda()
    h = K.embed(ids, table)
    assert h.dtype == torch.float32 and torch.equal(h, table[ids.long()].float())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,eps", [(72, 1e-5), (1024, 1e-6), (5120, 1e-6), (13, 0.1)])
def test_add_rmsnorm(kernels, dtype, hidden, eps):
    K = kernels(dtype)
    n = 37
    h0, gamma = _randn(n, hidden, seed=2, scale=3.0).float(), (1 + _randn(hidden, seed=3, scale=0.2)).float()
    delta = _randn(3, n, hidden, seed=4).float()

    def ref(v):
        v = v.double()
        return v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps) * gamma.double()
    h = h0.clone().cuda()
    x = K.add_rmsnorm(h, None, gamma.cuda(), eps)
    assert torch.equal(h.cpu(), h0) and helpers.rel_err(x, ref(h0)) < KTOL[dtype]
    x = K.add_rmsnorm(h, delta.cuda(), gamma.cuda(), eps)
    summed = ((h0 + delta[0]) + delta[1]) + delta[2]
    assert torch.equal(h.cpu(), summed), "the residual sum is 32-bit, partials added in ascending order"
    assert helpers.rel_err(x, ref(summed)) < KTOL[dtype]
    rows = torch.tensor([36, 0, 7], dtype=torch.int32).cuda()
    h2 = h0.clone().cuda()
    xr = K.add_rmsnorm(h2, delta.cuda(), gamma.cuda(), eps, rows=rows)
    assert torch.equal(h2.cpu(), h0), "selected rows leave the stream untouched"
    assert torch.equal(xr, x[rows.long()])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [1024, 72, 520])
def test_rmsnorm_of_many_rows_has_the_bits_of_few_rows(kernels, dtype, hidden):
    """From 64 rows on a warp norms a row by itself; a row's result must not depend on how many rows there are."""
    K = kernels(dtype)
    n = 203
    h = _randn(n, hidden, seed=5, scale=3.0).float().cuda()
    h[::7] *= 100.0
    gamma = (1 + _randn(hidden, seed=6, scale=0.2)).float().cuda()
    many = K.add_rmsnorm(h, None, gamma, 1e-6)
    few = torch.cat([K.add_rmsnorm(h[i:i + 29].contiguous(), None, gamma, 1e-6) for i in range(0, n, 29)])
    assert torch.equal(many, few)
    v = h.double().cpu()
    assert helpers.rel_err(many, v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.double().cpu()) < KTOL[dtype]
    rows = torch.arange(n - 1, -1, -1, dtype=torch.int32).cuda()
    assert torch.equal(K.add_rmsnorm(h, None, gamma, 1e-6, rows=rows), many.flip(0))


def test_rope_table(kernels):
    K = kernels("float32")
    pos = torch.tensor([0, 1, 63, 4095, 40959], dtype=torch.int32)
    j = torch.arange(0, 64, dtype=torch.float64)
    inv = 1e6 ** (-2.0 * j / 128)
    cs = K.rope_table(pos.cuda(), inv.cuda()).cpu()
    ang = pos.double()[:, None] * inv[None, :]
    assert (cs[..., 0].double() - torch.cos(ang)).abs().max() < 1e-7       # 32-bit rounding of an exact value
    assert (cs[..., 1].double() - torch.sin(ang)).abs().max() < 1e-7
    # from 257 positions on the table also comes by dim, the same values
    many = torch.arange(1000, 1300, dtype=torch.int32).cuda()
    cs = K.rope_table(many, inv.cuda())
    assert cs.by_dim is not None and tuple(cs.by_dim.shape) == (64, 300, 2)
    assert torch.equal(cs.by_dim.permute(1, 0, 2), cs)


def _cache_with(K, dtype, n_kv, hd, window, lens, seed, max_tokens=64 * 64):
    """A one-entry cache whose slots hold random keys/values for positions < lens[i]; returns
    (cache, slots, k_ref, v_ref) with references [len, n_kv, hd] per sequence in 64-bit."""
    need = CacheNeed("window" if window else "full", n_kv, hd, window=window)
    cache = SequenceCache({0: need}, max_tokens, DT[dtype], "cuda:0", max_seqs=len(lens) + 2)
    # poison: nothing outside the allowed keys may be read
    for g in cache.groups:
        g.k.fill_(float("nan")); g.v.fill_(float("nan"))
    cache.alloc_slot()                                   # shift slot numbers away from 0
    slots, ks, vs = [], [], []
    kv = cache.view(0)
    for i, L in enumerate(lens):
        s = cache.alloc_slot()
        cache.reserve([(s, L)]); cache.set_length(s, L); cache.flush()
        k = _randn(L, n_kv, hd, seed=seed + 2 * i).to(DT[dtype])
        v = _randn(L, n_kv, hd, seed=seed + 2 * i + 1).to(DT[dtype])
        for j in range(max(0, L - kv.ring) if kv.ring else 0, L):
            r = j % kv.ring if kv.ring else j
            page = int(kv.table[s, r // 64])
            kv.k[page, :, r % 64] = k[j].cuda(); kv.v[page, :, r % 64] = v[j].cuda()
        slots.append(s); ks.append(k.double()); vs.append(v.double())
    return cache, slots, ks, vs


def _attn_ref(q, k, v, scale, window, pos):
    """q [n_q, hd] at position pos against k, v [len, n_kv, hd]."""
    n_q, n_kv = q.shape[0], k.shape[1]
    lo = max(0, pos - window + 1) if window else 0
    out = torch.zeros_like(q)
    for h in range(n_q):
        s = (k[lo:pos + 1, h // (n_q // n_kv)] @ q[h]) * scale
        out[h] = torch.softmax(s, 0) @ v[lo:pos + 1, h // (n_q // n_kv)]
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_q,n_kv,hd,window", [(8, 2, 64, None), (6, 6, 128, None), (12, 4, 32, 100),
                                                (16, 2, 128, None), (3, 1, 256, None), (4, 2, 16, 70),
                                                (16, 8, 128, None), (8, 2, 128, None), (4, 2, 64, 300)])
def test_attention_decode_against_plain_and_general_kernel(kernels, dtype, n_q, n_kv, hd, window):
    K = kernels(dtype)
    if not K.lib.idm_attention_decode_supports(hd):
        pytest.skip("no decode kernel for this head size in this dtype; the general kernel serves it")
    lens = [1, 64, 65, 255, 256, 257, 700, 1030]
    cache, slots, ks, vs = _cache_with(K, dtype, n_kv, hd, window, lens, seed=5)
    kv = cache.view(0)
    scale = 1.0 / math.sqrt(hd)
    q = _randn(len(lens), n_q, hd, seed=9)
    far = {6: 3, 7: 300}                                  # sequence -> a far key that must dominate
    for i, j in far.items():
        if not window:
            ks_i = ks[i]
            q[i, 1] = ks_i[j, 1 // (n_q // n_kv)] * 4.0
    qd = q.to(DT[dtype]).cuda()
    packed, n, q_lens = pack_step_host(slots, [L - 1 for L in lens], [[0]] * len(lens))
    ctx = context_from_packed(packed.cuda(), n, slots, q_lens, [L - 1 for L in lens], max_kv_len=1100)
    out = K.attention_decode(qd, kv, ctx.slots, ctx.kv_len, 1100, scale, window or 0).view(len(lens), n_q, hd)
    gen = K.attention_generic(qd, kv, ctx, None, None, scale, window).view(len(lens), n_q, hd)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all() and torch.isfinite(gen).all(), "a key outside the allowed range was read"
    for i, L in enumerate(lens):
        ref = _attn_ref(qd[i].double().cpu(), ks[i], vs[i], scale, window, L - 1)
        assert helpers.rel_err(out[i], ref) < KTOL[dtype], f"decode kernel, length {L}"
        assert helpers.rel_err(gen[i], ref) < KTOL[dtype], f"general kernel, length {L}"
    if not window:
        got = out[7, 1].double().cpu()
        assert (got - vs[7][300, 1 // (n_q // n_kv)]).abs().max() < 0.05, "the far key did not dominate"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_q,n_kv,hd,window", [(4, 2, 48, None), (8, 2, 128, None), (6, 3, 80, 33), (2, 1, 16, 64)])
def test_attention_general_kernel_prompts_with_history_and_new_keys(kernels, dtype, n_q, n_kv, hd, window):
    K = kernels(dtype)
    # sequences with `hist` cached tokens bring `new` tokens each
    hist, new = [0, 10, 130, 64], [70, 5, 1, 140]
    lens = [h + n for h, n in zip(hist, new)]
    cache, slots, ks, vs = _cache_with(K, dtype, n_kv, hd, window, lens, seed=21)
    kv = cache.view(0)
    scale = 0.7 / math.sqrt(hd)
    q = [_randn(n, n_q, hd, seed=30 + i) for i, n in enumerate(new)]
    q[3][-1, 0] = ks[3][2, 0] * 5.0                       # the last query looks far back
    qd = torch.cat(q).to(DT[dtype]).cuda()
    packed, n, q_lens = pack_step_host(slots, hist, [[0] * m for m in new])
    ctx = context_from_packed(packed.cuda(), n, slots, q_lens, hist)
    k_new = v_new = None
    if window:
        # windowed layers read this step's keys from packed buffers: the ring may not hold them all
        k_new = torch.cat([k[h:] for k, h in zip(ks, hist)]).to(DT[dtype]).cuda()
        v_new = torch.cat([v[h:] for v, h in zip(vs, hist)]).to(DT[dtype]).cuda()
    out = K.attention_generic(qd, kv, ctx, k_new, v_new, scale, window).view(-1, n_q, hd)
    assert torch.isfinite(out).all()
    off = 0
    for i, (h, m) in enumerate(zip(hist, new)):
        for t in range(m):
            if window and h + t - window + 1 < h and h + t - window + 1 < lens[i] - kv.ring:
                continue                                  # that history has left the ring by construction
            ref = _attn_ref(qd[off + t].double().cpu(), ks[i], vs[i], scale, window, h + t)
            assert helpers.rel_err(out[off + t], ref) < KTOL[dtype], f"sequence {i} token {t}"
        off += m


@pytest.mark.parametrize("n_q,n_kv,hd", [(8, 2, 128), (4, 4, 64), (6, 1, 128), (16, 8, 128), (32, 2, 64)])
def test_attention_tensor_core_kernel(kernels, n_q, n_kv, hd):
    """Tiles of 128 rows (the q-heads of a kv-head x tokens) against pages of 64 keys: lengths straddle
    both borders, one sequence continues from cached history, unused page tails and free pages hold NaN,
    one query looks at a single far key."""
    K = kernels("bfloat16")
    hist, new = [0, 0, 70, 0, 300], [1, 128, 200, 129, 333]
    lens = [h + n for h, n in zip(hist, new)]
    cache, slots, ks, vs = _cache_with(K, "bfloat16", n_kv, hd, None, lens, seed=90)
    kv = cache.view(0)
    scale = 1.0 / math.sqrt(hd)
    q = [_randn(n, n_q, hd, seed=95 + i) for i, n in enumerate(new)]
    q[4][-1, 0] = ks[4][5, 0] * 4.0                        # the last query of the longest sequence looks at key 5
    q[2][100, n_q - 1] = ks[2][69, n_kv - 1] * 4.0         # a query looking at the last key of the history
    qd = torch.cat(q).to(torch.bfloat16).cuda()
    packed, n, q_lens = pack_step_host(slots, hist, [[0] * m for m in new])
    ctx = context_from_packed(packed.cuda(), n, slots, q_lens, hist)
    out = K.attention_tc(qd, kv, ctx, scale).view(-1, n_q, hd)
    torch.cuda.synchronize()
    assert K.attention_tc_status() == 0, "a bounded wait inside the kernel ran out"
    gen = K.attention_generic(qd, kv, ctx, None, None, scale, None).view(-1, n_q, hd)
    assert torch.isfinite(out).all(), "stale page contents leaked into the result"
    off = 0
    for i, (h, m) in enumerate(zip(hist, new)):
        for t in list(range(min(m, 3))) + list(range(max(0, m - 3), m)) + [m // 2, min(m - 1, 127), min(m - 1, 128)]:
            ref = _attn_ref(qd[off + t].double().cpu(), ks[i], vs[i], scale, None, h + t)
            assert helpers.rel_err(out[off + t], ref) < KTOL["bfloat16"], f"sequence {i} token {t} of {m}"
        off += m
    # everywhere: against the general kernel (both round p or the output to bfloat16 once)
    assert helpers.rel_err(out, gen) < 2 * KTOL["bfloat16"]
    got = out[sum(new) - 1, 0].double().cpu()
    assert (got - vs[4][5, 0]).abs().max() < 0.05, "the far key did not dominate"


@pytest.mark.parametrize("run_blocks", [8, 3, 2, 1])
@pytest.mark.parametrize("n_q,n_kv,hd", [(2, 1, 128), (3, 3, 64), (8, 2, 128), (16, 1, 64)])
def test_attention_tensor_core_runs_and_cuts(kernels, run_blocks, n_q, n_kv, hd):
    """A row's keys are worked in runs of key blocks that are folded in ascending order.  The bits of a row
    must not depend on who works the runs (one block walking them, or a block per run meeting in
    scratch), on what else the step holds, or on whether the row came with its prompt or alone as a single
    token.  Queries of the last tiles look at one key in the first run, at one in a middle run and at the last
    key before the diagonal; a second launch gives the same bits (the arrival counters are back at zero)."""
    K = kernels("bfloat16")
    hist, new = [0, 450, 0], [1300, 900, 130]
    lens = [h + n for h, n in zip(hist, new)]
    cache, slots, ks, vs = _cache_with(K, "bfloat16", n_kv, hd, None, lens, seed=130, max_tokens=64 * 64)
    kv = cache.view(0)
    scale = 1.0 / math.sqrt(hd)
    q = [_randn(n, n_q, hd, seed=140 + i) for i, n in enumerate(new)]
    planted = [(0, 1299, 0, 7), (0, 1250, n_q - 1, 700), (0, 1200, 0, 1151), (1, 899, n_q - 1, 449), (1, 600, 0, 1000)]
    for i, t, h, key in planted:
        q[i][t, h] = ks[i][key, h // (n_q // n_kv)] * 4.0
    qd = torch.cat(q).to(torch.bfloat16).cuda()
    packed, n, q_lens = pack_step_host(slots, hist, [[0] * m for m in new])
    ctx = context_from_packed(packed.cuda(), n, slots, q_lens, hist)
    old = K.attention_run_blocks
    K.attention_run_blocks = run_blocks
    try:
        out = K.attention_tc(qd, kv, ctx, scale, through_scratch=False, share=False).view(-1, n_q, hd)
        again = K.attention_tc(qd, kv, ctx, scale, through_scratch=False, share=False).view(-1, n_q, hd)
        # long tiles shared by several blocks that each walk a few runs (the default for prompts), twice
        for _ in range(2):
            shared = K.attention_tc(qd, kv, ctx, scale, through_scratch=False).view(-1, n_q, hd)
            assert torch.equal(out, shared), "a tile shared by several blocks gives other bits than one block walking it"
        assert ctx.memo[("attention_tc_tiles", K.lib.idm_attention_tc_heads_per_tile(n_q, n_kv))][5][3] > 0, "no tile was shared"

        met = K.attention_tc(qd, kv, ctx, scale, through_scratch=True).view(-1, n_q, hd)
        met2 = K.attention_tc(qd, kv, ctx, scale, through_scratch=True).view(-1, n_q, hd)
        torch.cuda.synchronize()
        assert K.attention_tc_status() == 0, "a bounded wait inside the kernel ran out"
        assert torch.equal(out, again)
        assert torch.equal(met, met2), "the fold of the runs depends on which block came last"
        assert torch.equal(out, met), "one block walking the runs and a block per run give other bits"
        gen = K.attention_generic(qd, kv, ctx, None, None, scale, None).view(-1, n_q, hd)
        assert torch.isfinite(out).all()
        assert helpers.rel_err(out, gen) < 2 * KTOL["bfloat16"]
        off = [0, new[0], new[0] + new[1]]
        for i, t, h, key in planted:
            ref = _attn_ref(qd[off[i] + t].double().cpu(), ks[i], vs[i], scale, None, hist[i] + t)
            assert helpers.rel_err(out[off[i] + t], ref) < KTOL["bfloat16"], f"sequence {i} token {t}"
            got = out[off[i] + t, h].double().cpu()
            assert (got - vs[i][key, h // (n_q // n_kv)]).abs().max() < 0.05, f"key {key} did not dominate"
        for i, m in enumerate(new):
            for t in [0, 1, 127, 128, m // 2, m - 2, m - 1]:
                ref = _attn_ref(qd[off[i] + t].double().cpu(), ks[i], vs[i], scale, None, hist[i] + t)
                assert helpers.rel_err(out[off[i] + t], ref) < KTOL["bfloat16"], f"sequence {i} token {t} of {m}"
        # other sequences, other counters in use: only the last two
        packed, n2, q_lens2 = pack_step_host(slots[1:], hist[1:], [[0] * m for m in new[1:]])
        ctx2 = context_from_packed(packed.cuda(), n2, slots[1:], q_lens2, hist[1:])
        out2 = K.attention_tc(qd[new[0]:].contiguous(), kv, ctx2, scale).view(-1, n_q, hd)
        assert torch.equal(out2, out[new[0]:]), "a tile's result depends on what else the step holds"
        # the same queries as single tokens (and as a few tokens that straddle a run's border): the same bits
        picks = [(0, 0), (0, 63), (0, 64), (0, 511), (0, 512), (0, 1299), (1, 0), (1, 61), (1, 62), (1, 899), (2, 129)]
        for i, t in picks:
            packed, n1, ql = pack_step_host([slots[i]], [hist[i] + t], [[0]])
            ctx1 = context_from_packed(packed.cuda(), n1, [slots[i]], ql, [hist[i] + t], max_kv_len=2048)
            one = K.attention_tc(qd[off[i] + t:off[i] + t + 1].contiguous(), kv, ctx1, scale).view(1, n_q, hd)
            assert torch.equal(one[0], out[off[i] + t]), f"sequence {i} token {t} alone (position {hist[i] + t})"
        for i, t, m in [(0, 500, 20), (1, 55, 12), (0, 1290, 10)]:
            packed, nm, ql = pack_step_host([slots[i]], [hist[i] + t], [[0] * m])
            ctxm = context_from_packed(packed.cuda(), nm, [slots[i]], ql, [hist[i] + t])
            for ts in (None, True, False):
                few = K.attention_tc(qd[off[i] + t:off[i] + t + m].contiguous(), kv, ctxm, scale, through_scratch=ts)
                assert torch.equal(few.view(m, n_q, hd), out[off[i] + t:off[i] + t + m]), f"sequence {i} tokens {t}..{t + m}"
        torch.cuda.synchronize()
        assert K.attention_tc_status() == 0
    finally:
        K.attention_run_blocks = old


@pytest.mark.parametrize("n_q,n_kv,hd", [(16, 8, 128), (4, 4, 64), (32, 2, 128), (12, 4, 64), (8, 1, 128)])
def test_attention_of_single_tokens_has_the_tile_kernel_s_bits(kernels, n_q, n_kv, hd):
    """Steps of single tokens have a kernel of their own (a run's key blocks side by side on mma.sync
    fragments).  It must give every row the bits of the kernel that all other steps take: lengths on
    both sides of a page's and a run's border, free pages and page tails full of NaN, one query that
    looks at a single far key and one at its own (the last) key."""
    K = kernels("bfloat16")
    lens = [1, 2, 63, 64, 65, 511, 512, 513, 1024, 1300, 3000]
    cache, slots, ks, vs = _cache_with(K, "bfloat16", n_kv, hd, None, lens, seed=400, max_tokens=64 * 160)
    kv = cache.view(0)
    scale = 1.0 / math.sqrt(hd)
    q = _randn(len(lens), n_q, hd, seed=410)
    q[10, 0] = ks[10][70, 0] * 4.0                         # the longest sequence's first head looks at key 70
    q[9, n_q - 1] = ks[9][1299, n_kv - 1] * 4.0            # a query that looks at its own position's key
    qd = q.to(torch.bfloat16).cuda()
    starts = [L - 1 for L in lens]
    packed, n, q_lens = pack_step_host(slots, starts, [[0]] * len(lens))
    ctx = context_from_packed(packed.cuda(), n, slots, q_lens, starts)
    assert K.attention_tc_few_rows(True) is True           # (the default)
    try:
        mine = K.attention_tc(qd, kv, ctx, scale).view(-1, n_q, hd)
        mine2 = K.attention_tc(qd, kv, ctx, scale).view(-1, n_q, hd)
        K.attention_tc_few_rows(False)
        tile = K.attention_tc(qd, kv, ctx, scale).view(-1, n_q, hd)
        walk = K.attention_tc(qd, kv, ctx, scale, through_scratch=False).view(-1, n_q, hd)
    finally:
        K.attention_tc_few_rows(True)
    torch.cuda.synchronize()
    assert K.attention_tc_status() == 0, "a bounded wait inside the kernel ran out"
    assert torch.isfinite(mine).all(), "stale page contents leaked into the result"
    for i in range(len(lens)):
        assert torch.equal(mine[i], tile[i]), f"length {lens[i]}: other bits than the tile kernel's"
    assert torch.equal(mine, mine2) and torch.equal(tile, walk)
    for i, L in enumerate(lens):
        ref = _attn_ref(qd[i].double().cpu(), ks[i], vs[i], scale, None, L - 1)
        assert helpers.rel_err(mine[i], ref) < KTOL["bfloat16"], f"length {L}"
    assert (mine[10, 0].double().cpu() - vs[10][70, 0]).abs().max() < 0.05, "the far key did not dominate"
    assert (mine[9, n_q - 1].double().cpu() - vs[9][1299, n_kv - 1]).abs().max() < 0.05
    # a shorter step: other blocks, other counters, the same rows
    sub = [2, 7, 10]
    packed, n3, ql3 = pack_step_host([slots[i] for i in sub], [starts[i] for i in sub], [[0]] * 3)
    ctx3 = context_from_packed(packed.cuda(), n3, [slots[i] for i in sub], ql3, [starts[i] for i in sub], max_kv_len=4096)
    part = K.attention_tc(qd[sub].contiguous(), kv, ctx3, scale).view(-1, n_q, hd)
    assert torch.equal(part, mine[sub]), "a row's result depends on what else the step holds"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_qkv_finish_norm_rotation_and_cache_write(kernels, dtype):
    K = kernels(dtype)
    n_q, n_kv, hd, eps, theta = 6, 2, 48, 1e-5, 5e4
    lens, starts = [3, 70], [5, 64]
    need = CacheNeed("full", n_kv, hd)
    cache = SequenceCache({0: need}, 64 * 8, DT[dtype], "cuda:0", max_seqs=4)
    slots = [cache.alloc_slot() for _ in lens]
    cache.reserve([(s, st + L) for s, st, L in zip(slots, starts, lens)]); cache.flush()
    packed, n, q_lens = pack_step_host(slots, starts, [[0] * L for L in lens])
    ctx = context_from_packed(packed.cuda(), n, slots, q_lens, starts)
    width = (n_q + 2 * n_kv) * hd
    parts = _randn(2, n, width, seed=40).float()
    gq, gk = (1 + _randn(hd, seed=41, scale=0.3)).float(), (1 + _randn(hd, seed=42, scale=0.3)).float()
    inv = theta ** (-2.0 * torch.arange(0, hd // 2, dtype=torch.float64) / hd)
    cs = K.rope_table(ctx.positions, inv.cuda())
    kv = cache.view(0)
    q, k_new, v_new = K.qkv_finish(parts.cuda(), n_q, n_kv, hd, gq.cuda(), gk.cuda(), eps, cs, ctx, kv, keep_new=True)
    x = (parts[0] + parts[1]).double().view(n, n_q + 2 * n_kv, hd)
    pos = ctx.positions.cpu().double()
    ang = torch.cat([pos[:, None] * inv[None, :]] * 2, -1)
    cos, sin = torch.cos(ang).float().double()[:, None, :], torch.sin(ang).float().double()[:, None, :]

    def fin(t, g):
        t = t / torch.sqrt(t.pow(2).mean(-1, keepdim=True) + eps) * g.double()
        return t * cos + torch.cat([-t[..., hd // 2:], t[..., :hd // 2]], -1) * sin
    assert helpers.rel_err(q, fin(x[:, :n_q], gq)) < KTOL[dtype]
    assert helpers.rel_err(k_new, fin(x[:, n_q:n_q + n_kv], gk)) < KTOL[dtype]
    assert helpers.rel_err(v_new, x[:, n_q + n_kv:]) < KTOL[dtype]
    t = 0
    for s, st, L in zip(slots, starts, lens):
        for j in range(st, st + L):
            page = int(kv.table[s, j // 64])
            assert torch.equal(kv.k[page, :, j % 64], k_new[t]) and torch.equal(kv.v[page, :, j % 64], v_new[t])
            t += 1
    # without norm weights and without a table the heads pass through
    q2, _, _ = K.qkv_finish(parts.cuda(), n_q, n_kv, hd, None, None, eps, None, ctx, None, keep_new=False)
    assert helpers.rel_err(q2, x[:, :n_q]) < KTOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_ring_write_keeps_the_last_ring_tokens(kernels, dtype):
    K = kernels(dtype)
    n_kv, hd, window = 2, 16, 70                          # ring of 128
    cache = SequenceCache({0: CacheNeed("window", n_kv, hd, window=window)}, 64 * 8, DT[dtype], "cuda:0", max_seqs=3)
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    starts, lens = [0, 100], [300, 40]
    cache.reserve([(s, st + L) for s, st, L in zip(slots, starts, lens)]); cache.flush()
    packed, n, q_lens = pack_step_host(slots, starts, [[0] * L for L in lens])
    ctx = context_from_packed(packed.cuda(), n, slots, q_lens, starts)
    k_new = _randn(n, n_kv, hd, seed=50).to(DT[dtype]).cuda()
    v_new = _randn(n, n_kv, hd, seed=51).to(DT[dtype]).cuda()
    kv = cache.view(0)
    kv.k.zero_(); kv.v.zero_()
    K.kv_write_ring(k_new, v_new, kv, ctx)
    for (s, st, L), off in zip(zip(slots, starts, lens), (0, 300)):
        for j in range(max(st, st + L - 128), st + L):
            page, r = int(kv.table[s, (j % 128) // 64]), (j % 128) % 64
            assert torch.equal(kv.k[page, :, r], k_new[off + j - st]), f"slot {s} position {j}"
            assert torch.equal(kv.v[page, :, r], v_new[off + j - st])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu(kernels, dtype):
    K = kernels(dtype)
    n, inter = 19, 1000
    gu = _randn(2, n, 2 * inter, seed=60, scale=4.0).float()
    gu[0, 0, 0], gu[1, 0, 0] = -200.0, 0.0                # a saturated gate stays finite
    y = K.swiglu(gu.cuda())
    x = (gu[0] + gu[1]).double()
    g, u = x[:, :inter], x[:, inter:]
    assert torch.isfinite(y).all() and helpers.rel_err(y, g * torch.sigmoid(g) * u) < KTOL[dtype]


@pytest.mark.parametrize("M,N,K_", [(1, 320, 96), (7, 1000, 160), (130, 257, 224), (64, 64, 16), (3, 5, 7)])
def test_gemm_32_bit_is_true_32_bit_and_row_independent(kernels, M, N, K_):
    K = kernels("float32")
    x, w = _randn(M, K_, seed=70).float(), _randn(N, K_, seed=71).float()
    out = K.gemm(x.cuda(), w.cuda())
    assert out.shape == (1, M, N)
    ref = x.double() @ w.double().T
    # TF32 would give ~1e-3; true 32-bit FMA chains of K_ terms give ~1e-6
    assert helpers.rel_err(out[0], ref) < 2e-6
    one = K.gemm(x[M // 2:M // 2 + 1].contiguous().cuda(), w.cuda())
    assert torch.equal(one[0, 0], out[0, M // 2]), "a row's result must not depend on the other rows"


# Token counts on both sides of every border between kernels and tile shapes (16, 32, 64, 128 tokens on
# the lanes of one kernel; 128- and 256-token tiles of another above that).
CUTS = (1, 2, 16, 17, 32, 33, 64, 65, 128, 129, 200, 256, 257, 300)


@pytest.mark.parametrize("M,N,K_", [(1, 320, 96), (8, 1000, 160), (200, 512, 1024), (17, 130, 72), (64, 1024, 3072),
                                    (33, 257, 2048), (300, 384, 136), (1, 151936, 64), (2048, 1024, 1024),
                                    (130, 4096, 4096), (200, 1024, 12288), (256, 5120, 5120), (96, 40, 8), (100, 20000, 128),
                                    (3000, 1024, 256), (5000, 2048, 192)])   # (the last two: several tiles per block)
def test_gemm_bfloat16(kernels, M, N, K_):
    K = kernels("bfloat16")
    x, w = _randn(M, K_, seed=72).bfloat16(), _randn(N, K_, seed=73).bfloat16()
    xd, wd = x.cuda(), w.cuda()
    out = K.gemm(xd, wd)
    torch.cuda.synchronize()
    assert K.gemm_status() == 0, "a bounded wait inside the kernel ran out"
    assert out.dtype == torch.float32 and out.shape == (1, M, N)
    ref = x.double() @ w.double().T
    # products of bfloat16 values are exact in 32-bit; only the accumulation rounds
    assert helpers.rel_err(out[0], ref) < 2e-5
    # a token's product is the same bits whatever else is in the step and however many tokens it has
    for m in CUTS:
        if m < M:
            assert torch.equal(K.gemm_store(xd[:m].contiguous(), wd), out[0, :m]), f"the first {m} of {M} tokens alone"
    mid = K.gemm_store(xd[M // 2:M // 2 + 1].contiguous(), wd)
    assert torch.equal(mid[0], out[0, M // 2]), "a row alone"


def test_a_product_element_is_one_chain_whatever_the_instruction(kernels):
    """What the kernels rest on, asked of the hardware: an element of a tcgen05 product has the same
    bits for every shape of the instruction, whatever its neighbours hold, and whichever operand
    carries the tokens; a sum of partial chains does not have them."""
    K = kernels("bfloat16")
    Kd = 3072
    x = (_randn(600, Kd, seed=170)).bfloat16().cuda()
    w = (_randn(520, Kd, seed=171, scale=0.05)).bfloat16().cuda()
    full = K.gemm_store(x, w)                                  # 600 tokens: 128 features on the lanes, 128/256 tokens a tile
    # neighbours: other rows of the operand replaced
    x2 = x[:16].clone()
    x2[4:] = 7.0
    assert torch.equal(K.gemm_store(x2, w)[3], full[3])
    # roles exchanged: (w . x^T)^T
    for a, b in ((x[:512], w[:512]), (x[:8], w[:512]), (x[:300], w[:40])):
        a, b = a.contiguous(), b.contiguous()
        assert torch.equal(K.gemm_store(a, b), K.gemm_store(b, a).T.contiguous())
    # two half chains added differ from the one chain somewhere (else splitting the inner axis would be free)
    halves = K.gemm_store(x[:64, :Kd // 2].contiguous(), w[:, :Kd // 2].contiguous()) + \
        K.gemm_store(x[:64, Kd // 2:].contiguous(), w[:, Kd // 2:].contiguous())
    assert not torch.equal(halves, full[:64]) and helpers.rel_err(halves, full[:64]) < 1e-5
    assert K.gemm_status() == 0


@pytest.mark.parametrize("M,N,K_", [(1, 320, 96), (8, 1024, 2048), (64, 1024, 3072), (200, 512, 1024), (300, 384, 136),
                                    (2048, 1024, 1024), (5, 151936, 64), (1030, 4096, 192), (700, 16000, 72),
                                    (130, 4096, 4096), (8, 131, 80),
                                    (513, 256, 512), (640, 1024, 2048)])   # (tokens on the lanes, a block per 128 tokens)
def test_gemm_fused_store_and_residual(kernels, M, N, K_):
    K = kernels("bfloat16")
    x, w = _randn(M, K_, seed=74).bfloat16(), _randn(N, K_, seed=75).bfloat16()
    ref = x.double() @ w.double().T
    for _ in range(2):
        out = K.gemm_store(x.cuda(), w.cuda())
        assert out.shape == (M, N) and helpers.rel_err(out, ref) < 2e-5
    h0 = _randn(M, N, seed=76, scale=3.0).float()
    h = h0.clone().cuda()
    K.gemm_residual(x.cuda(), w.cuda(), h)
    assert helpers.rel_err(h, h0.double() + ref) < 2e-5
    assert torch.equal(h, h0.cuda() + out), "the residual epilogue adds the product's bits to the stream once"
    for m in CUTS:
        if m < M:
            hm = h0[:m].clone().cuda()
            K.gemm_residual(x[:m].contiguous().cuda(), w.cuda(), hm)
            assert torch.equal(hm, h[:m]), f"the first {m} of {M} tokens alone"
    torch.cuda.synchronize()
    assert K.gemm_status() == 0


@pytest.mark.parametrize("M,N,K_", [(2048, 2048, 512), (1500, 4000, 200), (777, 16000, 72), (300, 1024, 2048)])
def test_every_way_to_make_a_product_of_many_tokens_gives_the_same_bits(kernels, M, N, K_):
    """One block per tile, the two blocks of a cluster on one tile (cta_group::2), the kernel with the tokens on
    the lanes taken beyond 128 tokens, and the tiles walked in bands of other widths: one chain per element in
    all of them."""
    K = kernels("bfloat16")
    x, w = _randn(M, K_, seed=84).bfloat16().cuda(), _randn(N, K_, seed=85).bfloat16().cuda()
    h0 = _randn(M, N, seed=86, scale=3.0).float().cuda()
    ways = {"single blocks": dict(pair=False, lanes_up_to_tiles=0, band_mb=32),
            "pairs of blocks": dict(pair=True, lanes_up_to_tiles=0, band_mb=32),
            "tokens on the lanes": dict(pair=False, lanes_up_to_tiles=1 << 20, band_mb=32),
            "narrow bands": dict(pair=True, lanes_up_to_tiles=0, band_mb=1)}
    got = {}
    try:
        for name, how in ways.items():
            K.gemm_choices(**how)
            h = h0.clone()
            K.gemm_residual(x, w, h)
            got[name] = (K.gemm_store(x, w), h)
    finally:
        K.gemm_choices(pair=True, lanes_up_to_tiles=64, band_mb=32)
    torch.cuda.synchronize()
    assert K.gemm_status() == 0
    ref = x.double().cpu() @ w.double().cpu().T
    assert helpers.rel_err(got["single blocks"][0], ref) < 2e-5
    for name in list(ways)[1:]:
        assert torch.equal(got[name][0], got["single blocks"][0]), name
        assert torch.equal(got[name][1], got["single blocks"][1]), name + " (added to the stream)"


@pytest.mark.parametrize("M,inter,K_", [(1, 128, 64), (8, 3072, 1024), (7, 224, 96), (130, 136, 80), (2048, 288, 160),
                                        (1030, 2000, 192), (400, 600, 256)])
def test_gemm_fused_swiglu(kernels, M, inter, K_):
    K = kernels("bfloat16")
    x = _randn(M, K_, seed=77).bfloat16()
    gate, up = _randn(inter, K_, seed=78, scale=0.3).bfloat16(), _randn(inter, K_, seed=79, scale=0.3).bfloat16()
    tiled = K.tile_gate_up(gate.cuda(), up.cuda())
    assert tiled.shape == (-(-inter // 64) * 128, K_)
    for _ in range(2):
        y = K.gemm_swiglu(x.cuda(), tiled, inter)
        g, u = x.double() @ gate.double().T, x.double() @ up.double().T
        assert y.shape == (M, inter) and helpers.rel_err(y, g * torch.sigmoid(g) * u) < KTOL["bfloat16"]
    unfused = K.swiglu(K.gemm(x.cuda(), torch.cat([gate, up]).cuda()))
    assert torch.equal(unfused, y), "fused and separate kernels apply one formula to the same products"
    for m in CUTS:
        if m < M:
            assert torch.equal(K.gemm_swiglu(x[:m].contiguous().cuda(), tiled, inter), y[:m]), f"the first {m} of {M} tokens alone"
    assert torch.equal(K.swiglu(K.gemm(x.cuda(), tiled), tiled_inter=inter), y), "the tiled layout read by the separate kernel"


@pytest.mark.parametrize("M,n_q,n_kv,hd,hidden", [(3, 6, 2, 32, 96), (9, 16, 8, 128, 1024),
                                                  (300, 8, 2, 128, 160), (64, 2, 1, 64, 72), (1030, 24, 4, 128, 192),
                                                  (520, 40, 12, 64, 136), (300, 6, 2, 32, 96), (130, 32, 8, 128, 4096),
                                                  (2500, 16, 8, 128, 256),    # (three tiles per block)
                                                  (513, 4, 2, 64, 128)])      # (tokens on the lanes, five blocks of tokens)
def test_gemm_fused_qkv_matches_the_separate_kernels(kernels, M, n_q, n_kv, hd, hidden):
    K = kernels("bfloat16")
    x_all = _randn(M, hidden, seed=80).bfloat16().cuda()
    w = _randn((n_q + 2 * n_kv) * hd, hidden, seed=81, scale=0.2).bfloat16().cuda()
    gq, gk = (1 + _randn(hd, seed=82, scale=0.3)).float().cuda(), (1 + _randn(hd, seed=83, scale=0.3)).float().cuda()
    inv = 3e4 ** (-2.0 * torch.arange(0, hd // 2, dtype=torch.float64) / hd)

    def run(fused, m=M, by_dim=True, split=True):
        """The first ``m`` tokens, as two sequences (``split``) or one, starting at positions 5 and 64."""
        starts, lens = ([5, 64], [m // 2, m - m // 2]) if split and m >= 2 else ([5], [m])
        cache = SequenceCache({0: CacheNeed("full", n_kv, hd)}, 64 * max(40, M // 64 + 6), torch.bfloat16, "cuda:0", max_seqs=4)
        slots = [cache.alloc_slot() for _ in lens]
        cache.reserve([(s_, st + L) for s_, st, L in zip(slots, starts, lens)]); cache.flush()
        packed, n, q_lens = pack_step_host(slots, starts, [[0] * L for L in lens])
        ctx = context_from_packed(packed.cuda(), n, slots, q_lens, starts)
        cs = K.rope_table(ctx.positions, inv.cuda())
        if not by_dim:
            cs.by_dim = None                               # the table by token only, as another position encoding gives it
        kv = cache.view(0)
        x = x_all[:m].contiguous()
        if fused:
            q, kn, vn = K.gemm_qkv(x, w, n_q, n_kv, hd, gq, gk, 1e-5, cs, ctx, kv, keep_new=True)
        else:
            q, kn, vn = K.qkv_finish(K.gemm(x, w), n_q, n_kv, hd, gq, gk, 1e-5, cs, ctx, kv, keep_new=True)
        torch.cuda.synchronize()
        # the cache rows of the tokens, gathered in token order
        rows_k, rows_v = [], []
        for s_, st, L in zip(slots, starts, lens):
            for pos in range(st, st + L):
                page = int(kv.table[s_, pos // 64])
                rows_k.append(kv.k[page, :, pos % 64]); rows_v.append(kv.v[page, :, pos % 64])
        return q, kn, vn, torch.stack(rows_k), torch.stack(rows_v)
    a, b = run(True), run(False)
    names = ("q", "k_new", "v_new", "cache k", "cache v")
    for t_a, t_b, name in zip(a, b, names):
        # the same numbers; a head's sum of squares is added in another order by the separate kernel
        assert helpers.rel_err(t_a, t_b) < KTOL["bfloat16"], name
    assert torch.equal(a[1], a[3]) and torch.equal(a[2], a[4]), "what goes to the cache is what goes to the packed buffers"
    # one sequence of the same tokens at positions 5 ..: the bits of a token do not depend on how many tokens the step has
    whole = run(True, split=False)
    for m in CUTS:
        if m < M:
            part = run(True, m=m, split=False)
            for t_w, t_p, name in zip(whole, part, names):
                assert torch.equal(t_w[:m], t_p), f"{name}: the first {m} of {M} tokens alone"
    if M > 128:
        for t_a, t_c, name in zip(a, run(True, by_dim=False), names):
            assert torch.equal(t_a, t_c), name + ": the table read by dim or by token gives other bits"
    assert K.gemm_status() == 0


def test_sampler_argmax_ties_and_gumbel(kernels):
    import plain_qwen3 as plain
    from idempotent_llm_b200.sampling.sampler import _as_i64, row_key
    K = kernels("float32")
    V = 151937
    lg = _randn(3, V, seed=80).float()
    lg[0, 777] = lg[0, 99999] = 50.0                      # a tie: the lower id wins
    lg[1, V - 1] = 60.0
    lg[2, 5] = float("nan")
    got = K.sample(lg.cuda(), 0.0, None).tolist()
    assert got[0] == 777 and got[1] == V - 1 and got[2] == int(torch.nan_to_num(lg[2], nan=-1e30).argmax())
    small = _randn(4, 300, seed=81).float() * 2
    keys = torch.tensor([_as_i64(row_key(3, r, 9)) for r in range(4)], dtype=torch.int64)
    got = K.sample(small.cuda(), 0.7, keys.cuda()).tolist()
    for r in range(4):
        sc = plain.gumbel_scores(small[r], 0.7, 3, r, 9)
        assert float(sc.max() - sc[got[r]]) < 1e-4        # the same draw up to 32-bit rounding of the noise
    with pytest.raises(Exception, match="keys"):
        K.sample(small.cuda(), 0.7, None)


def test_sampler_never_draws_an_infinite_score_over_a_whole_vocabulary(kernels):
    """One logit far above the rest, the real vocabulary, many rows and keys: the peak is chosen every
    time.  (A uniform number of exactly 1 gave its token the score +inf: about one draw in 110 at this
    vocabulary was a random id.)"""
    from idempotent_llm_b200.sampling.sampler import _as_i64, row_key
    K = kernels("float32")
    V, rows = 151936, 512
    lg = torch.zeros(rows, V)
    peak = torch.randint(0, V, (rows,), generator=torch.Generator().manual_seed(5))
    lg[torch.arange(rows), peak] = 200.0
    for seed in (0, 1, 2, 3):
        keys = torch.tensor([_as_i64(row_key(seed, r, 17 + seed)) for r in range(rows)], dtype=torch.int64)
        got = K.sample(lg.cuda(), 1.0, keys.cuda()).cpu()
        assert torch.equal(got.long(), peak), f"seed {seed}: rows {(got.long() != peak).nonzero().flatten().tolist()[:5]}"


def test_sizes_the_kernels_cannot_take_are_refused(kernels):
    from idempotent_llm_b200.kernels import KernelError
    K = kernels("bfloat16")
    with pytest.raises(KernelError, match="head_dim"):
        K.qkv_finish(torch.zeros(1, 1, 3 * 272, device="cuda"), 1, 1, 272, None, None, 1e-6, None,
                     type("C", (), {"token_seq": torch.zeros(1, dtype=torch.int32, device="cuda"),
                                    "positions": torch.zeros(1, dtype=torch.int32, device="cuda"),
                                    "slots": torch.zeros(1, dtype=torch.int32, device="cuda")})(), None, False)
    with pytest.raises(KernelError, match="contiguous|expected"):
        K.swiglu(torch.zeros(1, 4, 8, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(KernelError, match="rows"):
        K.gemm(torch.zeros(2, 8, device="cuda", dtype=torch.bfloat16), torch.zeros(4, 16, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(KernelError, match="multiple of 8"):
        K.gemm(torch.zeros(2, 12, device="cuda", dtype=torch.bfloat16), torch.zeros(4, 12, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(KernelError, match="head_dim"):
        K.gemm_qkv(torch.zeros(1, 64, device="cuda", dtype=torch.bfloat16), torch.zeros(48, 64, device="cuda", dtype=torch.bfloat16),
                   1, 1, 16, None, None, 1e-6, None, None, None, False)


def test_a_bounded_wait_that_runs_out_reports_and_the_kernel_ends_normally(kernels):
    """The wait every tensor-core kernel uses, on a barrier nothing arrives at, with a limit of a few
    thousand cycles: it gives up, the block's other role leaves through the abort flag, tensor memory is
    freed, the kernel returns, the status word says so once, and the device goes on working.  With an
    arrival the same kernel reports nothing."""
    K = kernels("bfloat16")
    assert K.gemm_status() == 0
    ran_out, cycles, other_left = K.wait_probe(5000)
    assert ran_out and other_left and 5000 <= cycles < 5_000_000
    assert K.gemm_status() == 1, "the run-out wait is not reported"
    assert K.gemm_status() == 0, "the report is not cleared by reading it"
    ran_out, cycles, other_left = K.wait_probe(5000, arrive=True)
    assert not ran_out and not other_left and K.gemm_status() == 0
    # the context is as usable as before
    x, w = _randn(8, 128, seed=1).bfloat16().cuda(), _randn(32, 128, seed=2).bfloat16().cuda()
    assert helpers.rel_err(K.gemm_store(x, w), x.double().cpu() @ w.double().cpu().T) < 2e-5
    with pytest.raises(Exception, match="limit"):
        K.wait_probe(0)
