"""The entry point that allocates nothing (csrc/idm_no_alloc.h), called through its exported C
symbol the way a host without torch's allocator would call it: the caller passes inputs and
outputs only, the scratch between the two kernels lives inside the library.  Its output must
equal the usual entry point's, on calls in a row (a later call finds an earlier call's
leftovers in the shared array), also after a call that was refused.  This file sorts last so that a run that stops at the first
failure has already run every other test."""

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(dtype, n_q, n_kv, hd, lens, seed, window=None):
    from idempotent_llm_b200.cache import CacheNeed, SequenceCache
    from idempotent_llm_b200.kernels import Kernels
    K = Kernels(dtype, "cuda:0")
    need = CacheNeed("window", n_kv, hd, window=window) if window else CacheNeed("full", n_kv, hd)
    cache = SequenceCache({0: need}, 64 * 64, dtype, "cuda:0", max_seqs=len(lens))
    g = torch.Generator(device="cuda").manual_seed(seed)
    for grp in cache.groups:
        grp.k.copy_(torch.randn(grp.k.shape, generator=g, device="cuda").to(dtype))
        grp.v.copy_(torch.randn(grp.v.shape, generator=g, device="cuda").to(dtype))
    slots = [cache.alloc_slot() for _ in lens]
    cache.reserve(list(zip(slots, lens)))
    cache.flush()
    q = torch.randn((len(lens), n_q, hd), generator=g, device="cuda").to(dtype)
    return K, cache.view(0), torch.tensor(slots, dtype=torch.int32, device="cuda"), \
        torch.tensor(lens, dtype=torch.int32, device="cuda"), q


@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_entry_point_matches_the_usual_one_twice(dtype, window):
    n_q, n_kv, hd, lens = 8, 2, 64, [700, 64, 1, 300, 257]
    K, kv, slots, kv_len, q = _setup(dtype, n_q, n_kv, hd, lens, seed=3, window=window)
    scale, max_len = 1.0 / math.sqrt(hd), 1024
    fn = K.lib.idm_attention_decode_static
    fn.restype = c_int
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)

    def static_call(qq):
        out = torch.empty((len(lens), n_q * hd), dtype=dtype, device="cuda")
        rc = fn(c_void_p(qq.data_ptr()), c_void_p(out.data_ptr()), c_void_p(kv.k.data_ptr()),
                c_void_p(kv.v.data_ptr()), c_void_p(kv.table.data_ptr()), c_int(kv.table.shape[1]), c_int(kv.ring),
                c_void_p(slots.data_ptr()), c_void_p(kv_len.data_ptr()), c_int(len(lens)), c_int(n_q),
                c_int(n_kv), c_int(hd), c_int(max_len_now[0]), c_float(scale), c_int(window or 0), stream)
        assert rc == 0, K.lib.idm_last_error().decode()
        return out

    max_len_now = [max_len]
    for call in range(3):
        qq = q if call == 0 else (q * 1.5 + 0.25).to(dtype)      # other inputs: stale partials would show
        if call == 1:
            # a wrong call in between: max_kv_len below the longest sequence.  Its answer for that sequence is
            # cut short; what matters is that it leaves the arrival counters at zero for the call after it
            max_len_now[0] = 256
            static_call(qq)
            max_len_now[0] = max_len
            continue
        want = K.attention_decode(qq, kv, slots, kv_len, max_len, scale, window or 0)
        got = static_call(qq)
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        # the same kernels in the same order on the same inputs: the same bits
        assert torch.equal(got, want), f"call {call}: max diff {float((got.float() - want.float()).abs().max())}"


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from idempotent_llm_b200.kernels import Kernels
    K = Kernels(torch.bfloat16, "cuda:0")
    fn = K.lib.idm_attention_decode_static
    fn.restype = c_int
    z = c_void_p(0)
    # 64 sequences x 64 heads x 160 chunks x 130 floats is far beyond the built-in 4 Mi floats
    rc = fn(z, z, z, z, z, c_int(1), c_int(0), z, z, c_int(64), c_int(64), c_int(8), c_int(128), c_int(40960),
            c_float(0.1), c_int(0), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0
    msg = K.lib.idm_last_error().decode()
    assert "floats of scratch" in msg and "holds" in msg
