"""The step program's host side without a GPU: buffers by name, what is refused, how calls are written down
(what the library does with them is covered by the GPU tests)."""
import types

import pytest
import torch

from idempotent_llm_b200.kernels import program
from idempotent_llm_b200.kernels.program import NotProgrammable, StepProgram


class _Lib:
    @staticmethod
    def idm_attention_tc_supports(hd):
        return 1 if hd in (64, 128) else 0


def _kernels(**over):
    k = types.SimpleNamespace(dtype=torch.bfloat16, fused=True, attention_impl="tcgen05", lib=_Lib(),
                              QKV_FUSED_HEAD_DIMS=(32, 64, 128), _need=lambda t, dtype, what: None,
                              _check_kv=lambda kv, n_kv, hd: None)
    for name, value in over.items():
        setattr(k, name, value)
    return k


def _kv(hd=128, n_kv=2, ring=0, window=None):
    return types.SimpleNamespace(k=torch.zeros(4, n_kv, 64, hd), v=torch.zeros(4, n_kv, 64, hd),
                                 table=torch.zeros(3, 5, dtype=torch.int32), ring=ring, window=window,
                                 n_kv_heads=n_kv, head_dim=hd)


def test_only_the_fused_bfloat16_kernels_have_programs():
    for over in (dict(dtype=torch.float32), dict(fused=False), dict(attention_impl="generic")):
        with pytest.raises(NotProgrammable):
            StepProgram(_kernels(**over))


def test_a_name_is_one_buffer_with_the_largest_need():
    p = StepProgram(_kernels())
    a = p.buffer("x", per_token=100)
    b = p.buffer("y", per_row=8)
    assert p.buffer("x", per_token=60, per_row=4) == a and a != b
    assert p._buffers["x"][1:] == [100, 4] and p._buffers["y"][1:] == [0, 8]
    for i in range(program.MAX_BUFFERS - 2):
        p.buffer(f"more{i}")
    with pytest.raises(NotProgrammable):
        p.buffer("one too many")


def test_calls_are_written_down_with_their_constant_arguments():
    p = StepProgram(_kernels())
    h, x, q, o = (p.buffer(n) for n in ("h", "x", "q", "o"))
    gamma = torch.ones(160)
    p.add_rmsnorm(h, gamma, 1e-5, x, 160, rows=True)
    w = torch.zeros((8 + 2 * 2) * 128, 160, dtype=torch.bfloat16)
    kv = _kv()
    p.gemm_qkv(x, w, 160, 8, 2, 128, torch.ones(128), None, 1e-6, (6, 7), q, kv)
    p.attention(q, kv, 8, 0.125, o)
    p.attention(q, _kv(hd=64, n_kv=4), 8, 0.25, o)
    wo = torch.zeros(160, 1024, dtype=torch.bfloat16)
    p.gemm_residual(o, wo, 1024, h)
    norm, qkv, att, att2, res = p._ops
    assert (norm.kind, list(norm.i[:4]), round(norm.f[0], 9)) == (program.ADD_RMSNORM, [160, h, x, 1], 1e-5)
    assert norm.p[0] == gamma.data_ptr()
    assert (qkv.kind, list(qkv.i[:10])) == (program.GEMM_QKV, [160, 8, 2, 128, x, q, 6, 7, 5, 0])
    assert qkv.p[0] == w.data_ptr() and qkv.p[2] is None and qkv.p[3] == kv.k.data_ptr() and qkv.p[5] == kv.table.data_ptr()
    assert (att.kind, list(att.i[:8])) == (program.ATTENTION, [4, 5, 8, 2, 128, q, o, 0])
    assert att2.i[7] == 1 and p._plans == [(8, 2, 128), (8, 4, 64)]      # a plan per arrangement of heads
    assert (res.kind, list(res.i[:4])) == (program.GEMM_RESIDUAL, [160, 1024, o, h])
    p.finish(o, 160)
    assert p.n_calls == 5
    with pytest.raises(RuntimeError):
        p.add_rmsnorm(h, gamma, 1e-5, x, 160)


def test_what_a_program_cannot_hold_is_refused_by_name():
    p = StepProgram(_kernels())
    w48 = torch.zeros(6 * 48, 96, dtype=torch.bfloat16)
    with pytest.raises(NotProgrammable, match="head size 48"):
        p.gemm_qkv(0, w48, 96, 4, 1, 48, None, None, 1e-6, None, 1, None)
    with pytest.raises(NotProgrammable, match="window"):
        p.gemm_qkv(0, torch.zeros(6 * 64, 96, dtype=torch.bfloat16), 96, 4, 1, 64, None, None, 1e-6, None, 1, _kv(hd=64, n_kv=1, ring=128))
    with pytest.raises(NotProgrammable):
        p.attention(0, _kv(hd=64, window=80), 4, 0.1, 1)
    with pytest.raises(NotProgrammable):
        p.attention(0, _kv(hd=48), 4, 0.1, 1)
    with pytest.raises(ValueError, match="multiple of 8"):
        p.gemm_residual(0, torch.zeros(64, 100, dtype=torch.bfloat16), 100, 1)
    with pytest.raises(ValueError):
        p.gemm_swiglu(0, torch.zeros(100, 64, dtype=torch.bfloat16), 64, 64, 1)       # not the tiled layout's row count
    with pytest.raises(ValueError):
        p.add_rmsnorm(0, torch.ones(7), 1e-6, 1, 8)
