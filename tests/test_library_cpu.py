"""CPU-side checks: the shared library loads, exports every symbol the header
declares, validates arguments, and the host-side operator wrappers keep the
reference's argument contract.  No kernel is launched."""
import ctypes
import os
import re

import pytest
import torch

from flash_bla import _C
from flash_bla.ops import _passes as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "flash_bla_sm100.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fbla_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _C.lib()
    names = declared_symbols()
    assert len(names) >= 21
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_C.exported_symbols()) == [n for n in names if n in _C.exported_symbols()]
    assert lib.fbla_version() == 2


def test_problem_struct_matches_header_layout():
    # 4-byte fields packed, 8-byte fields aligned: the C compiler's layout for the header's struct
    assert _C.Problem.seq_len.offset == 24 and _C.Problem.norm_len.offset == 32
    assert _C.Problem.cu_seqlens.offset == 40 and _C.Problem.num_seqs.offset == 48
    assert _C.Problem.flags.offset == 72 and ctypes.sizeof(_C.Problem) == 80


def test_sizes_and_validation_without_a_device():
    lib = _C.lib()
    like = torch.empty(0, dtype=torch.bfloat16)
    p = P.make_problem(like, batch=8, heads=16, seq_len=32768, dk=64, dv=64, normalize=True, scale=1.0)
    assert lib.fbla_state_floats(ctypes.byref(p)) == 8 * 16 * (64 * 64 + 64)
    assert lib.fbla_workspace_bytes(ctypes.byref(p)) >= 0
    p2 = P.make_problem(like, batch=4, heads=32, seq_len=262144, dk=128, dv=128, normalize=False)
    assert lib.fbla_state_floats(ctypes.byref(p2)) == 4 * 32 * 128 * 128
    bad = P.make_problem(like, batch=1, heads=1, seq_len=8, dk=129, dv=8, normalize=True)
    assert lib.fbla_state_floats(ctypes.byref(bad)) == -1
    assert b"feature dims" in lib.fbla_last_error()
    # a NULL tensor pointer is rejected before anything is launched
    rc = lib.fbla_linear_attn_fwd_out(ctypes.byref(p), None, None, None, None)
    assert rc == 1 and b"NULL" in lib.fbla_last_error()
    # normalize flag must match the operator
    rc = lib.fbla_simple_la_fwd_out(ctypes.byref(p), None, None, None, None)
    assert rc == 1


def test_narrow_route_sizes_and_refusals_without_a_device():
    """FBLA_FLAG_NARROW: the library answers with the sizes of the widened problem and refuses what the route does
    not serve; the Python mirror asks for it exactly for 16-bit head dims that are multiples of 16 but not 64 / 128."""
    lib = _C.lib()
    like = torch.empty(0, dtype=torch.bfloat16)
    p = P.make_problem(like, batch=2, heads=3, seq_len=1000, dk=32, dv=48, normalize=True, flags=_C.FLAG_NARROW)
    assert lib.fbla_state_floats(ctypes.byref(p)) == 2 * 3 * (64 * 64 + 64)
    p = P.make_problem(like, batch=2, heads=3, seq_len=1000, dk=96, dv=32, normalize=False, flags=_C.FLAG_NARROW)
    assert lib.fbla_state_floats(ctypes.byref(p)) == 2 * 3 * 128 * 64
    for kw, dtype in ((dict(dk=64, dv=128), torch.bfloat16),          # already the kernels' own widths
                      (dict(dk=24, dv=32), torch.bfloat16),           # rows of 48 bytes: not a multiple of 16 features
                      (dict(dk=32, dv=32), torch.float32)):           # fp32 runs on the CUDA cores
        bad = P.make_problem(torch.empty(0, dtype=dtype), batch=1, heads=1, seq_len=64, normalize=True,
                             flags=_C.FLAG_NARROW, **kw)
        assert lib.fbla_state_floats(ctypes.byref(bad)) == -1 and b"FBLA_FLAG_NARROW" in lib.fbla_last_error()
    # the mirror's own decision (pure host logic)
    def route(dtype, dk, dv, **kw):
        return P.narrow_route(P.make_problem(torch.empty(0, dtype=dtype), batch=1, heads=2, seq_len=300, dk=dk, dv=dv,
                                             normalize=True, **kw))
    assert route(torch.bfloat16, 32, 32) and route(torch.float16, 16, 112) and route(torch.bfloat16, 64, 48)
    assert not route(torch.bfloat16, 64, 64) and not route(torch.bfloat16, 128, 64)
    assert not route(torch.bfloat16, 24, 32) and not route(torch.float32, 32, 32) and not route(torch.bfloat16, 8, 8)
    assert not route(torch.bfloat16, 32, 32, flags=_C.FLAG_GENERIC)


def test_operators_refuse_cpu_tensors():
    from flash_bla.ops.linear_attn.fused import linear_attention
    from flash_bla.ops.simple_la.fused import simple_la
    x = torch.rand(1, 1, 4, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        linear_attention(x, x, x)
    with pytest.raises(RuntimeError, match="CUDA"):
        simple_la(x, x, x)


def test_varlen_argument_contract_on_cpu():
    from flash_bla.ops.linear_attn.varlen import varlen_linear_attention
    q = torch.rand(10, 2, 16)
    cu = torch.tensor([0, 4, 10], dtype=torch.int32)
    with pytest.raises(ValueError, match="CUDA tensors"):
        varlen_linear_attention(q, q, q, cu, 6)
    with pytest.raises(ValueError, match="identical shapes"):
        varlen_linear_attention(q, q[:, :1], q, cu, 6)
    with pytest.raises(ValueError, match="shape"):
        varlen_linear_attention(q[0], q[0], q[0], cu, 6)
    with pytest.raises(ValueError, match="same dtype"):
        varlen_linear_attention(q, q, q.double(), cu, 6)


def test_naive_statements_match_the_oracle():
    from oracle import bla_oracle as O
    from flash_bla.ops.linear_attn.naive import naive_decoupled_la, naive_linear_attn, naive_varlen_linear_attn
    from flash_bla.ops.simple_la.naive import naive_simple_la
    torch.manual_seed(0)
    q, k, qr, kr = (torch.rand(2, 2, 33, 8, dtype=torch.float64) for _ in range(4))
    v = torch.randn(2, 2, 33, 6, dtype=torch.float64)
    assert torch.allclose(naive_linear_attn(q, k, v), O.linear_attn_fwd(q, k, v), atol=1e-12)
    assert torch.allclose(naive_decoupled_la(q, k, qr, kr, v), O.decoupled_la_fwd(q, k, qr, kr, v), atol=1e-12)
    assert torch.allclose(naive_simple_la(q, k, v), O.simple_la_fwd(q, k, v), atol=1e-12)
    cu = torch.tensor([0, 5, 20, 33], dtype=torch.int32)
    qq, kk, vv = q[0].transpose(0, 1).contiguous(), k[0].transpose(0, 1).contiguous(), v[0].transpose(0, 1).contiguous()
    assert torch.allclose(naive_varlen_linear_attn(qq, kk, vv, cu), O.varlen_linear_attn_fwd(qq, kk, vv, cu), atol=1e-12)
