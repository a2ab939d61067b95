"""The no-allocation forward state pass, fbla_linear_attn_fwd_state_noalloc.

It exists for embedders that hold nothing but the tensors they were given and may not
allocate device memory themselves (a plugin inside another runtime's operator, a serving
loop with a fixed memory budget): the scratch lives in a device array inside the library.
The test calls it through the C ABI twice in a row, with different inputs, and checks each
result against the regular entry point fed a caller-allocated workspace.  The file name
sorts last so that a run stopping at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

from flash_bla import _C
from flash_bla.ops import _passes as P

pytestmark = pytest.mark.gpu


def _inputs(seed, B, H, T, D, dtype):
    g = torch.Generator(device="cuda").manual_seed(seed)
    k = torch.rand(B, H, T, D, device="cuda", generator=g).to(dtype)
    v = torch.randn(B, H, T, D, device="cuda", generator=g).to(dtype)
    return k, v


def _state_noalloc(prob, k, v):
    lib = _C.lib()
    n = lib.fbla_state_floats(ctypes.byref(prob))
    state = torch.full((n,), float("nan"), dtype=torch.float32, device="cuda")
    rc = lib.fbla_linear_attn_fwd_state_noalloc(ctypes.byref(prob), k.data_ptr(), v.data_ptr(), state.data_ptr(),
                                                _C.stream_of(k))
    _C.check(rc)
    return state


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_two_calls_match_the_workspace_entry_point(dtype):
    B, H, T, D = 2, 4, 3000, 64
    prob = P.make_problem(torch.empty(0, dtype=dtype), batch=B, heads=H, seq_len=T, dk=D, dv=D, normalize=True,
                          scale=1.0 / T, eps=1e-6)
    assert P.kernel_path(prob) == 1
    for seed in (0, 1):                      # the second call finds the first call's partials in the array
        k, v = _inputs(seed, B, H, T, D, dtype)
        got = _state_noalloc(prob, k, v)
        ref = P.fwd_state("linear_attn", prob, k, v)
        torch.cuda.synchronize()
        # same kernels, same schedule, same summation order: the tolerance of the other tests
        # (1e-5 relative for fp32 quantities) is met with equality
        assert torch.isfinite(got).all()
        assert torch.equal(got, ref)
        exact = torch.cat([(k.float().transpose(-1, -2) @ v.float()).flatten(-2), k.float().sum(-2)], -1).flatten()
        assert ((got - exact).norm() / exact.norm()).item() < 1e-5
    # no kernel of the entry point gave up a wait: its status word reads zero
    status = ctypes.c_int(-1)
    _C.check(_C.lib().fbla_noalloc_status(ctypes.byref(status), 0))
    assert status.value == 0


def test_refuses_what_it_cannot_serve():
    lib = _C.lib()
    k, v = _inputs(0, 1, 1, 256, 64, torch.bfloat16)
    state = torch.empty(64 * 64 + 64, dtype=torch.float32, device="cuda")
    # more scratch than the built-in array holds
    big = P.make_problem(k, batch=64, heads=64, seq_len=1 << 20, dk=128, dv=128, normalize=True, scale=1.0)
    rc = lib.fbla_linear_attn_fwd_state_noalloc(ctypes.byref(big), k.data_ptr(), v.data_ptr(), state.data_ptr(), None)
    assert rc == 4 and b"scratch" in lib.fbla_last_error()
    # shapes of the CUDA-core kernels
    odd = P.make_problem(k.float(), batch=1, heads=1, seq_len=256, dk=64, dv=64, normalize=True, scale=1.0)
    rc = lib.fbla_linear_attn_fwd_state_noalloc(ctypes.byref(odd), k.data_ptr(), v.data_ptr(), state.data_ptr(), None)
    assert rc == 2
    # a NULL tensor
    ok = P.make_problem(k, batch=1, heads=1, seq_len=256, dk=64, dv=64, normalize=True, scale=1.0)
    rc = lib.fbla_linear_attn_fwd_state_noalloc(ctypes.byref(ok), None, v.data_ptr(), state.data_ptr(), None)
    assert rc == 1
