"""Failure paths on the GPU, without faulting or hanging it: a wait for a peer that never answers
runs into its (shortened) limit, the kernel returns, the status word names the wait, the next call
is refused, and after clearing the status the library works again.  Each case runs in a child
process (the wait limit is read from the environment once per process) on ONE GPU: the "peer" is a
second set of buffers on the same device that nothing ever writes."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "flash-bidirectional-linear-attention_b200")

_PRELUDE = """
import ctypes, os, sys
os.environ["FBLA_PEER_WAIT_MS"] = "100"
sys.path.insert(0, %r)
import torch
from flash_bla import _C
from flash_bla.ops import _passes as P
from flash_bla.ops.linear_attn.fused import linear_attention
L = _C.lib()
torch.manual_seed(0)
B, H, T, D = 1, 2, 512, 64
q = (torch.rand(B, H, T, D, device="cuda") + 0.1).bfloat16()
k = (torch.rand(B, H, T, D, device="cuda") + 0.1).bfloat16()
v = torch.randn(B, H, T, D, device="cuda").bfloat16()

def works_again():
    o = linear_attention(q, k, v)
    qf, kf, vf = q.float(), k.float(), v.float()
    ref = (qf @ (kf.transpose(-1, -2) @ vf / T)) / ((qf * kf.mean(-2, keepdim=True)).sum(-1, keepdim=True) + 1e-6)
    torch.cuda.synchronize()
    assert ((o.float() - ref).abs().max() / ref.pow(2).mean().sqrt()).item() < 2e-2

def refused():
    try:
        linear_attention(q, k, v)
    except RuntimeError as e:
        return "bounded wait" in str(e)
    return False
""" % PKG


def _run(body):
    code = _PRELUDE + textwrap.dedent(body)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "CHILD-OK" in out.stdout


_GROUP = """
def make_group(prob):
    n = L.fbla_state_floats(ctypes.byref(prob))
    n_parts = L.fbla_seq_sharded_part_floats(ctypes.byref(prob))
    assert n > 0 and n_parts >= n
    parts = [torch.zeros(n_parts, device="cuda") for _ in range(2)]
    full = [torch.zeros(n, device="cuda") for _ in range(2)]
    flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2)]
    arr = ctypes.c_void_p * 2
    tabs = [arr(*[t.data_ptr() for t in ts]) for ts in (parts, full, flags)]
    g = _C.PeerGroup()
    g.world, g.rank, g.epoch, g.reserved = 2, 0, 1, 0
    g.parts, g.full, g.flags = (ctypes.cast(t, ctypes.POINTER(ctypes.c_void_p)) for t in tabs)
    return g, parts, full, flags, tabs, n
"""


def test_sequence_sharded_exchange_gives_up_on_a_silent_peer_and_recovers():
    _run(_GROUP + """
prob = P.make_problem(q, batch=B, heads=H, seq_len=T, dk=D, dv=D, normalize=True, scale=1.0 / (2 * T),
                      eps=1e-6, norm_len=2 * T)
assert L.fbla_seq_sharded_supported(ctypes.byref(prob)) == 1
g, parts, full, flags, tabs, n = make_group(prob)
st = _C.stream_of(q)
_C.check(L.fbla_seq_sharded_fwd_state(ctypes.byref(prob), k.data_ptr(), None, v.data_ptr(), ctypes.byref(g), st))
state = torch.zeros(n, device="cuda")
_C.check(L.fbla_seq_sharded_exchange(ctypes.byref(prob), ctypes.byref(g), state.data_ptr(), st))
torch.cuda.synchronize()                                         # returns: the wait is bounded
assert flags[0][0].item() == 1 and flags[1][0].item() == 1      # rank 0 told both ranks; rank 1 stays silent
assert L.fbla_device_status() == 911, L.fbla_device_status()
assert torch.isnan(state).all()                                  # no sum without the peer
assert refused()
L.fbla_clear_device_status()
assert L.fbla_device_status() == 0
works_again()
print("CHILD-OK")
""")


@pytest.mark.parametrize("two_round", ["0", "1"])
def test_sequence_sharded_calls_dry_run_with_the_peer_flags_preset(two_round):
    """The sequence-sharded calls on one GPU: rank 0 of two, with rank 1's flags already at the exchange
    number (nothing waits) and rank 1's pieces all zero, in the one-round and in the two-round form of the
    exchange.  Outputs and gradients must be bit-identical to the plain operator (same pieces, same order
    of addition; in the two-round form for the units rank 0 owns, the others come from rank 1's zeros)."""
    _run("os.environ['FBLA_PEER_TWO_ROUND'] = '%s'\n" % two_round + _GROUP + """
two_round = os.environ['FBLA_PEER_TWO_ROUND'] == '1'
B, H = 1, 4                                           # rank 0 owns units 0 and 1
q4 = (torch.rand(B, H, T, D, device="cuda") + 0.1).bfloat16()
k4 = (torch.rand(B, H, T, D, device="cuda") + 0.1).bfloat16()
v4 = torch.randn(B, H, T, D, device="cuda").bfloat16()
do4 = torch.randn(B, H, T, D, device="cuda").bfloat16()
prob = P.make_problem(q4, batch=B, heads=H, seq_len=T, dk=D, dv=D, normalize=True, scale=1.0 / T,
                      eps=1e-6, norm_len=T)
g, parts, full, flags, tabs, n = make_group(prob)
st = _C.stream_of(q4)
o, dq, dk, dv = (torch.empty_like(q4) for _ in range(4))
xs = [x.clone().requires_grad_() for x in (q4, k4, v4)]
want = linear_attention(*xs)
want.backward(do4)
own = slice(0, 2) if two_round else slice(0, 4)       # one round: rank 0 sums every unit itself
for epoch in (1, 2, 3, 4):                            # two forward + backward rounds
    g.epoch = epoch
    flags[0][1] = epoch                               # "rank 1 has entered the exchange" (its pieces: all zero)
    flags[0][17] = epoch                              # "rank 1 has summed its units"
    if epoch % 2 == 1:
        _C.check(L.fbla_seq_sharded_fwd_state(ctypes.byref(prob), k4.data_ptr(), None, v4.data_ptr(), ctypes.byref(g), st))
        state = torch.full((n,), float("nan"), device="cuda")
        _C.check(L.fbla_seq_sharded_exchange(ctypes.byref(prob), ctypes.byref(g), state.data_ptr(), st))
        P.fwd_out("linear_attn", prob, q4, state, o)
    else:
        _C.check(L.fbla_seq_sharded_bwd_state(ctypes.byref(prob), q4.data_ptr(), None, do4.data_ptr(), state.data_ptr(),
                                              ctypes.byref(g), dq.data_ptr(), None, st))
        dstate = torch.full((n,), float("nan"), device="cuda")
        _C.check(L.fbla_seq_sharded_exchange(ctypes.byref(prob), ctypes.byref(g), dstate.data_ptr(), st))
        P.bwd_in("linear_attn", prob, k4, v4, dstate, dk, dv)
    torch.cuda.synchronize()
    assert L.fbla_device_status() == 0
    if epoch % 2 == 1:
        assert torch.isfinite(state).all()
        assert torch.equal(o[:, own], want[:, own])
    else:
        assert torch.equal(dq[:, own], xs[0].grad[:, own])
        assert torch.equal(dk[:, own], xs[1].grad[:, own]) and torch.equal(dv[:, own], xs[2].grad[:, own])
    assert flags[0][32].item() == 0                   # the CTA ticket is back at zero
print("CHILD-OK")
""")


def test_state_sum_kernel_gives_up_on_a_silent_peer_and_recovers():
    _run("""
    n = 4096
    bufs = [torch.ones(n, device="cuda") for _ in range(2)]
    flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2)]
    arr = ctypes.c_void_p * 2
    out = torch.zeros(n, device="cuda")
    rc = L.fbla_peer_state_sum(2, 0, arr(*[b.data_ptr() for b in bufs]), arr(*[f.data_ptr() for f in flags]), n, 1,
                               out.data_ptr(), _C.stream_of(out))
    _C.check(rc)
    torch.cuda.synchronize()
    assert L.fbla_device_status() == 901
    assert torch.isnan(out).all()                                    # no sum without the peer
    assert refused()
    L.fbla_clear_device_status()
    works_again()
    print("CHILD-OK")
    """)
