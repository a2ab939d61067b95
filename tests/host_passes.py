"""A host-side stand-in for ``flash_bla.ops._passes`` (the four passes on CPU tensors with
the library's state layout), used ONLY by the CPU tests of the multi-rank wrappers: the
wrappers' algebra (global length, one all-reduce per direction, what is summed) can then be
checked with gloo ranks on a machine without a GPU.  It follows the oracle's formulas."""
import types

import torch


def make_problem(like, *, batch, heads, seq_len, dk, dv, normalize, scale=1.0, eps=0.0, norm_len=0, flags=0, **_):
    return types.SimpleNamespace(batch=batch, heads=heads, seq_len=seq_len, dk=dk, dv=dv, normalize=normalize,
                                 scale=scale, eps=eps, norm_len=norm_len or seq_len)


def default_flags():
    return 0


def _split(prob, state):
    B, H, K, V = prob.batch, prob.heads, prob.dk, prob.dv
    st = state.view(B, H, -1)
    S = st[..., :K * V].view(B, H, K, V)
    vec = st[..., K * V:] if prob.normalize else None
    return S, vec


def _pack(prob, S, vec):
    parts = [S.flatten(-2)] + ([vec] if prob.normalize else [])
    return torch.cat(parts, -1).contiguous().view(-1).float()


def fwd_state(op, prob, k, v, k_rope=None, out=None):
    kr = (k if k_rope is None else k_rope).double()
    return _pack(prob, kr.transpose(-1, -2) @ v.double(), k.double().sum(-2))


def _z(prob, q, vec):
    return (q.double() * (vec.double() / prob.norm_len)[..., None, :]).sum(-1, keepdim=True) + prob.eps


def fwd_out(op, prob, q, state, o, q_rope=None):
    S, vec = _split(prob, state)
    qr = (q if q_rope is None else q_rope).double()
    num = qr @ (S.double() * prob.scale)
    o.copy_(num / _z(prob, q, vec) if prob.normalize else num)
    return o


def bwd_state(op, prob, q, d_o, state, dq, q_rope=None, dq_rope=None, out=None):
    S, vec = _split(prob, state)
    qr = (q if q_rope is None else q_rope).double()
    t = d_o.double() @ (S.double() * prob.scale).transpose(-1, -2)
    if not prob.normalize:
        dq.copy_(t)
        return _pack(prob, qr.transpose(-1, -2) @ d_o.double(), None)
    z = _z(prob, q, vec)
    km = vec.double() / prob.norm_len
    dz = -(qr * t).sum(-1, keepdim=True) / (z * z)
    if dq_rope is None:
        dq.copy_(t / z + dz * km[..., None, :])
    else:
        dq_rope.copy_(t / z)
        dq.copy_(dz * km[..., None, :])
    return _pack(prob, (qr / z).transpose(-1, -2) @ d_o.double(), (dz * q.double()).sum(-2))


def bwd_in(op, prob, k, v, dstate, dk, dv, dk_rope=None):
    dS, dvec = _split(prob, dstate)
    dS = dS.double() * prob.scale
    g = v.double() @ dS.transpose(-1, -2)
    dv.copy_(k.double() @ dS)
    if not prob.normalize:
        dk.copy_(g)
        return
    dkm = (dvec.double() / prob.norm_len)[..., None, :]
    if dk_rope is None:
        dk.copy_(g + dkm)
    else:
        dk_rope.copy_(g)
        dk.copy_(dkm.expand_as(dk))
