"""The four streaming passes every operator is built from, as thin Python calls
into the C ABI.  Tensors are allocated by torch (caching allocator, current
stream); the library only enqueues kernels.

    forward :  state = fwd_state(k, v)            [S = K^T V | sum k]   fp32
               o     = fwd_out(q, state)
    backward:  dq, dstate = bwd_state(q, dO, state)
               dk, dv     = bwd_in(k, v, dstate)

A caller that shards the sequence over ranks all-reduces ``state`` / ``dstate``
between the two passes (see ``flash_bla.ops.sharded``).
"""
import ctypes
import os

import torch

from flash_bla import _C


def make_problem(like, *, batch, heads, seq_len, dk, dv, normalize, scale=1.0, eps=0.0, norm_len=0,
                 cu_seqlens=None, num_seqs=0, max_seqlen=0, scale_per_seq=False, flags=0):
    p = _C.Problem()
    p.dtype = _C.dtype_code(like.dtype)
    p.batch, p.heads, p.dk, p.dv = int(batch), int(heads), int(dk), int(dv)
    p.seq_len, p.norm_len = int(seq_len), int(norm_len)
    p.cu_seqlens = None if cu_seqlens is None else cu_seqlens.data_ptr()
    p.num_seqs, p.max_seqlen = int(num_seqs), int(max_seqlen)
    p.scale = float(scale)
    p.scale_per_seq = int(bool(scale_per_seq))
    p.eps = float(eps)
    p.normalize = int(bool(normalize))
    p.flags = int(flags)
    return p


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("flash_bla operators run on CUDA tensors only (there is no CPU path)")


def _workspace(prob, like):
    n = _C.lib().fbla_workspace_bytes(ctypes.byref(prob))
    if n < 0:
        _C.check(1)
    if n == 0:
        return None, 0
    return torch.empty(n, dtype=torch.uint8, device=like.device), n


def _state_like(prob, like):
    n = _C.lib().fbla_state_floats(ctypes.byref(prob))
    if n < 0:
        _C.check(1)
    return torch.empty(n, dtype=torch.float32, device=like.device)


def state_floats(prob):
    n = _C.lib().fbla_state_floats(ctypes.byref(prob))
    if n < 0:
        _C.check(1)
    return n


def _check_state(prob, out):
    if out.dtype != torch.float32 or not out.is_contiguous() or out.numel() != state_floats(prob):
        raise ValueError("state buffer must be contiguous fp32 with fbla_state_floats() elements")
    return out


def fwd_state(op, prob, k, v, k_rope=None, out=None):
    """``out``: optional preallocated fp32 state buffer (e.g. memory that peer GPUs have mapped)."""
    _require_cuda(k, v, k_rope)
    L = _C.lib()
    with _C.device_guard(k):
        state = _state_like(prob, k) if out is None else _check_state(prob, out)
        ws, n = _workspace(prob, k)
        f = getattr(L, f"fbla_{op}_fwd_state")
        if op == "decoupled_la":
            rc = f(ctypes.byref(prob), _C.ptr(k), _C.ptr(k_rope), _C.ptr(v), _C.ptr(state), _C.ptr(ws), n,
                   _C.stream_of(k))
        else:
            rc = f(ctypes.byref(prob), _C.ptr(k), _C.ptr(v), _C.ptr(state), _C.ptr(ws), n, _C.stream_of(k))
    _C.check(rc)
    return state


def fwd_out(op, prob, q, state, o, q_rope=None):
    _require_cuda(q, state, o, q_rope)
    L = _C.lib()
    with _C.device_guard(q):
        f = getattr(L, f"fbla_{op}_fwd_out")
        if op == "decoupled_la":
            rc = f(ctypes.byref(prob), _C.ptr(q), _C.ptr(q_rope), _C.ptr(state), _C.ptr(o), _C.stream_of(q))
        else:
            rc = f(ctypes.byref(prob), _C.ptr(q), _C.ptr(state), _C.ptr(o), _C.stream_of(q))
    _C.check(rc)
    return o


def bwd_state(op, prob, q, d_o, state, dq, q_rope=None, dq_rope=None, out=None):
    _require_cuda(q, d_o, state, dq, q_rope, dq_rope)
    L = _C.lib()
    with _C.device_guard(q):
        dstate = _state_like(prob, q) if out is None else _check_state(prob, out)
        ws, n = _workspace(prob, q)
        f = getattr(L, f"fbla_{op}_bwd_state")
        if op == "decoupled_la":
            rc = f(ctypes.byref(prob), _C.ptr(q), _C.ptr(q_rope), _C.ptr(d_o), _C.ptr(state), _C.ptr(dq),
                   _C.ptr(dq_rope), _C.ptr(dstate), _C.ptr(ws), n, _C.stream_of(q))
        else:
            rc = f(ctypes.byref(prob), _C.ptr(q), _C.ptr(d_o), _C.ptr(state), _C.ptr(dq), _C.ptr(dstate),
                   _C.ptr(ws), n, _C.stream_of(q))
    _C.check(rc)
    return dstate


def bwd_in(op, prob, k, v, dstate, dk, dv, dk_rope=None):
    """``k`` is the key tensor the state was built from (k_rope when decoupled)."""
    _require_cuda(k, v, dstate, dk, dv, dk_rope)
    L = _C.lib()
    with _C.device_guard(k):
        f = getattr(L, f"fbla_{op}_bwd_in")
        if op == "decoupled_la":
            rc = f(ctypes.byref(prob), _C.ptr(k), _C.ptr(v), _C.ptr(dstate), _C.ptr(dk), _C.ptr(dk_rope),
                   _C.ptr(dv), _C.stream_of(k))
        else:
            rc = f(ctypes.byref(prob), _C.ptr(k), _C.ptr(v), _C.ptr(dstate), _C.ptr(dk), _C.ptr(dv),
                   _C.stream_of(k))
    _C.check(rc)


# ---- sequence-sharded passes on the tensor-core kernels: pieces, then one exchange kernel ---------
def sharded_supported(prob):
    return _C.lib().fbla_seq_sharded_supported(ctypes.byref(prob)) == 1


def sharded_fwd_state(prob, k, v, grp, k_rope=None):
    _require_cuda(k, v, k_rope)
    with _C.device_guard(k):
        rc = _C.lib().fbla_seq_sharded_fwd_state(ctypes.byref(prob), _C.ptr(k), _C.ptr(k_rope), _C.ptr(v),
                                                 ctypes.byref(grp), _C.stream_of(k))
    _C.check(rc)


def sharded_exchange(prob, grp, like):
    """Sum over the ranks of the pieces the preceding sharded state pass left: a new fp32 state tensor."""
    out = torch.empty(state_floats(prob), dtype=torch.float32, device=like.device)
    with _C.device_guard(like):
        rc = _C.lib().fbla_seq_sharded_exchange(ctypes.byref(prob), ctypes.byref(grp), _C.ptr(out), _C.stream_of(like))
    _C.check(rc)
    return out


def sharded_bwd_state(prob, q, d_o, state, grp, dq, q_rope=None, dq_rope=None):
    _require_cuda(q, d_o, state, dq, q_rope, dq_rope)
    with _C.device_guard(q):
        rc = _C.lib().fbla_seq_sharded_bwd_state(ctypes.byref(prob), _C.ptr(q), _C.ptr(q_rope), _C.ptr(d_o),
                                                 _C.ptr(state), ctypes.byref(grp), _C.ptr(dq), _C.ptr(dq_rope),
                                                 _C.stream_of(q))
    _C.check(rc)


# ---- one call per direction (single GPU: nothing happens between the two passes) -------------
# On the tensor-core kernels the state is left in the per-segment pieces of the reducing pass
# (FLAG_UNREDUCED): the consuming pass adds them itself, which saves a kernel per direction.  What
# forward() returns as "state" is then the workspace (a uint8 tensor) and backward() recognises it
# by that dtype.  FBLA_REDUCED_STATE=1 in the environment switches this off.
_ws_cache = {}
_want_unreduced = os.environ.get("FBLA_REDUCED_STATE", "0") != "1"


def _sizes(prob):
    """(state floats, workspace bytes, unreduced?) of a problem; the library is asked once per shape."""
    key = (prob.dtype, prob.batch, prob.heads, prob.dk, prob.dv, prob.seq_len, prob.num_seqs, prob.normalize,
           prob.flags, prob.cu_seqlens is not None)
    got = _ws_cache.get(key)
    if got is None:
        L = _C.lib()
        got = (L.fbla_state_floats(ctypes.byref(prob)), L.fbla_workspace_bytes(ctypes.byref(prob)),
               L.fbla_unreduced_state(ctypes.byref(prob)) == 1)
        if got[0] < 0 or got[1] < 0:
            _C.check(1)
        if len(_ws_cache) > 256:
            _ws_cache.clear()
        _ws_cache[key] = got
    return got


def narrow_route(prob):
    """Whether the library serves this problem on its narrow route: 16-bit linear_attn (fixed-length or packed) /
    simple_la whose feature dims are multiples of 16 but not the tensor-core kernels' own 64 / 128 (the reference's layers
    use 32).  The 64- / 128-wide kernels then read and write the tensors at their own width through TMA boxes
    that zero-fill / clip the missing features.  ``FBLA_NARROW_DIMS=0`` switches the route off."""
    if prob.dtype == _C.dtype_code(torch.float32) or (prob.flags & _C.FLAG_GENERIC):
        return False
    if os.environ.get("FBLA_NARROW_DIMS", "1") == "0":
        return False
    K, V = prob.dk, prob.dv
    if K % 16 or V % 16 or K > 128 or V > 128 or K < 16 or V < 16:
        return False
    return not (K in (64, 128) and V in (64, 128))


_narrow_cache = {}


def use_narrow(prob):
    """Sets FLAG_NARROW on ``prob`` if the narrow route applies and the tensor-core kernels take the problem with it
    (the packed layout has limits of its own: number of sequences, heads); returns whether it did."""
    if not narrow_route(prob):
        return False
    key = (prob.dtype, prob.batch, prob.heads, prob.dk, prob.dv, prob.seq_len, prob.num_seqs, prob.normalize,
           prob.cu_seqlens is not None)
    ok = _narrow_cache.get(key)
    prob.flags |= _C.FLAG_NARROW
    if ok is None:
        ok = kernel_path(prob) == 1
        if len(_narrow_cache) > 256:
            _narrow_cache.clear()
        _narrow_cache[key] = ok
    if not ok:
        prob.flags &= ~_C.FLAG_NARROW
    return ok


def _aligned16(*tensors):
    """The tensors as 16-byte aligned ones (a contiguous view at an odd storage offset is copied)."""
    return [t if t.data_ptr() % 16 == 0 else t.clone() for t in tensors]


def forward(prob, q, k, v):
    """fwd_state + fwd_out of linear_attention / simple_la / varlen; returns (o, state)."""
    _require_cuda(q, k, v)
    if use_narrow(prob):
        q, k, v = _aligned16(q, k, v)
    # the unreduced route needs the tensor-core kernels, and those need 16-byte aligned tensors (a contiguous
    # view at an odd storage offset is served by the CUDA-core kernels, as the reference serves it)
    if _want_unreduced and all(t.data_ptr() % 16 == 0 for t in (q, k, v)):
        prob.flags |= _C.FLAG_UNREDUCED
    n_state, n_ws, unreduced = _sizes(prob)
    dev = q.device
    ws = torch.empty(n_ws, dtype=torch.uint8, device=dev) if n_ws else None
    state = None if unreduced else torch.empty(n_state, dtype=torch.float32, device=dev)
    o = torch.empty_like(v)
    with _C.device_guard(q):
        rc = _C.lib().fbla_linear_attn_fwd(ctypes.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                           _C.ptr(state), _C.ptr(ws), n_ws, _C.stream_of(q))
    _C.check(rc)
    return o, (ws if unreduced else state)


def backward(prob, q, k, v, d_o, state):
    """bwd_state + bwd_in; returns (dq, dk, dv).  ``state`` is what ``forward`` returned."""
    _require_cuda(q, k, v, d_o, state)
    if use_narrow(prob):
        q, k, v, d_o = _aligned16(q, k, v, d_o)
    if state.dtype == torch.uint8:
        prob.flags |= _C.FLAG_UNREDUCED
    else:
        prob.flags &= ~_C.FLAG_UNREDUCED
    n_state, n_ws, unreduced = _sizes(prob)
    if unreduced != (state.dtype == torch.uint8):
        raise RuntimeError("the kernel path changed between forward and backward (unreduced state saved)")
    if unreduced and d_o.data_ptr() % 16 != 0:
        d_o = d_o.clone()           # the saved pieces commit the backward to the tensor-core kernels
    dev = q.device
    dstate = None if unreduced else torch.empty(n_state, dtype=torch.float32, device=dev)
    ws = torch.empty(n_ws, dtype=torch.uint8, device=dev) if n_ws else None
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    with _C.device_guard(q):
        rc = _C.lib().fbla_linear_attn_bwd(ctypes.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(), d_o.data_ptr(),
                                           state.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                           _C.ptr(dstate), _C.ptr(ws), n_ws, _C.stream_of(q))
    _C.check(rc)
    return dq, dk, dv


# Head dims the tensor-core kernels do not take (anything but 64 and 128; the reference's layers use 32) would
# run on the CUDA-core kernels at a fraction of the bandwidth.  For 16-bit inputs of streaming size it is
# cheaper to zero-pad the feature dim up to 64 / 128 -- zero key features add nothing to the state or the
# normaliser, zero value features give zero output columns -- and slice the result; autograd handles both ends.
_PAD_MIN_ROWS = 1 << 17      # batch * heads * tokens from which padding pays (below, launch cost dominates)


def padded_dims(q, v):
    """(K', V') to pad the feature dims to, or None when the tensors are served as they are."""
    if q.dtype not in (torch.float16, torch.bfloat16) or not q.is_cuda or q.dim() != 4:
        return None
    # FBLA_PAD_SMALL_DIMS=0 switches the route off (the CUDA-core kernels then serve these shapes)
    if _default_flags & _C.FLAG_GENERIC or os.environ.get("FBLA_PAD_SMALL_DIMS", "1") == "0":
        return None
    K, V = q.shape[-1], v.shape[-1]
    if K in (64, 128) and V in (64, 128):
        return None
    if K % 16 == 0 and V % 16 == 0 and K <= 128 and V <= 128 and os.environ.get("FBLA_NARROW_DIMS", "1") != "0":
        return None             # the library's narrow route reads them as they are (no copies)
    if K > 128 or V > 128 or q.shape[0] * q.shape[1] * q.shape[2] < _PAD_MIN_ROWS:
        return None
    up = lambda d: 64 if d <= 64 else 128
    return up(K), up(V)


def pad_last(x, d):
    return x if x.shape[-1] == d else torch.nn.functional.pad(x, (0, d - x.shape[-1]))


def kernel_path(prob):
    """1 when the tensor-core kernels serve ``prob``, 0 for the CUDA-core kernels."""
    return _C.lib().fbla_kernel_path(ctypes.byref(prob))


# Kernel-path override used by tests and benchmarks: inside ``generic_kernels()`` the
# CUDA-core kernels serve every call, whatever the shape.
_default_flags = 0


class generic_kernels:
    def __enter__(self):
        global _default_flags
        self._saved = _default_flags
        _default_flags = _C.FLAG_GENERIC
        return self

    def __exit__(self, *exc):
        global _default_flags
        _default_flags = self._saved
        return False


def default_flags():
    return _default_flags
