"""Piecewise sparse attention (PISA): softmax attention that is exact on the top-scoring key
blocks of every query block and approximated on the rest by the blocks' mean key / summed
value (zeroth order) plus one global first-order term.

Same public surface as the reference module ``flash_bla/ops/piecewise_attn/kernel.py``
(``chunk_reduce`` :131-149, ``fused_chunk_reduce`` :152-176, ``piecewise_sparse_attention``
:295-333).  As there, the block scores and the top-k selection are a few torch calls between
the two CUDA stages; everything that touches q, k, v runs in the sm_100a library.
"""
import ctypes
import os

import torch

from flash_bla import _C
from flash_bla.ops import _passes as P


def _problem(q, v, block_size, num_selected, scale):
    B, H, T, K = q.shape
    p = _C.PisaProblem()
    p.dtype = _C.dtype_code(q.dtype)
    p.batch, p.heads, p.dk, p.dv = B, H, K, v.shape[-1]
    p.block_size, p.num_selected, p.seq_len = int(block_size), int(num_selected), T
    p.scale = float(scale)
    return p


def _check(q, k, v):
    if q.dim() != 4 or k.shape != q.shape or v.dim() != 4 or v.shape[:3] != q.shape[:3]:
        raise ValueError("expected q, k of shape (B, H, T, K) and v of shape (B, H, T, V)")
    if not (q.dtype == k.dtype == v.dtype):
        raise ValueError("q, k and v must have the same dtype")
    if not q.is_cuda:
        raise RuntimeError("flash_bla operators run on CUDA tensors only (there is no CPU path)")


def block_statistics(q, k, v, block_size):
    """fp32 block statistics: qc, kc ``(B,H,NT,K)`` block means (true length of a ragged last
    block), vc ``(B,H,NT,V)`` block sums."""
    _check(q, k, v)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, H, T, K = q.shape
    V = v.shape[-1]
    nt = -(-T // block_size)
    prob = _problem(q, v, block_size, 1, 1.0)
    qc = torch.empty(B, H, nt, K, dtype=torch.float32, device=q.device)
    kc = torch.empty_like(qc)
    vc = torch.empty(B, H, nt, V, dtype=torch.float32, device=q.device)
    with _C.device_guard(q):
        _C.check(_C.lib().fbla_pisa_block_stats(ctypes.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), _C.stream_of(q)))
    return qc, kc, vc


def first_order_state(k, v, kc, vc, block_size):
    """h = sum over blocks of (K_c - kc_c)^T V_c = K^T V - sum_c kc_c (x) vc_c, fp32 ``(B,H,K,V)``.
    K^T V is the state pass of ``simple_la`` (tensor cores for 16-bit inputs with K, V in {64, 128})."""
    B, H, T, K = k.shape
    V = v.shape[-1]
    sp = P.make_problem(k, batch=B, heads=H, seq_len=T, dk=K, dv=V, normalize=False, scale=1.0,
                        flags=P.default_flags())
    kv = P.fwd_state("simple_la", sp, k, v)
    prob = _problem(k, v, block_size, 1, 1.0)
    h = torch.empty(B, H, K, V, dtype=torch.float32, device=k.device)
    with _C.device_guard(k):
        _C.check(_C.lib().fbla_pisa_first_order_state(ctypes.byref(prob), kv.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                                      h.data_ptr(), _C.stream_of(k)))
    return h


def block_state_norms(k, v, kc, block_size, p=2):
    """fp32 ``(B,H,NT)``: p-norm of every block's first-order state (K_c - kc_c)^T V_c over its K*V
    entries (``torch.norm(hc.flatten(-2, -1), p=p, dim=-1)`` in the reference, kernel.py:172-173),
    without materialising the per-block states."""
    k, v = k.contiguous(), v.contiguous()
    B, H, T, K = k.shape
    prob = _problem(k, v, block_size, 1, 1.0)
    nt = kc.shape[-2]
    out = torch.empty(B, H, nt, dtype=torch.float32, device=k.device)
    with _C.device_guard(k):
        _C.check(_C.lib().fbla_pisa_block_hnorm(ctypes.byref(prob), k.data_ptr(), v.data_ptr(), kc.contiguous().data_ptr(),
                                                float(p), out.data_ptr(), _C.stream_of(k)))
    return out


def chunk_reduce(q, k, v, chunk_size):
    """Block means of q and k and block sums of v, in the dtype of the inputs."""
    qc, kc, vc = block_statistics(q, k, v, chunk_size)
    return qc.to(q.dtype), kc.to(k.dtype), vc.to(v.dtype)


def fused_chunk_reduce(q, k, v, chunk_size, use_bias=False, p=2):
    """``(qc, kc, vc, h, bias)`` in the dtype of the inputs; ``bias`` is ``None`` unless ``use_bias``."""
    qc, kc, vc = block_statistics(q, k, v, chunk_size)
    h = first_order_state(k.contiguous(), v.contiguous(), kc, vc, chunk_size)
    bias = None
    if use_bias:        # (B, H, 1, NT), as the reference's h_norm[..., None, :]
        bias = block_state_norms(k, v, kc, chunk_size, p).to(v.dtype)[..., None, :]
    return qc.to(q.dtype), kc.to(k.dtype), vc.to(v.dtype), h.to(v.dtype), bias


_SELECT_MAX_BLOCKS = 1024


def select_blocks(qc, kc, scale, density, dtype, bias=None, use_torch=False):
    """Indices ``(B,H,NT,NS)`` of the key blocks each query block attends exactly: top-k of the
    block-mean scores computed in the dtype of the inputs, ``NS = max(1, int(density * NT))``.
    ``bias`` ``(B,H,1,NT)``: rank ``softmax(score + log(bias + 1e-5))`` instead (kernel.py:314-315).

    One CUDA kernel (``fbla_pisa_select_blocks``, int32 indices, equal scores to the lower block) for up
    to 1024 blocks; beyond that, or with ``use_torch``, the reference's einsum / softmax / topk."""
    nt = kc.shape[-2]
    top_k = max(1, int(density * nt))
    if use_torch or not qc.is_cuda or nt > _SELECT_MAX_BLOCKS:
        score = torch.einsum('bhid,bhjd->bhij', qc.to(dtype), (kc * scale).to(dtype))
        if bias is not None:
            score = torch.softmax(score + torch.log(bias.to(dtype) + 1e-5), dim=-1)
        return torch.topk(score, k=top_k, dim=-1).indices
    B, H, _, K = qc.shape
    qc, kc = qc.float().contiguous(), kc.float().contiguous()
    p = _C.PisaProblem()
    p.dtype = _C.dtype_code(dtype)
    p.batch, p.heads, p.dk, p.dv = B, H, K, K
    p.block_size, p.num_selected, p.seq_len = 1, top_k, nt          # one "token" per block: NT blocks
    p.scale = float(scale)
    hn = None if bias is None else bias.float().reshape(B, H, nt).contiguous()
    idx = torch.empty(B, H, nt, top_k, dtype=torch.int32, device=qc.device)
    with _C.device_guard(qc):
        _C.check(_C.lib().fbla_pisa_select_blocks(ctypes.byref(p), qc.data_ptr(), kc.data_ptr(), _C.ptr(hn),
                                                  idx.data_ptr(), _C.stream_of(qc)))
    return idx


def attention_forward(q, k, v, kc, vc, h, indices, block_size, scale, want_stats=False):
    """The attention stage with statistics and selection given (all fp32 statistics)."""
    _check(q, k, v)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, H, T, K = q.shape
    idx = indices.to(torch.int32).contiguous()
    prob = _problem(q, v, block_size, idx.shape[-1], scale)
    o = torch.empty_like(v)
    stats = torch.empty(B, H, T, 4, dtype=torch.float32, device=q.device) if want_stats else None
    kc, vc, h = kc.contiguous(), vc.contiguous(), h.contiguous()
    with _C.device_guard(q):
        # the tcgen05 kernel wants 16-bit copies of the statistics: scratch from the caching allocator
        need = 0 if os.environ.get("FBLA_PISA_TC", "1") == "0" else _C.lib().fbla_pisa_fwd_scratch_bytes(ctypes.byref(prob))
        scratch = torch.empty(need, dtype=torch.uint8, device=q.device) if need > 0 else None
        _C.check(_C.lib().fbla_pisa_fwd_ws(ctypes.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                           kc.data_ptr(), vc.data_ptr(), h.data_ptr(), idx.data_ptr(), o.data_ptr(),
                                           _C.ptr(stats), _C.ptr(scratch), max(need, 0), _C.stream_of(q)))
    return (o, stats) if want_stats else o


def attention_backward(q, k, v, o, do, kc, vc, h, indices, stats, block_size, scale):
    """Gradients (dq, dk, dv) of ``attention_forward`` composed with the block statistics, the
    selection ``indices`` held constant."""
    q, k, v, o, do = (x.contiguous() for x in (q, k, v, o, do))
    B, H, T, K = q.shape
    V = v.shape[-1]
    idx = indices.to(torch.int32).contiguous()
    nt = idx.shape[-2]
    prob = _problem(q, v, block_size, idx.shape[-1], scale)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    n = _C.lib().fbla_pisa_bwd_scratch_floats(ctypes.byref(prob))
    if n < 0:
        _C.check(1)
    scratch = torch.empty(n, dtype=torch.float32, device=q.device)
    with _C.device_guard(q):
        _C.check(_C.lib().fbla_pisa_bwd(ctypes.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                        do.data_ptr(), kc.contiguous().data_ptr(), vc.contiguous().data_ptr(),
                                        h.contiguous().data_ptr(), idx.data_ptr(), stats.data_ptr(), dq.data_ptr(),
                                        dk.data_ptr(), dv.data_ptr(), scratch.data_ptr(), n, _C.stream_of(q)))
    return dq, dk, dv


class PiecewiseSparseAttnFunction(torch.autograd.Function):
    """Forward as the reference; the backward (which the reference lacks) treats the selected
    block indices as constants."""

    @staticmethod
    def forward(ctx, q, k, v, density, block_size, scale, use_bias=False):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        qc, kc, vc = block_statistics(q, k, v, block_size)
        h = first_order_state(k, v, kc, vc, block_size)
        bias = block_state_norms(k, v, kc, block_size)[..., None, :] if use_bias else None
        indices = select_blocks(qc, kc, scale, density, q.dtype, bias)
        o, stats = attention_forward(q, k, v, kc, vc, h, indices, block_size, scale, want_stats=True)
        ctx.save_for_backward(q, k, v, o, kc, vc, h, indices, stats)
        ctx.block_size, ctx.scale = block_size, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, kc, vc, h, indices, stats = ctx.saved_tensors
        dq, dk, dv = attention_backward(q, k, v, o, do, kc, vc, h, indices, stats, ctx.block_size, ctx.scale)
        return dq, dk, dv, None, None, None, None


def piecewise_sparse_attention(q, k, v, density=0.1, block_size=64, scale=None, use_bias=False):
    r"""
    Args:
        q, k: queries / keys `(B, H, T, K)`; v: values `(B, H, T, V)`.
        density: fraction of key blocks attended exactly per query block (at least one).
        block_size: tokens per block.
        scale: logit scale, `K ** -0.5` by default.
        use_bias: add the log of the blocks' first-order norm to the selection scores.
    Returns the attention output `(B, H, T, V)`.
    """
    _check(q, k, v)
    K = k.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    return PiecewiseSparseAttnFunction.apply(q, k, v, density, block_size, scale, bool(use_bias))
