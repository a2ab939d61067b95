"""Decoupled bidirectional linear attention: the numerator uses the rotary
q_rope / k_rope, the normaliser the plain q / k.

    S = K_rope^T (V * scale),  kmean = mean_t K,  O = Q_rope S / (Q . kmean + eps)

Same public surface as the reference module
``flash_bla/ops/linear_attn/decoupled.py`` (``DecoupledLAFunction`` :411-509,
``decoupled_la`` :512-542).
"""
from typing import Optional

import torch

from flash_bla.ops import _passes as P
from flash_bla import _C
from flash_bla.utils import contiguous

_OP = "decoupled_la"


def _problem(q, v, scale, eps, norm_len=0):
    B, H, L, K = q.shape
    prob = P.make_problem(q, batch=B, heads=H, seq_len=L, dk=K, dv=v.shape[-1], normalize=True,
                          scale=scale, eps=eps, norm_len=norm_len, flags=P.default_flags())
    # head dims below the 64 x 64 tensor-core kernels of this operator (the reference layers use 32)
    if K <= 64 and v.shape[-1] <= 64 and q.is_cuda:
        P.use_narrow(prob)
    return prob


def _aligned(prob, *tensors):
    """The narrow route reads through TMA: contiguous views at an odd storage offset are copied."""
    if prob.flags & _C.FLAG_NARROW:
        return [t if t.data_ptr() % 16 == 0 else t.clone() for t in tensors]
    return list(tensors)


def _check(q, k, q_rope, k_rope, v):
    if q.dim() != 4 or v.dim() != 4 or any(x.shape != q.shape for x in (k, q_rope, k_rope)) \
            or v.shape[:3] != q.shape[:3]:
        raise ValueError("expected q, k, q_rope, k_rope of shape (B, H, L, K) and v of shape (B, H, L, V)")
    if not (q.dtype == k.dtype == q_rope.dtype == k_rope.dtype == v.dtype):
        raise ValueError("all inputs must have the same dtype")


class DecoupledLAFunction(torch.autograd.Function):

    @staticmethod
    @contiguous
    def forward(ctx, q, k, q_rope, k_rope, v, scale, eps):
        _check(q, k, q_rope, k_rope, v)
        prob = _problem(q, v, scale, eps)
        q, k, q_rope, k_rope, v = _aligned(prob, q, k, q_rope, k_rope, v)
        state = P.fwd_state(_OP, prob, k, v, k_rope=k_rope)
        o = P.fwd_out(_OP, prob, q, state, torch.empty_like(v), q_rope=q_rope)
        ctx.save_for_backward(q, q_rope, k_rope, v, state)
        ctx.scale, ctx.eps = scale, eps
        return o

    @staticmethod
    @contiguous
    def backward(ctx, do):
        q, q_rope, k_rope, v, state = ctx.saved_tensors
        prob = _problem(q, v, ctx.scale, ctx.eps)
        do, = _aligned(prob, do)
        dq, dq_rope = torch.empty_like(q), torch.empty_like(q_rope)
        dstate = P.bwd_state(_OP, prob, q, do, state, dq, q_rope=q_rope, dq_rope=dq_rope)
        dk, dk_rope, dv = torch.empty_like(k_rope), torch.empty_like(k_rope), torch.empty_like(v)
        P.bwd_in(_OP, prob, k_rope, v, dstate, dk, dv, dk_rope=dk_rope)
        return dq, dk, dq_rope, dk_rope, dv, None, None


def decoupled_la(
    q: torch.Tensor,
    k: torch.Tensor,
    q_rope: torch.Tensor,
    k_rope: torch.Tensor,
    v: torch.Tensor,
    scale: Optional[float] = None,
    eps: float = 1e-6,
) -> torch.Tensor:
    r"""
    Args:
        q, k: plain queries / keys `(B, H, L, K)` (normaliser)
        q_rope, k_rope: rotary queries / keys `(B, H, L, K)` (numerator)
        v: values `(B, H, L, V)`
        scale: multiplies the values inside the state; defaults to `1 / L`.
        eps: added to the normaliser.
    """
    if scale is None:
        scale = k.shape[-2] ** -1.0
    pad = P.padded_dims(q, v) if (k.shape == q.shape == q_rope.shape == k_rope.shape) else None
    if pad is not None and pad == (64, 64):      # the decoupled tensor-core kernels exist at 64 x 64 only
        o = DecoupledLAFunction.apply(*(P.pad_last(x, 64) for x in (q, k, q_rope, k_rope, v)), scale, eps)
        return o[..., :v.shape[-1]]
    return DecoupledLAFunction.apply(q, k, q_rope, k_rope, v, scale, eps)
