"""Un-normalised bidirectional linear attention:  O = Q (K^T (V * scale)).

Same public surface as the reference module ``flash_bla/ops/simple_la/fused.py``
(``SimpleLinearAttnFunction`` :495-626, ``simple_la`` :629-656), including the
accepted-and-ignored ``retuen_states`` keyword (sic).
"""
from typing import Optional

import torch

from flash_bla.ops import _passes as P
from flash_bla.utils import contiguous

_OP = "simple_la"


def _problem(q, v, scale):
    B, H, L, K = q.shape
    return P.make_problem(q, batch=B, heads=H, seq_len=L, dk=K, dv=v.shape[-1], normalize=False,
                          scale=scale, flags=P.default_flags())


class SimpleLinearAttnFunction(torch.autograd.Function):

    @staticmethod
    @contiguous
    def forward(ctx, q, k, v, scale):
        if q.dim() != 4 or k.shape != q.shape or v.dim() != 4 or v.shape[:3] != q.shape[:3]:
            raise ValueError("expected q, k of shape (B, H, L, K) and v of shape (B, H, L, V)")
        prob = _problem(q, v, scale)
        o, state = P.forward(prob, q, k, v)
        ctx.save_for_backward(q, k, v, state)
        ctx.scale = scale
        return o

    @staticmethod
    @contiguous
    def backward(ctx, do):
        q, k, v, state = ctx.saved_tensors
        prob = _problem(q, v, ctx.scale)
        dq, dk, dv = P.backward(prob, q, k, v, do, state)
        return dq, dk, dv, None


def simple_la(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: Optional[float] = None,
    retuen_states: Optional[bool] = False,
) -> torch.Tensor:
    r"""
    Args:
        q: queries of shape `(B, H, L, K)`
        k: keys of shape `(B, H, L, K)`
        v: values of shape `(B, H, L, V)`
        scale: multiplies the values inside the state; defaults to `K ** -0.5`.
        retuen_states: accepted for compatibility and ignored, as in the reference.
    """
    if scale is None:
        scale = q.shape[-1] ** -0.5
    pad = P.padded_dims(q, v) if k.shape == q.shape else None
    if pad is not None:
        o = SimpleLinearAttnFunction.apply(P.pad_last(q, pad[0]), P.pad_last(k, pad[0]), P.pad_last(v, pad[1]), scale)
        return o[..., :v.shape[-1]]
    return SimpleLinearAttnFunction.apply(q, k, v, scale)
