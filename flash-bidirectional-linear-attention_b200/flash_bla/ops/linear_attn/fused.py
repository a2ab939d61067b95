"""Normalised bidirectional linear attention.

    S = K^T (V * scale),   kmean = mean_t K,   O = Q S / (Q . kmean + eps)

Same public surface as the reference module ``flash_bla/ops/linear_attn/fused.py``
(``LinearAttnFunction`` :350-453, ``linear_attention`` :456-480); the work is done
by the sm_100a library through ``flash_bla.ops._passes``.  The feature map is
applied by the caller: q and k are expected to be positive already.
"""
from typing import Optional

import torch

from flash_bla.ops import _passes as P
from flash_bla.utils import contiguous

_OP = "linear_attn"


def _problem(q, v, scale, eps, norm_len=0):
    B, H, L, K = q.shape
    return P.make_problem(q, batch=B, heads=H, seq_len=L, dk=K, dv=v.shape[-1], normalize=True,
                          scale=scale, eps=eps, norm_len=norm_len, flags=P.default_flags())


def _check(q, k, v):
    if q.dim() != 4 or k.shape != q.shape or v.dim() != 4 or v.shape[:3] != q.shape[:3]:
        raise ValueError(f"expected q, k of shape (B, H, L, K) and v of shape (B, H, L, V); got "
                         f"{tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    if not (q.dtype == k.dtype == v.dtype):
        raise ValueError("q, k and v must have the same dtype")


class LinearAttnFunction(torch.autograd.Function):

    @staticmethod
    @contiguous
    def forward(ctx, q, k, v, scale, eps):
        _check(q, k, v)
        prob = _problem(q, v, scale, eps)
        o, state = P.forward(prob, q, k, v)
        # The fp32 state is a few KB per head; keeping it avoids pass 1 in backward.
        ctx.save_for_backward(q, k, v, state)
        ctx.scale, ctx.eps = scale, eps
        return o

    @staticmethod
    @contiguous
    def backward(ctx, do):
        q, k, v, state = ctx.saved_tensors
        prob = _problem(q, v, ctx.scale, ctx.eps)
        dq, dk, dv = P.backward(prob, q, k, v, do, state)
        return dq, dk, dv, None, None


def linear_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: Optional[float] = None,
    eps: float = 1e-6,
    layout: str = "bhld",
) -> torch.Tensor:
    r"""
    Args:
        q: queries of shape `(B, H, L, K)`
        k: keys of shape `(B, H, L, K)`
        v: values of shape `(B, H, L, V)`
        scale: multiplies the values inside the state; defaults to `1 / L`.
        eps: added to the normaliser `q . mean_t k`.
        layout: `"bhld"` (the reference's layout, default) or `"blhd"`: q, k `(B, L, H, K)`, v and the
            result `(B, L, H, V)` -- the layout a projection followed by a head split produces, so the
            caller's `permute(0, 2, 1, 3).contiguous()` copies (reference layers, e.g.
            `flash_bla/layers/mlla.py:74-80`) are not needed.  Served by the packed-sequence kernels.
    """
    if layout == "blhd":
        return _linear_attention_blhd(q, k, v, scale, eps)
    if layout != "bhld":
        raise ValueError(f"layout must be 'bhld' or 'blhd', got {layout!r}")
    if scale is None:
        scale = k.shape[-2] ** -1.0
    pad = P.padded_dims(q, v) if k.shape == q.shape else None
    if pad is not None:
        o = LinearAttnFunction.apply(P.pad_last(q, pad[0]), P.pad_last(k, pad[0]), P.pad_last(v, pad[1]), scale, eps)
        return o[..., :v.shape[-1]]
    return LinearAttnFunction.apply(q, k, v, scale, eps)


_cu_cache = {}


def _linear_attention_blhd(q, k, v, scale, eps):
    # (B, L, H, D) contiguous is the packed layout with B sequences of L tokens each.
    from flash_bla.ops.linear_attn.varlen import VarlenLinearAttnFunction
    if q.dim() != 4 or k.shape != q.shape or v.dim() != 4 or v.shape[:3] != q.shape[:3]:
        raise ValueError(f"expected q, k of shape (B, L, H, K) and v of shape (B, L, H, V); got "
                         f"{tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    B, L, H, K = q.shape
    key = (B, L, q.device)
    cu = _cu_cache.get(key)
    if cu is None:
        if len(_cu_cache) > 64:
            _cu_cache.clear()
        cu = _cu_cache[key] = torch.arange(0, (B + 1) * L, max(L, 1), dtype=torch.int32, device=q.device)[:B + 1]
    o = VarlenLinearAttnFunction.apply(q.reshape(B * L, H, K), k.reshape(B * L, H, K), v.reshape(B * L, H, v.shape[-1]),
                                       cu, max(L, 1), None if scale is None else float(scale), eps)
    return o.view(B, L, H, v.shape[-1])
