"""Bidirectional linear attention over packed variable-length sequences.

Same public surface and argument contract as the reference module
``flash_bla/ops/linear_attn/varlen.py`` (``VarlenLinearAttnFunction`` :335-505,
``varlen_linear_attention`` :508-568, argument checks :544-565).
"""
from typing import Optional, Union

import torch

from flash_bla.ops import _passes as P
from flash_bla.utils import contiguous

_OP = "varlen_linear_attn"


def _problem(q, v, cu_seqlens, max_seqlen, scale, eps):
    total, H, K = q.shape
    return P.make_problem(q, batch=1, heads=H, seq_len=total, dk=K, dv=v.shape[-1], normalize=True,
                          scale=0.0 if scale is None else scale, eps=eps, cu_seqlens=cu_seqlens,
                          num_seqs=cu_seqlens.numel() - 1, max_seqlen=max_seqlen,
                          scale_per_seq=scale is None, flags=P.default_flags())


class VarlenLinearAttnFunction(torch.autograd.Function):

    @staticmethod
    @contiguous
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, scale, eps):
        # max_seqlen is only an upper bound; the kernels clip at each sequence's end.
        max_seqlen = min(int(max_seqlen), q.shape[0]) if q.shape[0] > 0 else 1
        prob = _problem(q, v, cu_seqlens, max_seqlen, scale, eps)
        o, state = P.forward(prob, q, k, v)
        ctx.save_for_backward(q, k, v, cu_seqlens, state)
        ctx.max_seqlen, ctx.scale, ctx.eps = max_seqlen, scale, eps
        return o

    @staticmethod
    @contiguous
    def backward(ctx, do):
        q, k, v, cu_seqlens, state = ctx.saved_tensors
        prob = _problem(q, v, cu_seqlens, ctx.max_seqlen, ctx.scale, ctx.eps)
        dq, dk, dv = P.backward(prob, q, k, v, do, state)
        return dq, dk, dv, None, None, None, None


def varlen_linear_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens: torch.Tensor,
    max_seqlen: int,
    scale: Optional[Union[float, int]] = None,
    eps: float = 1e-6,
) -> torch.Tensor:
    """
    Args:
        q, k: packed queries / keys ``(total_tokens, heads, key_dim)``.
        v: packed values ``(total_tokens, heads, value_dim)``.
        cu_seqlens: int32 cumulative sequence lengths ``(num_sequences + 1,)``,
            starting at zero, ending at ``total_tokens``, strictly increasing.
        max_seqlen: an upper bound on the sequence lengths.
        scale: multiplies the values inside the state; if omitted each sequence
            uses the reciprocal of its own length.
        eps: added to the normaliser.

    Returns:
        packed outputs ``(total_tokens, heads, value_dim)``.
    """
    if q.ndim != 3 or k.ndim != 3 or v.ndim != 3:
        raise ValueError("q, k, and v must have shape (total_tokens, heads, dim), got "
                         f"q.shape={q.shape}, k.shape={k.shape}, v.shape={v.shape}")
    if q.shape != k.shape:
        raise ValueError(f"q and k must have identical shapes, got {q.shape} and {k.shape}")
    if q.shape[:2] != v.shape[:2]:
        raise ValueError("q, k, and v must have matching token and head dimensions")
    if q.device != k.device or q.device != v.device:
        raise ValueError("q, k, and v must have the same device")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise ValueError("q, k, and v must have the same dtype")
    if not q.is_cuda:
        raise ValueError("q, k, and v must be CUDA tensors")
    if q.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError("q, k, and v must have dtype float16, bfloat16, or float32")
    if not (0 < q.shape[-1] <= 128 and 0 < v.shape[-1] <= 128):
        raise ValueError("key_dim and value_dim must be between 1 and 128")
    if cu_seqlens.ndim != 1 or cu_seqlens.numel() < 2:
        raise ValueError("cu_seqlens must have shape (num_sequences + 1,)")
    if cu_seqlens.device != q.device or cu_seqlens.dtype != torch.int32:
        raise ValueError("cu_seqlens must be an int32 tensor on the same device as q")
    if not isinstance(max_seqlen, int) or isinstance(max_seqlen, bool) or max_seqlen <= 0:
        raise ValueError("max_seqlen must be a positive integer")

    scale = None if scale is None else float(scale)
    return VarlenLinearAttnFunction.apply(q, k, v, cu_seqlens, max_seqlen, scale, eps)
