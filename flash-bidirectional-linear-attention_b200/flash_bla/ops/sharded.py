"""Multi-GPU use of the operators (one process per GPU, ``torch.distributed``).

The reference runs on one GPU only.  Because the state of bidirectional linear
attention is a dk x dv matrix per (batch, head) whatever the sequence length, a
sequence split along T over the ranks of a process group needs exactly one
exchange per direction:

    forward : local [S_r | sum k_r]  --all_reduce(SUM)-->  global state  -> local o
    backward: local dq and [dS_r | sum dz q_r]  --all_reduce(SUM)-->  -> local dk, dv

The key mean and the default scale use the GLOBAL sequence length.  Batch, head
and whole-sequence (varlen) sharding need no communication at all: each rank
calls the plain operator on its own slice; ``partition_sequences`` balances packed
sequences over ranks by token count.
"""
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from flash_bla.ops import _passes

# The four passes are looked up through this name so that the CPU tests of the
# multi-rank logic can substitute a host-side implementation.
_backend = _passes


def _global_len(local_len, group, global_len):
    if global_len is not None:
        return int(global_len)
    return int(local_len) * dist.get_world_size(group)


def _all_reduce(t, group):
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


class _SeqSharded(torch.autograd.Function):
    """linear_attention / simple_la on a T-shard; ``normalize`` selects which."""

    @staticmethod
    def forward(ctx, q, k, v, scale, eps, norm_len, normalize, group):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        B, H, L, K = q.shape
        op = "linear_attn" if normalize else "simple_la"
        prob = _backend.make_problem(q, batch=B, heads=H, seq_len=L, dk=K, dv=v.shape[-1],
                                     normalize=normalize, scale=scale, eps=eps, norm_len=norm_len,
                                     flags=_backend.default_flags())
        state = _all_reduce(_backend.fwd_state(op, prob, k, v), group)
        o = _backend.fwd_out(op, prob, q, state, torch.empty_like(v))
        ctx.save_for_backward(q, k, v, state)
        ctx.args = (scale, eps, norm_len, normalize, group)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, state = ctx.saved_tensors
        scale, eps, norm_len, normalize, group = ctx.args
        do = do.contiguous()
        B, H, L, K = q.shape
        op = "linear_attn" if normalize else "simple_la"
        prob = _backend.make_problem(q, batch=B, heads=H, seq_len=L, dk=K, dv=v.shape[-1],
                                     normalize=normalize, scale=scale, eps=eps, norm_len=norm_len,
                                     flags=_backend.default_flags())
        dq = torch.empty_like(q)
        dstate = _all_reduce(_backend.bwd_state(op, prob, q, do, state, dq), group)
        dk, dv = torch.empty_like(k), torch.empty_like(v)
        _backend.bwd_in(op, prob, k, v, dstate, dk, dv)
        return dq, dk, dv, None, None, None, None, None


class _SeqShardedDecoupled(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, q_rope, k_rope, v, scale, eps, norm_len, group):
        q, k, q_rope, k_rope, v = (x.contiguous() for x in (q, k, q_rope, k_rope, v))
        B, H, L, K = q.shape
        prob = _backend.make_problem(q, batch=B, heads=H, seq_len=L, dk=K, dv=v.shape[-1], normalize=True,
                                     scale=scale, eps=eps, norm_len=norm_len, flags=_backend.default_flags())
        state = _all_reduce(_backend.fwd_state("decoupled_la", prob, k, v, k_rope=k_rope), group)
        o = _backend.fwd_out("decoupled_la", prob, q, state, torch.empty_like(v), q_rope=q_rope)
        ctx.save_for_backward(q, q_rope, k_rope, v, state)
        ctx.args = (scale, eps, norm_len, group)
        return o

    @staticmethod
    def backward(ctx, do):
        q, q_rope, k_rope, v, state = ctx.saved_tensors
        scale, eps, norm_len, group = ctx.args
        do = do.contiguous()
        B, H, L, K = q.shape
        prob = _backend.make_problem(q, batch=B, heads=H, seq_len=L, dk=K, dv=v.shape[-1], normalize=True,
                                     scale=scale, eps=eps, norm_len=norm_len, flags=_backend.default_flags())
        dq, dq_rope = torch.empty_like(q), torch.empty_like(q_rope)
        dstate = _all_reduce(_backend.bwd_state("decoupled_la", prob, q, do, state, dq, q_rope=q_rope,
                                                dq_rope=dq_rope), group)
        dk, dk_rope, dv = torch.empty_like(k_rope), torch.empty_like(k_rope), torch.empty_like(v)
        _backend.bwd_in("decoupled_la", prob, k_rope, v, dstate, dk, dv, dk_rope=dk_rope)
        return dq, dk, dq_rope, dk_rope, dv, None, None, None, None


def seq_sharded_linear_attention(q, k, v, scale: Optional[float] = None, eps: float = 1e-6, group=None,
                                 global_len: Optional[int] = None):
    """``linear_attention`` where q, k, v ``(B, H, L_local, D)`` hold this rank's slice
    of the sequence.  ``global_len`` defaults to ``L_local * world_size``."""
    n = _global_len(q.shape[-2], group, global_len)
    if scale is None:
        scale = 1.0 / n
    return _SeqSharded.apply(q, k, v, scale, eps, n, True, group)


def seq_sharded_simple_la(q, k, v, scale: Optional[float] = None, group=None):
    """``simple_la`` on this rank's slice of the sequence."""
    if scale is None:
        scale = q.shape[-1] ** -0.5
    return _SeqSharded.apply(q, k, v, scale, 0.0, 0, False, group)


def seq_sharded_decoupled_la(q, k, q_rope, k_rope, v, scale: Optional[float] = None, eps: float = 1e-6,
                             group=None, global_len: Optional[int] = None):
    """``decoupled_la`` on this rank's slice of the sequence."""
    n = _global_len(q.shape[-2], group, global_len)
    if scale is None:
        scale = 1.0 / n
    return _SeqShardedDecoupled.apply(q, k, q_rope, k_rope, v, scale, eps, n, group)


def partition_sequences(lengths: Sequence[int], world_size: int) -> List[List[int]]:
    """Assign whole packed sequences to ranks, balancing token counts (longest first
    onto the lightest rank).  Returns, per rank, the sorted sequence indices it owns;
    each rank then packs its own sequences and calls ``varlen_linear_attention``."""
    if world_size < 1:
        raise ValueError("world_size must be positive")
    owners: List[List[int]] = [[] for _ in range(world_size)]
    load = [0] * world_size
    for i in sorted(range(len(lengths)), key=lambda j: (-int(lengths[j]), j)):
        r = min(range(world_size), key=lambda x: (load[x], x))
        owners[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(o) for o in owners]


def shard_units(n_units: int, world_size: int, rank: int) -> range:
    """Contiguous block of (batch, head) units owned by ``rank`` (no communication)."""
    base, rem = divmod(n_units, world_size)
    lo = rank * base + min(rank, rem)
    return range(lo, lo + base + (1 if rank < rem else 0))
