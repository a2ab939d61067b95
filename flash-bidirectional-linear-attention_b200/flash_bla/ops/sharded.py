"""Multi-GPU use of the operators (one process per GPU, ``torch.distributed``).

The reference runs on one GPU only.  Because the state of bidirectional linear
attention is a dk x dv matrix per (batch, head) whatever the sequence length, a
sequence split along T over the ranks of a process group needs exactly one
exchange per direction:

    forward : local [S_r | sum k_r]  --sum over ranks-->  global state  -> local o
    backward: local dq and [dS_r | sum dz q_r]  --sum over ranks-->  -> local dk, dv

On NCCL groups of GPUs of one node the sum is ONE kernel that reads the peers' memory over NVLink
(symmetric memory, plain peer loads): for the shapes the tensor-core kernels serve it adds the
per-segment pieces the reducing pass left, without a reduction kernel in between, and from three ranks
on sums each unit once at its owner (``fbla_seq_sharded_*``); other shapes use the one-round sum of the
reduced states (``fbla_peer_state_sum``).  That is the default up to four ranks; beyond (where NCCL's
in-switch reduction measured faster), on other groups, or with ``FBLA_PEER_EXCHANGE=0``, the sum is
``all_reduce(SUM)``; ``FBLA_PEER_EXCHANGE=1`` forces the kernels.

Every rank must make the same calls in the same order with the same local shapes.  A kernel waits
for its peers for at most ``FBLA_PEER_WAIT_MS`` (default 5000); ranks that may drift further apart
(one of them writing a checkpoint) should meet at ``dist.barrier()`` before the call.

The key mean and the default scale use the GLOBAL sequence length.  Batch, head
and whole-sequence (varlen) sharding need no communication at all: each rank
calls the plain operator on its own slice; ``partition_sequences`` balances packed
sequences over ranks by token count.
"""
import os
import warnings
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


def _symm():
    # peers are reached with plain loads and stores; no multicast object is needed or wanted
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch.distributed._symmetric_memory as symm
    return symm


class _PeerExchange:
    """State sum over the GPUs of one node through peer memory (``fbla_peer_state_sum``).

    Two symmetric-memory buffers of ``n`` floats (used alternately) and one array of flag words per
    rank, all mapped by every peer.  Not safe for exchanges issued on several streams at once.
    """

    def __init__(self, group, device, n):
        import ctypes
        from flash_bla import _C
        symm = _symm()
        self._C = _C
        self.n = n
        self.data = symm.empty(2 * n, dtype=torch.float32, device=device)
        self.flags = symm.empty(64, dtype=torch.int32, device=device)
        self.flags.zero_()
        hd = symm.rendezvous(self.data, group)
        hf = symm.rendezvous(self.flags, group)
        self.world, self.rank = hd.world_size, hd.rank
        if self.world > 16:
            raise RuntimeError("at most 16 ranks")
        self._hd, self._hf = hd, hf
        arr = ctypes.c_void_p * self.world
        self._bufs = [arr(*[int(p) + b * n * 4 for p in hd.buffer_ptrs]) for b in (0, 1)]
        self._flags = arr(*[int(p) for p in hf.buffer_ptrs])
        self.epoch = 0
        torch.cuda.synchronize(device)

    def buffer(self):
        """The buffer the next exchange reads; the producing pass writes the local state into it."""
        b = (self.epoch + 1) & 1
        return self.data[b * self.n:(b + 1) * self.n]

    def sum(self):
        self.epoch += 1
        out = torch.empty(self.n, dtype=torch.float32, device=self.data.device)
        with self._C.device_guard(out):
            rc = self._C.lib().fbla_peer_state_sum(self.world, self.rank, self._bufs[self.epoch & 1], self._flags,
                                                   self.n, self.epoch, out.data_ptr(), self._C.stream_of(out))
        self._C.check(rc)
        return out


class _FusedExchange:
    """Buffers of the piece-level exchange (``fbla_seq_sharded_*``) for one problem shape: two (piece
    buffer, owner-sum buffer) pairs used alternately and one array of flag words, in symmetric memory
    that every peer has mapped."""

    def __init__(self, group, device, prob):
        import ctypes
        from flash_bla import _C
        symm = _symm()
        L = _C.lib()
        world = dist.get_world_size(group)
        self.n = int(L.fbla_state_floats(ctypes.byref(prob)))
        self.n_parts = int(L.fbla_seq_sharded_part_floats(ctypes.byref(prob)))
        if self.n <= 0 or self.n_parts <= 0:
            raise RuntimeError("the fused exchange does not serve this problem")
        per = self.n_parts + self.n
        self.data = symm.empty(2 * per, dtype=torch.float32, device=device)
        self.flags = symm.empty(64, dtype=torch.int32, device=device)
        self.flags.zero_()
        hd = symm.rendezvous(self.data, group)
        hf = symm.rendezvous(self.flags, group)
        self.world, self.rank = hd.world_size, hd.rank
        self._hd, self._hf = hd, hf
        arr = ctypes.c_void_p * self.world
        self._tables = []
        self._groups = []
        for b in (0, 1):
            parts = arr(*[int(p) + b * per * 4 for p in hd.buffer_ptrs])
            full = arr(*[int(p) + (b * per + self.n_parts) * 4 for p in hd.buffer_ptrs])
            flags = arr(*[int(p) for p in hf.buffer_ptrs])
            g = _C.PeerGroup()
            g.world, g.rank, g.epoch, g.reserved = self.world, self.rank, 0, 0
            g.parts = ctypes.cast(parts, ctypes.POINTER(ctypes.c_void_p))
            g.full = ctypes.cast(full, ctypes.POINTER(ctypes.c_void_p))
            g.flags = ctypes.cast(flags, ctypes.POINTER(ctypes.c_void_p))
            self._tables.append((parts, full, flags))          # keep the arrays alive
            self._groups.append(g)
        self.epoch = 0
        torch.cuda.synchronize(device)

    def begin(self):
        """Starts the next exchange: the group both of its passes are called with."""
        self.epoch += 1
        g = self._groups[self.epoch & 1]
        g.epoch = self.epoch
        return g


_exchanges = {}


# Up to this many ranks the library's own exchange kernel is used by default; beyond it NCCL's
# all-reduce.  Measured on B200 (bf16 B8-H16-D64, 32768 tokens per rank, ms per forward + backward,
# own kernel / NCCL): 2 ranks 1.041 / 1.043, 4 ranks 1.073 / 1.069, 8 ranks 1.111 / 1.089 -- NCCL adds
# inside the NVSwitch, which two rounds of flags and peer loads do not beat at 8 ranks.
_PEER_EXCHANGE_MAX_WORLD = 4


def _peer_capable(group, device):
    """FBLA_PEER_EXCHANGE: "1" = the library's exchange kernels on any NCCL group of one node, "0" = always
    ``all_reduce``; unset = the kernels up to four ranks, ``all_reduce`` beyond."""
    if not (dist.is_available() and dist.is_initialized()) or device.type != "cuda":
        return False
    world = dist.get_world_size(group)
    if world < 2 or dist.get_backend(group) != "nccl":
        return False
    mode = os.environ.get("FBLA_PEER_EXCHANGE", "auto")
    if mode == "0":
        return False
    return mode == "1" or world <= _PEER_EXCHANGE_MAX_WORLD


def _agreed(make, group, device, same=()):
    """``make()`` on every rank; the result, or None when it failed on ANY rank or the integers in
    ``same`` differ between ranks (decided collectively, so that all ranks take the same path)."""
    ex = None
    try:
        ex = make()
    except Exception as e:          # noqa: BLE001 - any failure means "use the library all-reduce"
        warnings.warn(f"peer-memory state exchange unavailable ({type(e).__name__}: {e}); using all_reduce")
    vals = [1 if ex is not None else 0]
    for x in same:
        vals += [int(x), -int(x)]
    t = torch.tensor(vals, device=device, dtype=torch.int64)
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)   # also: every rank's flags are zeroed by now
    t = t.tolist()
    ok = t[0] == 1 and all(t[1 + 2 * i] == -t[2 + 2 * i] for i in range(len(same)))
    return ex if ok else None


def _peer_exchange(group, device, n):
    """The exchange object for (group, device, state size), or None when the group is not an NCCL
    group of more than one GPU rank, the switch ``FBLA_PEER_EXCHANGE=0`` is set, the state size is
    not a multiple of four floats, or setting it up failed on any rank."""
    if not _peer_capable(group, device) or n % 4 != 0 or dist.get_world_size(group) > 16:
        return None
    key = (id(group) if group is not None else 0, device.index, n)
    if key not in _exchanges:
        grp = group if group is not None else dist.group.WORLD
        _exchanges[key] = _agreed(lambda: _PeerExchange(grp, device, n), group, device)
    return _exchanges[key]


def _fused_exchange(group, prob, tensors):
    """The in-kernel exchange for this problem, or None when it does not apply (not an NCCL group of
    2 to 8 GPUs, a shape the tensor-core kernels do not serve, ranks that disagree on the local
    shape, or a set-up failure on any rank)."""
    like = tensors[0]
    if not hasattr(_backend, "sharded_fwd_state") or not _peer_capable(group, like.device):
        return None
    if dist.get_world_size(group) > 8 or not _backend.sharded_supported(prob):
        return None
    key = (id(group) if group is not None else 0, like.device.index, "fused", prob.dtype, prob.batch, prob.heads,
           prob.seq_len, prob.dk, prob.dv, prob.normalize)
    if key not in _exchanges:
        grp = group if group is not None else dist.group.WORLD
        sms = torch.cuda.get_device_properties(like.device).multi_processor_count
        _exchanges[key] = _agreed(lambda: _FusedExchange(grp, like.device, prob), group, like.device,
                                  same=(prob.seq_len, prob.batch, prob.heads, sms))
    return _exchanges[key]


def _aligned(*tensors):
    """Contiguous tensors whose storage starts on a 16-byte boundary (what the tensor-core kernels
    need); a view at an odd offset is copied."""
    return [t if t is None or t.data_ptr() % 16 == 0 else t.clone() for t in tensors]


def _narrow(prob, *tensors):
    """Head dims below the tensor-core tiles (multiples of 16 that are not 64 / 128): the passes' narrow route,
    which reads the tensors at their own width and wants them 16-byte aligned (CUDA tensors only)."""
    if tensors[0].is_cuda and _passes.use_narrow(prob):
        return _aligned(*tensors)
    return tensors


def _summed_state(produce, prob, like, group):
    """Runs ``produce(out)`` (a state pass; ``out`` None = allocate) and returns the sum of the
    resulting states over the group."""
    n = _backend.state_floats(prob) if hasattr(_backend, "state_floats") else 0
    ex = _peer_exchange(group, like.device, n) if n else None
    if ex is None:
        return _all_reduce(produce(None), group)
    produce(ex.buffer())
    return ex.sum()


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
        q, k, v = _narrow(prob, q, k, v)
        fx = _fused_exchange(group, prob, (q, k, v))
        if fx is not None:
            q, k, v = _aligned(q, k, v)
            grp = fx.begin()
            _backend.sharded_fwd_state(prob, k, v, grp)
            state = _backend.sharded_exchange(prob, grp, q)
            o = _backend.fwd_out(op, prob, q, state, torch.empty_like(v))
        else:
            state = _summed_state(lambda out: _backend.fwd_state(op, prob, k, v, out=out), prob, q, group)
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
        do, = _narrow(prob, do)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        fx = _fused_exchange(group, prob, (q, k, v))
        if fx is not None:
            do, = _aligned(do)
            grp = fx.begin()
            _backend.sharded_bwd_state(prob, q, do, state, grp, dq)
            _backend.bwd_in(op, prob, k, v, _backend.sharded_exchange(prob, grp, q), dk, dv)
        else:
            dstate = _summed_state(lambda out: _backend.bwd_state(op, prob, q, do, state, dq, out=out), prob, q, group)
            _backend.bwd_in(op, prob, k, v, dstate, dk, dv)
        return dq, dk, dv, None, None, None, None, None


class _SeqShardedDecoupled(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, q_rope, k_rope, v, scale, eps, norm_len, group):
        q, k, q_rope, k_rope, v = (x.contiguous() for x in (q, k, q_rope, k_rope, v))
        B, H, L, K = q.shape
        prob = _backend.make_problem(q, batch=B, heads=H, seq_len=L, dk=K, dv=v.shape[-1], normalize=True,
                                     scale=scale, eps=eps, norm_len=norm_len, flags=_backend.default_flags())
        fx = _fused_exchange(group, prob, (q, k, v)) if (K, v.shape[-1]) == (64, 64) else None
        if fx is not None:
            q, k, q_rope, k_rope, v = _aligned(q, k, q_rope, k_rope, v)
            grp = fx.begin()
            _backend.sharded_fwd_state(prob, k, v, grp, k_rope=k_rope)
            state = _backend.sharded_exchange(prob, grp, q)
            o = _backend.fwd_out("decoupled_la", prob, q, state, torch.empty_like(v), q_rope=q_rope)
        else:
            state = _summed_state(lambda out: _backend.fwd_state("decoupled_la", prob, k, v, k_rope=k_rope, out=out),
                                  prob, q, group)
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
        dk, dk_rope, dv = torch.empty_like(k_rope), torch.empty_like(k_rope), torch.empty_like(v)
        fx = _fused_exchange(group, prob, (q, k_rope, v)) if (K, v.shape[-1]) == (64, 64) else None
        if fx is not None:
            do, = _aligned(do)
            grp = fx.begin()
            _backend.sharded_bwd_state(prob, q, do, state, grp, dq, q_rope=q_rope, dq_rope=dq_rope)
            _backend.bwd_in("decoupled_la", prob, k_rope, v, _backend.sharded_exchange(prob, grp, q), dk, dv,
                            dk_rope=dk_rope)
        else:
            dstate = _summed_state(lambda out: _backend.bwd_state("decoupled_la", prob, q, do, state, dq, q_rope=q_rope,
                                                                  dq_rope=dq_rope, out=out), prob, q, group)
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
