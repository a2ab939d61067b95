"""Multi-rank logic of the sequence-sharded wrappers, on CPU: two gloo ranks, each holding
half of the sequence, the four passes replaced by the host-side stand-in.  Checks that the
wrappers reproduce the single-device operator (oracle) on the concatenated sequence."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import bla_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import host_passes
        from flash_bla.ops import sharded
        sharded._backend = host_passes
        torch.manual_seed(0)                                   # every rank builds the full problem
        B, H, T, K, V = 2, 2, 48, 8, 6
        q, k, qr, kr = (torch.rand(B, H, T, K, dtype=torch.float64) + 0.1 for _ in range(4))
        v = torch.randn(B, H, T, V, dtype=torch.float64)
        do = torch.randn(B, H, T, V, dtype=torch.float64)
        sl = slice(rank * T // world, (rank + 1) * T // world)
        loc = lambda x: x[:, :, sl].clone().requires_grad_()
        if case == "linear":
            xs = [loc(q), loc(k), loc(v)]
            o = sharded.seq_sharded_linear_attention(*xs, eps=1e-6)
            ref_o = O.linear_attn_fwd(q, k, v)
            ref_g = O.linear_attn_bwd(q, k, v, do)
        elif case == "linear_scale":
            xs = [loc(q), loc(k), loc(v)]
            o = sharded.seq_sharded_linear_attention(*xs, scale=0.37, eps=1e-4, global_len=T)
            ref_o = O.linear_attn_fwd(q, k, v, 0.37, 1e-4)
            ref_g = O.linear_attn_bwd(q, k, v, do, 0.37, 1e-4)
        elif case == "simple":
            xs = [loc(q), loc(k), loc(v)]
            o = sharded.seq_sharded_simple_la(*xs)
            ref_o = O.simple_la_fwd(q, k, v)
            ref_g = O.simple_la_bwd(q, k, v, do)
        else:
            xs = [loc(q), loc(k), loc(qr), loc(kr), loc(v)]
            o = sharded.seq_sharded_decoupled_la(*xs)
            ref_o = O.decoupled_la_fwd(q, k, qr, kr, v)
            ref_g = O.decoupled_la_bwd(q, k, qr, kr, v, do)
        o.backward(do[:, :, sl])
        err = (o.detach() - ref_o[:, :, sl]).abs().max().item()
        for x, g in zip(xs, ref_g):
            err = max(err, (x.grad - g[:, :, sl]).abs().max().item() / (g.abs().max().item() + 1e-30))
        ret[rank] = err
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", ["linear", "linear_scale", "simple", "decoupled"])
def test_two_rank_sequence_sharding_matches_single_device(case):
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), case, ret), nprocs=world, join=True)
    assert len(ret) == world
    assert max(ret.values()) < 1e-5, dict(ret)     # fp32 state packing bounds the agreement


def test_partition_sequences_balances_tokens():
    from flash_bla.ops.sharded import partition_sequences, shard_units
    lengths = [16384, 300, 9000, 256, 12000, 5000, 700, 8000]
    owners = partition_sequences(lengths, 4)
    assert sorted(i for o in owners for i in o) == list(range(len(lengths)))
    loads = [sum(lengths[i] for i in o) for o in owners]
    assert max(loads) <= 16384 and max(loads) - min(loads) <= 16384 - 8000
    assert partition_sequences([5, 5], 4) == [[0], [1], [], []]
    with pytest.raises(ValueError):
        partition_sequences(lengths, 0)
    cover = [list(shard_units(48, 8, r)) for r in range(8)]
    assert sum(cover, []) == list(range(48)) and all(len(c) == 6 for c in cover)
    assert [len(shard_units(10, 4, r)) for r in range(4)] == [3, 3, 2, 2]


def _leaver(rank, world, port, ret):
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    import host_passes
    from flash_bla.ops import sharded
    sharded._backend = host_passes
    if rank == 1:
        ret[rank] = "left"            # leaves between steps, before the exchange, with nothing in flight
        os._exit(0)
    q = torch.rand(1, 1, 8, 4, dtype=torch.float64)
    t0 = time.time()
    try:
        sharded.seq_sharded_linear_attention(q, q, q)
        ret[rank] = "returned"
    except Exception as e:            # noqa: BLE001 - whatever the process group raises
        ret[rank] = "raised after %.1f s: %s" % (time.time() - t0, type(e).__name__)


def test_a_rank_that_leaves_before_the_exchange_ends_the_others_call_with_an_error():
    """Rank 1 exits before the state exchange; rank 0's call must end with an exception within the
    process group's timeout instead of waiting for ever."""
    world = 2
    ret = mp.Manager().dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_leaver, args=(r, world, _free_port_shared(), ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    assert not alive
    assert ret.get(1) == "left"
    assert str(ret.get(0, "")).startswith("raised"), dict(ret)


_shared_port = []


def _free_port_shared():
    if not _shared_port:
        _shared_port.append(_free_port())
    return _shared_port[0]
