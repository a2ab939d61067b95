"""Sequence sharding on real GPUs: two NCCL ranks each hold half of the tokens; outputs and
gradients must match the single-GPU operator on the whole sequence.  Needs two GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flash_bla.ops.linear_attn.fused import linear_attention
        from flash_bla.ops.simple_la.fused import simple_la
        from flash_bla.ops.sharded import seq_sharded_linear_attention, seq_sharded_simple_la
        from flash_bla.ops import sharded
        from flash_bla import _C
        from flash_bla.ops.linear_attn.decoupled import decoupled_la
        from flash_bla.ops.sharded import seq_sharded_decoupled_la
        errs = {}
        # every case once with the peer-memory state exchange and once with NCCL's all-reduce
        cases = (("linear", 64, 64, torch.bfloat16), ("simple", 128, 128, torch.bfloat16),
                 ("linear_128x64", 128, 64, torch.float16), ("decoupled", 64, 64, torch.bfloat16),
                 ("simple_64x128", 64, 128, torch.bfloat16), ("linear_f32", 32, 32, torch.float32),
                 ("linear_narrow", 32, 48, torch.bfloat16))          # head dims below the tensor-core tiles
        for mode, (name, DK, DV, dtype) in [(m, c) for m in ("1", "0") for c in cases]:
            os.environ["FBLA_PEER_EXCHANGE"] = mode
            g = torch.Generator(device="cuda").manual_seed(7)
            B, H, T = 2, 5, 4096 * world                  # 10 units: they do not divide evenly over 4 or 8 ranks
            n_qk = 4 if name == "decoupled" else 2
            qk = [torch.rand(B, H, T, DK, device="cuda", generator=g).add_(0.1).to(dtype) for _ in range(n_qk)]
            v = torch.randn(B, H, T, DV, device="cuda", generator=g).to(dtype)
            do = torch.randn(B, H, T, DV, device="cuda", generator=g).to(dtype)
            assert T % world == 0
            sl = slice(rank * T // world, (rank + 1) * T // world)
            xs = [x[:, :, sl].contiguous().requires_grad_() for x in qk + [v]]
            full = [x.clone().requires_grad_() for x in qk + [v]]
            sharded_fn, plain_fn = {"linear": (seq_sharded_linear_attention, linear_attention),
                                    "simple": (seq_sharded_simple_la, simple_la),
                                    "decoupled": (seq_sharded_decoupled_la, decoupled_la)}[name.split("_")[0]]
            o = sharded_fn(*xs)
            o_ref = plain_fn(*full)
            o.backward(do[:, :, sl].contiguous())
            o_ref.backward(do)
            grads = [x.grad.clone() for x in xs]
            # The sharded and the single-GPU run add the fp32 state in a different order, so 16-bit
            # outputs may land on neighbouring representable values: allow one unit in the last
            # place of the output type plus 0.2 % of the RMS (fp32: 1e-4 of the RMS).
            ulp = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10, torch.float32: 0.0}[dtype]
            worst = 0.0
            for a, b in [(o, o_ref[:, :, sl])] + [(x.grad, f.grad[:, :, sl]) for x, f in zip(xs, full)]:
                a, b = a.float(), b.float()
                rms = b.pow(2).mean().sqrt().item()
                slack = ulp * b.abs() + (2e-3 if ulp else 1e-4) * rms
                worst = max(worst, ((a - b).abs() / slack).max().item())
            errs[f"{name}/peer={mode}"] = worst
            if mode == "1":     # three steps in a row: the two exchange buffers alternate, the epochs advance
                for _ in range(3):
                    for x in xs:
                        x.grad = None
                    o2 = sharded_fn(*xs)
                    o2.backward(do[:, :, sl].contiguous())
                    same = torch.equal(o2, o) and all(torch.equal(x.grad, g) for x, g in zip(xs, grads))
                    errs[f"{name}/repeat"] = max(errs.get(f"{name}/repeat", 0.0), 0.0 if same else 2.0)
        # piecewise sparse attention: the (batch, head) pairs are split over the ranks without communication;
        # a rank's share must equal the same pairs of the whole problem (the forward bit for bit, the gradients up
        # to the order of the fp32 atomics that collect the block-statistics terms)
        from flash_bla.ops.piecewise_attn.kernel import piecewise_sparse_attention
        from flash_bla.ops.sharded import shard_units
        g = torch.Generator(device="cuda").manual_seed(9)
        n_units = 6
        q, k, v, do = (torch.randn(1, n_units, 1000, 128, device="cuda", generator=g).bfloat16() for _ in range(4))
        mine = shard_units(n_units, world, rank)
        if len(mine) > 0:
            lo, hi = mine[0], mine[-1] + 1
            part = [x[:, lo:hi].contiguous().requires_grad_() for x in (q, k, v)]
            whole = [x.clone().requires_grad_() for x in (q, k, v)]
            o = piecewise_sparse_attention(*part, density=0.2, block_size=64)
            o_ref = piecewise_sparse_attention(*whole, density=0.2, block_size=64)
            o.backward(do[:, lo:hi].contiguous())
            o_ref.backward(do)
            errs["piecewise/forward"] = 0.0 if torch.equal(o, o_ref[:, lo:hi]) else 2.0
            worst = 0.0
            for a, f in zip(part, whole):
                a, b = a.grad.float(), f.grad[:, lo:hi].float()
                slack = 2.0 ** -7 * b.abs() + 2e-3 * b.pow(2).mean().sqrt().item()
                worst = max(worst, ((a - b).abs() / slack).max().item())
            errs["piecewise/backward"] = worst
        kinds = {type(e).__name__ for e in sharded._exchanges.values() if e is not None}
        errs["fused_path_used"] = 0.0 if "_FusedExchange" in kinds else 2.0
        errs["peer_path_used"] = 0.0 if "_PeerExchange" in kinds else 2.0
        errs["device_status"] = float(_C.lib().fbla_device_status())
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


# FBLA_TEST_WORLD=4 or 8 runs the same check on more ranks (a box with that many GPUs)
_WORLD = int(os.environ.get("FBLA_TEST_WORLD", "2"))


@pytest.mark.skipif(torch.cuda.device_count() < _WORLD, reason="needs %d GPUs" % _WORLD)
def test_two_gpu_sequence_sharding_matches_one_gpu():
    world = _WORLD
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert len(ret) == world
    for errs in ret.values():
        assert all(e <= 1.0 for e in errs.values()), dict(ret)
