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
        errs = {}
        # every case once with the peer-memory state exchange and once with NCCL's all-reduce
        for mode, (name, D, dtype) in [(m, c) for m in ("1", "0") for c in (
                ("linear", 64, torch.bfloat16), ("simple", 128, torch.bfloat16), ("linear_f32", 32, torch.float32))]:
            os.environ["FBLA_PEER_EXCHANGE"] = mode
            g = torch.Generator(device="cuda").manual_seed(7)
            B, H, T = 2, 4, 2048
            q = torch.rand(B, H, T, D, device="cuda", generator=g).add_(0.1).to(dtype)
            k = torch.rand(B, H, T, D, device="cuda", generator=g).add_(0.1).to(dtype)
            v = torch.randn(B, H, T, D, device="cuda", generator=g).to(dtype)
            do = torch.randn(B, H, T, D, device="cuda", generator=g).to(dtype)
            sl = slice(rank * T // world, (rank + 1) * T // world)
            xs = [x[:, :, sl].contiguous().requires_grad_() for x in (q, k, v)]
            full = [x.clone().requires_grad_() for x in (q, k, v)]
            if name.startswith("linear"):
                o = seq_sharded_linear_attention(*xs)
                o_ref = linear_attention(*full)
            else:
                o = seq_sharded_simple_la(*xs)
                o_ref = simple_la(*full)
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
                    o2 = (seq_sharded_linear_attention if name.startswith("linear") else seq_sharded_simple_la)(*xs)
                    o2.backward(do[:, :, sl].contiguous())
                    same = torch.equal(o2, o) and all(torch.equal(x.grad, g) for x, g in zip(xs, grads))
                    errs[f"{name}/repeat"] = max(errs.get(f"{name}/repeat", 0.0), 0.0 if same else 2.0)
        errs["peer_path_used"] = 0.0 if any(e is not None for e in sharded._exchanges.values()) else 2.0
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
