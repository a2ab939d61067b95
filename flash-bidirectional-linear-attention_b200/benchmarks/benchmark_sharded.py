"""Where the time of a sequence-sharded forward + backward goes, per rank.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/benchmark_sharded.py [--op linear_attn|simple_la] [--seq-len T_per_rank] [--steps K]

Every rank holds T tokens of a global sequence of N*T (linear_attn: B8-H16-D64; simple_la: B4-H32-D128).
Printed per rank (medians over the steps, microseconds): CUDA-event durations of the four passes and of
the two exchange kernels of a sharded step (x_fwd between fwd_state and fwd_out, x_bwd between bwd_state
and bwd_in), and of the same four passes without any exchange (each rank on its own tokens, with the
reduction kernel the unsharded state pass runs), for comparison.
"""
import argparse
import os
import statistics
import sys

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, _PKG)

import torch
import torch.distributed as dist
import torch.nn.functional as F

from flash_bla.ops import _passes as P
from flash_bla.ops import sharded


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="linear_attn", choices=["linear_attn", "simple_la"])
    ap.add_argument("--seq-len", type=int, default=32768)
    ap.add_argument("--steps", type=int, default=40)
    args = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    normalize = args.op == "linear_attn"
    B, H, D = (8, 16, 64) if normalize else (4, 32, 128)
    T = args.seq_len
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    mk = lambda pos: ((F.elu(torch.randn(B, H, T, D, device=dev, generator=g)) + 1) if pos
                      else torch.randn(B, H, T, D, device=dev, generator=g)).bfloat16()
    q, k, v, do = mk(normalize), mk(normalize), mk(False), mk(False)
    Tg = T * world
    scale = 1.0 / Tg if normalize else D ** -0.5
    prob = P.make_problem(q, batch=B, heads=H, seq_len=T, dk=D, dv=D, normalize=normalize, scale=scale,
                          eps=1e-6 if normalize else 0.0, norm_len=Tg if normalize else 0)
    fx = sharded._fused_exchange(None, prob, (q, k, v)) if world > 1 else None
    o, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    names = ["fwd_state", "fwd_out", "bwd_state", "bwd_in"]
    op = args.op

    def step(ev, use_exchange):
        ev[0].record()
        if use_exchange:
            grp = fx.begin()
            P.sharded_fwd_state(prob, k, v, grp)
            ev[1].record()
            state = P.sharded_exchange(prob, grp, q)
            ev[2].record()
            P.fwd_out(op, prob, q, state, o)
            ev[3].record()
            grp = fx.begin()
            P.sharded_bwd_state(prob, q, do, state, grp, dq)
            ev[4].record()
            dstate = P.sharded_exchange(prob, grp, q)
            ev[5].record()
            P.bwd_in(op, prob, k, v, dstate, dk, dv)
        else:
            st = P.fwd_state(op, prob, k, v)
            ev[1].record()
            ev[2].record()
            P.fwd_out(op, prob, q, st, o)
            ev[3].record()
            dst = P.bwd_state(op, prob, q, do, st, dq)
            ev[4].record()
            ev[5].record()
            P.bwd_in(op, prob, k, v, dst, dk, dv)
        ev[6].record()

    cols = ["fwd_state", "x_fwd", "fwd_out", "bwd_state", "x_bwd", "bwd_in"]

    def run(use_exchange):
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(7)] for _ in range(args.steps + 5)]
        dist.barrier()
        torch.cuda.synchronize()
        for ev in evs:
            step(ev, use_exchange)
        torch.cuda.synchronize()
        per = {n: statistics.median(ev[i].elapsed_time(ev[i + 1]) * 1e3 for ev in evs[5:]) for i, n in enumerate(cols)}
        per["step"] = statistics.median(ev[0].elapsed_time(ev[6]) * 1e3 for ev in evs[5:])
        return per

    loc = run(False)
    lines = [f"rank {rank}: local    " + "  ".join(f"{n} {loc[n]:7.1f}" for n in cols + ["step"])]
    if fx is not None:
        shd = run(True)
        lines.append(f"rank {rank}: sharded  " + "  ".join(f"{n} {shd[n]:7.1f}" for n in cols + ["step"]))
    gathered = [None] * world
    dist.all_gather_object(gathered, lines)
    if rank == 0:
        print(f"# {args.op} bf16 B{B}-H{H}-D{D}, T = {T} per rank, {world} ranks, microseconds (medians of {args.steps} steps)")
        for ls in gathered:
            for ln in ls:
                print(ln)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
