"""Where the time of a sequence-sharded forward + backward goes, per rank.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/benchmark_sharded.py [--op linear_attn|simple_la] [--seq-len T_per_rank] [--steps K]

Every rank holds T tokens of a global sequence of N*T (linear_attn: B8-H16-D64; simple_la: B4-H32-D128).
Printed per rank (medians over the steps, microseconds):

  kernels   : CUDA-event durations of the four passes; the two consuming passes (fwd_out, bwd_in) contain
              the exchange, so their excess over the 1-GPU figure is what sharding costs;
  exchange  : from the library's timestamp trace (fbla_debug_peer_trace), inside the consuming pass:
                wait1 = gather entered -> pieces of all ranks in place   (skew between ranks + signal latency)
                sum   = -> own sums stored in every rank's copy          (local adds, peer stores, fence)
                wait2 = -> sums of all ranks in place                    (slowest rank's sum + signal latency)
                copy  = -> private copy of the state written             (forward only)
  local     : the same four passes without any exchange (each rank on its own tokens), for comparison.
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

from flash_bla import _C
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
    trace = torch.zeros(256 * 16, dtype=torch.int64, device=dev)
    if fx is not None:
        _C.lib().fbla_debug_peer_trace(trace.data_ptr())
    o, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    state = torch.empty(P.state_floats(prob), dtype=torch.float32, device=dev)
    names = ["fwd_state", "fwd_out", "bwd_state", "bwd_in"]

    def step(ev, use_exchange):
        ev[0].record()
        if use_exchange:
            grp = fx.begin()
            P.sharded_fwd_state(prob, k, v, grp)
            ev[1].record()
            P.sharded_fwd_out(prob, q, grp, o, state)
            ev[2].record()
            grp = fx.begin()
            P.sharded_bwd_state(prob, q, do, state, grp, dq)
            ev[3].record()
            P.sharded_bwd_in(prob, k, v, grp, dk, dv)
        else:
            op = args.op
            st = P.fwd_state(op, prob, k, v)
            ev[1].record()
            P.fwd_out(op, prob, q, st, o)
            ev[2].record()
            dst = P.bwd_state(op, prob, q, do, st, dq)
            ev[3].record()
            P.bwd_in(op, prob, k, v, dst, dk, dv)
        ev[4].record()

    def run(use_exchange):
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(args.steps + 5)]
        dist.barrier()
        torch.cuda.synchronize()
        for ev in evs:
            step(ev, use_exchange)
        torch.cuda.synchronize()
        per = {n: statistics.median(ev[i].elapsed_time(ev[i + 1]) * 1e3 for ev in evs[5:]) for i, n in enumerate(names)}
        per["step"] = statistics.median(ev[0].elapsed_time(ev[4]) * 1e3 for ev in evs[5:])
        return per

    loc = run(False)
    lines = [f"rank {rank}: local    " + "  ".join(f"{n} {loc[n]:7.1f}" for n in names + ["step"])]
    if fx is not None:
        shd = run(True)
        lines.append(f"rank {rank}: sharded  " + "  ".join(f"{n} {shd[n]:7.1f}" for n in names + ["step"]))
        t = trace.cpu().view(256, 16)
        last = fx.epoch
        rows = {"fwd": [], "bwd": []}
        for e in range(max(1, last - 2 * args.steps + 1), last + 1):
            r = t[e & 255]
            if r[8] == 0 or r[11] == 0:
                continue
            ph = [(r[9] - r[8]).item() / 1e3, (r[10] - r[9]).item() / 1e3, (r[11] - r[10]).item() / 1e3,
                  (r[12] - r[11]).item() / 1e3 if r[12] else 0.0]
            rows["fwd" if e % 2 == 1 else "bwd"].append(ph)      # odd epochs are forward exchanges here
        for d, rr in rows.items():
            if rr:
                med = [statistics.median(x[i] for x in rr) for i in range(4)]
                lines.append(f"rank {rank}: exchange {d}  wait1 {med[0]:6.1f}  sum {med[1]:6.1f}  wait2 {med[2]:6.1f}  "
                             f"copy {med[3]:6.1f}   (n={len(rr)})")
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
