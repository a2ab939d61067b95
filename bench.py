"""Benchmark of the hot path: linear_attention forward + backward, bf16, B=8 H=16 D=64.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--seq-len T] [--impl reference]

One step = one forward + backward of ``linear_attention`` over one batch of synthetic
inputs (q, k = elu(N(0,1))+1, v, dO ~ N(0,1), seeded), T = 32768 tokens per rank.
With N > 1 (launched by torch.distributed.run, one rank per GPU) the sequence is
sharded along T: every rank holds 32768 tokens of a global sequence of N*32768, and
the per-head state (and its gradient) is all-reduced once per direction over NCCL --
weak scaling.  Rank 0 prints one JSON line.

``value``  : tokens/s (tokens = B * T_global) with inputs resident in HBM, public API
             (``linear_attention(...).backward(dO)``), CUDA-event timed, max over ranks.
``e2e``    : the same metric with pinned host buffers: every step copies q, k, v, dO
             host->device and o, dq, dk, dv device->host inside the timed region.
``roofline``: the slowest of the four kernels (timed one by one with CUDA events on the
             launching stream): algorithmic bytes / duration against the measured copy
             bandwidth of this machine pool.
``cpu_baseline`` / ``--impl reference``: the reference's execution model on the host
             cores -- the dense torch statement in bf16 with autograd backward -- on a
             bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "flash-bidirectional-linear-attention_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch
import torch.distributed as dist
import torch.nn.functional as F

B, H, D = 8, 16, 64
METRIC = "linear_attn fwd+bwd tokens/s (bf16, B8-H16-D64)"
UNIT = "tokens/s"
CPU_SAMPLE_BATCH = 2          # the CPU arm runs B=2 of the 8 batch rows per step
FALLBACK_HBM_GBS = 6650.0


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only)."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            pass

    def run(self):
        while self.ok and not self._stop_evt.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                get = getattr(self.nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                    self.nv.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = get(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def make_inputs(T, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    q = (F.elu(torch.randn(B, H, T, D, device=device, generator=g)) + 1).to(torch.bfloat16)
    k = (F.elu(torch.randn(B, H, T, D, device=device, generator=g)) + 1).to(torch.bfloat16)
    v = torch.randn(B, H, T, D, device=device, generator=g).to(torch.bfloat16)
    do = torch.randn(B, H, T, D, device=device, generator=g).to(torch.bfloat16)
    return q, k, v, do


# ---------------------------------------------------------------------------------------
# CPU arm: the reference's torch path on the host cores
# ---------------------------------------------------------------------------------------
def cpu_step_factory(T):
    from oracle import bla_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, do = make_inputs(T, "cpu", 0)
    q, k, v, do = (x[:CPU_SAMPLE_BATCH].contiguous() for x in (q, k, v, do))

    def step():
        O.linear_attn_torch_fwd_bwd(q, k, v, do)
    return step, CPU_SAMPLE_BATCH * T


def time_cpu(T, steps, warmup):
    step, tokens = cpu_step_factory(T)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return tokens / dt, dt


def cpu_baseline_dict(value, T):
    return {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "host_cpus": os.cpu_count(),
            "sample": f"dense torch bf16 forward + autograd backward (the reference's naive path, restated in "
                      f"oracle/) on B={CPU_SAMPLE_BATCH} of the {B} batch rows, H={H}, T={T}, D={D} per step"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = args.seq_len
    value, dt = time_cpu(T, args.steps, max(1, args.warmup))
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"linear_attn fwd+bwd bf16 B{B}-H{H}-D{D} T={T}, CPU sample "
                                   f"B={CPU_SAMPLE_BATCH}"},
            "cpu_baseline": cpu_baseline_dict(value, T),
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------
def run_ours(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"

    from flash_bla import _C
    from flash_bla.ops import _passes as P
    from flash_bla.ops.linear_attn.fused import linear_attention
    from flash_bla.ops.sharded import seq_sharded_linear_attention

    T = args.seq_len                      # tokens per rank
    T_global = T * world
    tokens = B * T_global
    q, k, v, do = make_inputs(T, dev, 1000 + rank)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()

    def step():
        q.grad = k.grad = v.grad = None
        if world > 1:
            o = seq_sharded_linear_attention(q, k, v, global_len=T_global)
        else:
            o = linear_attention(q, k, v)
        o.backward(do)
        return o

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = _C.lib().fbla_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    launches = _C.lib().fbla_launch_count() - launches0
    clocks = sampler.stop()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = ms.item() / args.steps
    value = tokens / (ms_per_step * 1e-3)

    # ---- the four kernels one by one (same inputs, CUDA events on the launching stream)
    prob = P.make_problem(q, batch=B, heads=H, seq_len=T, dk=D, dv=D, normalize=True, scale=1.0 / T_global,
                          eps=1e-6, norm_len=T_global)
    path = P.kernel_path(prob)
    qd, kd, vd = q.detach(), k.detach(), v.detach()
    o_buf, dq, dk, dv = (torch.empty_like(qd) for _ in range(4))
    names = ["fwd_state", "fwd_out", "bwd_state", "bwd_in"]
    tensor_bytes = B * H * T * D * 2
    algo_bytes = {"fwd_state": 2 * tensor_bytes, "fwd_out": 2 * tensor_bytes,
                  "bwd_state": 3 * tensor_bytes, "bwd_in": 4 * tensor_bytes}
    # All repetitions are enqueued before the first synchronisation, so the host runs ahead of
    # the GPU and no launch latency leaks into an event interval; inputs (2.1 GB) exceed L2.
    reps = max(3, min(args.steps, 20))
    events = []
    for it in range(reps + 2):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        ev[0].record()
        state = P.fwd_state("linear_attn", prob, kd, vd)
        ev[1].record()
        P.fwd_out("linear_attn", prob, qd, state, o_buf)
        ev[2].record()
        dstate = P.bwd_state("linear_attn", prob, qd, do, state, dq)
        ev[3].record()
        P.bwd_in("linear_attn", prob, kd, vd, dstate, dk, dv)
        ev[4].record()
        events.append(ev)
    torch.cuda.synchronize()
    acc = {n: 0.0 for n in names}
    for ev in events[2:]:
        for i, n in enumerate(names):
            acc[n] += ev[i].elapsed_time(ev[i + 1]) / reps
    peak, peak_kind = peaks()
    passes = {n: {"ms": acc[n], "algo_gb": algo_bytes[n] / 1e9, "gbs": algo_bytes[n] / (acc[n] * 1e-3) / 1e9}
              for n in names}
    dom = max(names, key=lambda n: acc[n])
    total_gbs = sum(algo_bytes.values()) / (sum(acc.values()) * 1e-3) / 1e9
    # DRAM bytes (read + write) per launch from the ncu capture summarised in
    # profiles/ncu_linear_attn_bf16_b8h16d64.md (taken at T = 8192, proportional to T)
    ncu_traffic_at_8192 = {"fwd_state": 273.5e6, "fwd_out": 220.6e6, "bwd_state": 377.3e6, "bwd_in": 490.0e6}
    traffic = ncu_traffic_at_8192[dom] * (T / 8192.0) if (B, H, D) == (8, 16, 64) else None
    roofline = {"bound": "hbm", "kernel": dom, "achieved": passes[dom]["gbs"], "peak": peak, "unit": "GB/s",
                "frac": passes[dom]["gbs"] / peak, "traffic": traffic, "peak_kind": f"of {peak_kind}",
                "all_passes_gbs": total_gbs, "all_passes_frac": total_gbs / peak,
                "frac_of_nominal_8000": total_gbs / 8000.0}

    # ---- end to end: pinned host buffers, copies inside the timed region
    e2e_steps = max(4, min(args.steps, 8))
    host_in = [x.detach().cpu().pin_memory() for x in (q, k, v, do)]
    host_out = [torch.empty_like(h) for h in host_in]
    host_out = [h.pin_memory() for h in host_out]
    # A three-stage pipeline, as a data loader would run it: the inputs of step i+1 cross PCIe (copy stream 1)
    # while step i computes and the results of step i-1 go back (copy stream 2; PCIe is full duplex).  Every
    # step's four inputs are copied in and its four results copied out inside the timed region.
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    sets = [[torch.empty_like(qd).requires_grad_() for _ in range(3)] + [torch.empty_like(do)] for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    keep = [None, None]

    def e2e_step(i):
        b = i & 1
        dq_, dk_, dv_, do_dev = sets[b]
        with torch.cuda.stream(s_in), torch.no_grad():
            s_in.wait_event(ev_done[b])          # the step that last used this input set has finished
            for dst, src in zip(sets[b], host_in):
                dst.copy_(src, non_blocking=True)
            ev_in[b].record(s_in)
        cur.wait_event(ev_in[b])
        dq_.grad = dk_.grad = dv_.grad = None
        if world > 1:
            o = seq_sharded_linear_attention(dq_, dk_, dv_, global_len=T_global)
        else:
            o = linear_attention(dq_, dk_, dv_)
        o.backward(do_dev)
        ev_done[b].record(cur)
        outs = (o.detach(), dq_.grad, dk_.grad, dv_.grad)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[b])
            for dst, src in zip(host_out, outs):
                dst.copy_(src, non_blocking=True)
                src.record_stream(s_out)
        keep[b] = outs

    e2e_step(0)
    cur.wait_stream(s_out)
    barrier()
    e0.record()
    for i in range(e2e_steps):
        e2e_step(i + 1)
    cur.wait_stream(s_out)
    e1.record()
    barrier()
    ms2 = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
    e2e_value = tokens / (ms2.item() / e2e_steps * 1e-3)
    e2e = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * tensor_bytes * world,
           "d2h_bytes_per_step": 4 * tensor_bytes * world, "steps": e2e_steps}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cv, _ = time_cpu(T, 3, 1)
        cpu = cpu_baseline_dict(cv, T)

    exchange_kind = "NCCL all-reduce"
    if world > 1:
        from flash_bla.ops import sharded
        if any(e is not None for e in sharded._exchanges.values()):
            exchange_kind = "one peer-memory kernel per direction (NVLink loads)"
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"linear_attn fwd+bwd bf16 B{B}-H{H}-D{D} T={T} per GPU"
                                       + (f", T-sharded global T={T_global}, state summed over ranks by "
                                          + exchange_kind if world > 1 else ""),
                           "l2": "inputs larger than L2 (4 x %d MB per step)" % (tensor_bytes // 2 ** 20),
                           "kernel_path": "tcgen05+TMA" if path == 1 else "cuda-core"},
                "roofline": roofline, "passes": passes, "cpu_baseline": cpu, "e2e": e2e,
                "gpu_launches": int(launches), "clocks": clocks}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--seq-len", type=int, default=32768)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
