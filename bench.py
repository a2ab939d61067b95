"""Benchmark of the hot path: linear_attention forward + backward, bf16, B=8 H=16 D=64.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--seq-len T] [--impl reference]

One step = one forward + backward of ``linear_attention`` over one batch of synthetic
inputs (q, k = elu(N(0,1))+1, v, dO ~ N(0,1), seeded), T = 32768 tokens per rank.
With N > 1 (launched by torch.distributed.run, one rank per GPU) the sequence is
sharded along T: every rank holds 32768 tokens of a global sequence of N*32768, and
the per-head state (and its gradient) is summed over the ranks once per direction by
one kernel that reads the peers' memory over NVLink -- weak scaling.  Rank 0 prints one JSON line.

``value``  : tokens/s (tokens = B * T_global) with inputs resident in HBM, public API
             (``linear_attention(...).backward(dO)``), CUDA-event timed, max over ranks.
             The K steps are timed as a block, the block is repeated (>= 10 times, >= 0.2 s
             in all) and the MEDIAN block is reported (``blocks`` has min / max).
``e2e``    : the same metric with pinned host buffers: every step copies q, k, v, dO
             host->device and o, dq, dk, dv device->host inside the timed region.
``roofline``: the slowest of the four kernels (timed one by one with CUDA events on the
             launching stream): algorithmic bytes / duration against the measured copy
             bandwidth of this machine pool.
``parity`` : (N > 1) a small sharded forward + backward checked against the single-GPU
             operator on the gathered sequence and against the fp64 formula, before timing;
             a failure ends the run with a non-zero exit code.
``cfg3``   : simple_la bf16 B4-H32-D128 with a GLOBAL T of 262144 split over the N ranks
             (strong scaling), the configuration whose 8.4 MB state is the large exchange.
``triton_reference`` : (N = 1) the reference's own Triton ``linear_attention`` on the same GPU
             and inputs, when an installed copy of the reference is found next to this file.
``cpu_baseline`` / ``--impl reference``: the reference's torch path (``naive_linear_attn``,
             bf16, autograd backward) on the host cores, on a bounded sample of the workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "flash-bidirectional-linear-attention_b200")
REF = os.path.join(ROOT, "baseline", "_ref")
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
CFG3 = dict(B=4, H=32, D=128, T=262144)
CFG5 = dict(B=2, H=24, T=4608, D=128, block=64, density=0.1)
# DRAM bytes (read + write) of one launch of each pass at B8-H16-D64, T = 32768, from an ncu
# capture of dram__bytes_read.sum + dram__bytes_write.sum (one launch per kernel).
NCU_DRAM_BYTES_T32768 = {"fwd_state": 1.0789e9, "fwd_out": 1.0292e9, "bwd_state": 1.5895e9, "bwd_in": 2.1086e9}


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


def make_inputs(T, device, seed, shape=(B, H, D), positive=True):
    b, h, d = shape
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn(b, h, T, d, device=device, generator=g)
    k = torch.randn(b, h, T, d, device=device, generator=g)
    if positive:
        q, k = F.elu(q) + 1, F.elu(k) + 1
    v = torch.randn(b, h, T, d, device=device, generator=g)
    do = torch.randn(b, h, T, d, device=device, generator=g)
    return [x.to(torch.bfloat16) for x in (q, k, v, do)]


# ---------------------------------------------------------------------------------------
# CPU arm: the reference's torch path on the host cores
# ---------------------------------------------------------------------------------------
def _reference_naive():
    """``naive_linear_attn`` of the installed reference (plain torch), or None."""
    path = os.path.join(REF, "flash_bla", "ops", "linear_attn", "naive.py")
    if not os.path.exists(path):
        return None
    try:
        import importlib.util
        spec = importlib.util.spec_from_file_location("_ref_linear_attn_naive", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod.naive_linear_attn
    except Exception:
        return None


def cpu_step_factory(T):
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, do = make_inputs(T, "cpu", 0)
    q, k, v, do = (x[:CPU_SAMPLE_BATCH].contiguous() for x in (q, k, v, do))
    naive = _reference_naive()
    if naive is not None:
        kind = "reference"

        def step():
            xs = [x.clone().requires_grad_() for x in (q, k, v)]
            naive(*xs).backward(do)
    else:
        from oracle import bla_oracle as O
        kind = "port"

        def step():
            O.linear_attn_torch_fwd_bwd(q, k, v, do)
    return step, CPU_SAMPLE_BATCH * T, kind


def time_cpu(T, steps, warmup):
    step, tokens, kind = cpu_step_factory(T)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return tokens / dt, dt, kind


def cpu_baseline_dict(value, T, kind):
    what = ("the reference's naive_linear_attn (flash_bla/ops/linear_attn/naive.py of the installed reference)"
            if kind == "reference" else "the reference's naive path restated in oracle/")
    return {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
            "host_cpus": os.cpu_count(),
            "sample": f"dense torch bf16 forward + autograd backward ({what}) on B={CPU_SAMPLE_BATCH} of the "
                      f"{B} batch rows, H={H}, T={T}, D={D} per step"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = args.seq_len
    value, dt, kind = time_cpu(T, args.steps, max(1, args.warmup))
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"linear_attn fwd+bwd bf16 B{B}-H{H}-D{D} T={T}, CPU sample "
                                   f"B={CPU_SAMPLE_BATCH}"},
            "cpu_baseline": cpu_baseline_dict(value, T, kind),
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------
# the reference's Triton kernels on this GPU (a child process, so a failure there is only a note)
# ---------------------------------------------------------------------------------------
_TRITON_CHILD = r"""
import json, sys, time
sys.path.insert(0, sys.argv[1])
T = int(sys.argv[2])
import torch, torch.nn.functional as F
from flash_bla.ops.linear_attn.fused import linear_attention
g = torch.Generator(device="cuda").manual_seed(1000)
mk = lambda pos: (F.elu(torch.randn(8, 16, T, 64, device="cuda", generator=g)) + 1 if pos
                  else torch.randn(8, 16, T, 64, device="cuda", generator=g)).to(torch.bfloat16)
q, k, v, do = mk(True), mk(True), mk(False), mk(False)
q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
def step():
    q.grad = k.grad = v.grad = None
    linear_attention(q, k, v).backward(do)
t0 = time.time()
for _ in range(3):
    step()
torch.cuda.synchronize()
tune_s = time.time() - t0
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
best = []
for _ in range(5):
    e0.record()
    for _ in range(10):
        step()
    e1.record()
    torch.cuda.synchronize()
    best.append(e0.elapsed_time(e1) / 10)
best.sort()
print(json.dumps({"ms_per_step": best[len(best) // 2], "autotune_s": tune_s}))
"""


def triton_reference(T, ours_ms, limit_s=420):
    if not os.path.isdir(os.path.join(REF, "flash_bla", "ops", "linear_attn")):
        return {"unavailable": "no installed copy of the reference next to bench.py"}
    try:
        out = subprocess.run([sys.executable, "-c", _TRITON_CHILD, REF, str(T)], capture_output=True, text=True,
                             timeout=limit_s)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"the reference's autotuning did not finish within {limit_s} s"}
    if out.returncode != 0:
        return {"unavailable": "the reference failed: " + (out.stderr.strip().splitlines() or ["?"])[-1][:200]}
    try:
        got = json.loads(out.stdout.strip().splitlines()[-1])
    except Exception:
        return {"unavailable": "unreadable output of the reference run"}
    ms = got["ms_per_step"]
    return {"what": "flash_bla.ops.linear_attn.fused.linear_attention of the installed reference (Triton, autotuned), "
                    "same GPU, same input distribution, fwd+bwd, CUDA events, median of 5 x 10 steps",
            "ms_per_step": ms, "value": B * T / (ms * 1e-3), "unit": UNIT, "autotune_s": got["autotune_s"],
            "speedup_of_this_library": ms / ours_ms}


# ---------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------
def timed_blocks(step, steps, barrier, world, dev, min_blocks=10, min_total_s=0.2, max_blocks=200):
    """Times `steps` back-to-back steps as one block (barrier + synchronize on both sides, CUDA
    events, max over ranks) and repeats the block; returns the per-block milliseconds."""
    blocks = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    while len(blocks) < min_blocks or (sum(blocks) < min_total_s * 1e3 and len(blocks) < max_blocks):
        barrier()
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        blocks.append(ms.item())
    return blocks


def parity_check(world, rank, dev):
    """A small T-sharded forward + backward against (a) the single-GPU operator on the whole
    sequence and (b) the fp64 formula for one (batch, head) unit.  Returns the record for the JSON
    line; ``ok`` is the verdict."""
    from flash_bla.ops.linear_attn.fused import linear_attention
    from flash_bla.ops.sharded import seq_sharded_linear_attention
    worst, worst_formula, cases = 0.0, 0.0, []
    for dtype, name in ((torch.bfloat16, "bf16"), (torch.float32, "fp32")):
        b, h, d, t_loc = 2, 4, 64, 2048
        Tg = t_loc * world
        g = torch.Generator(device=dev).manual_seed(4242)           # the same full problem on every rank
        q = (F.elu(torch.randn(b, h, Tg, d, device=dev, generator=g)) + 1).to(dtype)
        k = (F.elu(torch.randn(b, h, Tg, d, device=dev, generator=g)) + 1).to(dtype)
        v = torch.randn(b, h, Tg, d, device=dev, generator=g).to(dtype)
        do = torch.randn(b, h, Tg, d, device=dev, generator=g).to(dtype)
        sl = slice(rank * t_loc, (rank + 1) * t_loc)
        xs = [x[:, :, sl].contiguous().requires_grad_() for x in (q, k, v)]
        o = seq_sharded_linear_attention(*xs, global_len=Tg)
        o.backward(do[:, :, sl].contiguous())
        mine = torch.stack([o.detach()] + [x.grad for x in xs])      # (4, b, h, t_loc, d)
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        if rank == 0:
            got = torch.cat(parts, dim=3).float()                    # whole sequence, rank order
            full = [x.clone().requires_grad_() for x in (q, k, v)]
            o1 = linear_attention(*full)
            o1.backward(do)
            ref = torch.stack([o1.detach()] + [x.grad for x in full]).float()
            ulp = {torch.bfloat16: 2.0 ** -7, torch.float32: 0.0}[dtype]
            for i in range(4):
                rms = ref[i].pow(2).mean().sqrt()
                slack = ulp * ref[i].abs() + (2e-3 if ulp else 1e-4) * rms
                worst = max(worst, ((got[i] - ref[i]).abs() / slack).max().item())
            # fp64 formula, unit (0, 0): o = q S / (q kmean + eps), S = K^T V / T
            q0, k0, v0 = (x[0, 0].double() for x in (q, k, v))
            o64 = (q0 @ (k0.t() @ v0 / Tg)) / ((q0 * k0.mean(0)).sum(-1, keepdim=True) + 1e-6)
            err = ((got[0, 0, 0].double() - o64).abs().max() / o64.pow(2).mean().sqrt()).item()
            bar = 2e-2 if dtype == torch.bfloat16 else 1e-5
            worst_formula = max(worst_formula, err / bar)
            cases.append(f"{name} B{b}-H{h}-D{d} T={Tg}")
    rec = {"cases": cases, "max_err_over_bar": worst, "formula_err_over_bar": worst_formula,
           "bar": "vs the 1-GPU operator: one ulp of the output type + 0.2 % of the RMS (fp32: 1e-4 of the RMS); "
                  "vs the fp64 formula: 2e-2 max-abs/RMS (bf16), 1e-5 (fp32)",
           "ok": bool(worst <= 1.0 and worst_formula <= 1.0)}
    flag = torch.tensor([1 if (rank != 0 or rec["ok"]) else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return rec, bool(flag.item())


def run_cfg3(world, rank, dev, barrier, peak):
    """simple_la bf16 B4-H32-D128, global T = 262144 split along T over the ranks."""
    from flash_bla.ops.sharded import seq_sharded_simple_la
    from flash_bla.ops.simple_la.fused import simple_la
    c = CFG3
    if c["T"] % world:
        return {"skipped": f"T={c['T']} does not split over {world} ranks"}
    t_loc = c["T"] // world
    need = 9 * c["B"] * c["H"] * t_loc * c["D"] * 2
    if torch.cuda.mem_get_info(dev)[0] < need * 1.1:
        return {"skipped": f"needs {need / 2 ** 30:.0f} GiB free on the device"}
    q, k, v, do = make_inputs(t_loc, dev, 3000 + rank, shape=(c["B"], c["H"], c["D"]), positive=False)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()

    def step():
        q.grad = k.grad = v.grad = None
        o = seq_sharded_simple_la(q, k, v) if world > 1 else simple_la(q, k, v)
        o.backward(do)

    for _ in range(3):
        step()
    blocks = timed_blocks(lambda: step(), 5, barrier, world, dev, min_blocks=5, min_total_s=0.2, max_blocks=40)
    ms = statistics.median(blocks) / 5
    nbytes = 11 * c["B"] * c["H"] * t_loc * c["D"] * 2          # per rank
    out = {"workload": f"simple_la fwd+bwd bf16 B{c['B']}-H{c['H']}-D{c['D']} global T={c['T']}, "
                       f"{t_loc} tokens per GPU" + (", state (8.4 MB) summed over ranks by one kernel per direction" if world > 1 else ""),
           "scaling": "strong", "ms_per_step": ms, "value": c["B"] * c["T"] / (ms * 1e-3), "unit": UNIT,
           "algo_gbs_per_gpu": nbytes / (ms * 1e-3) / 1e9, "frac_of_peak": nbytes / (ms * 1e-3) / 1e9 / peak,
           "blocks": {"n": len(blocks), "steps_each": 5, "min_ms": min(blocks) / 5, "max_ms": max(blocks) / 5}}
    del q, k, v, do
    torch.cuda.empty_cache()
    return out


def run_cfg4(world, rank, dev, barrier, peak):
    """varlen_linear_attention bf16 H16-D64 on 32 packed sequences of 256..16384 tokens (seeded lengths): whole
    sequences are dealt to the ranks (longest first onto the lightest rank), each rank packs its own and runs the
    operator on them; no communication."""
    from flash_bla.ops.linear_attn.varlen import varlen_linear_attention
    from flash_bla.ops.sharded import partition_sequences
    heads, d = 16, 64
    lengths = torch.randint(256, 16385, (32,), generator=torch.Generator().manual_seed(0)).tolist()
    mine = [lengths[i] for i in partition_sequences(lengths, world)[rank]]
    if not mine:
        return {"skipped": f"32 sequences do not cover {world} ranks"}
    tot, mx = sum(mine), max(mine)
    cu = torch.tensor([0] + list(torch.tensor(mine).cumsum(0)), dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev).manual_seed(4000 + rank)
    q = (F.elu(torch.randn(tot, heads, d, device=dev, generator=g)) + 1).bfloat16().requires_grad_()
    k = (F.elu(torch.randn(tot, heads, d, device=dev, generator=g)) + 1).bfloat16().requires_grad_()
    v = torch.randn(tot, heads, d, device=dev, generator=g).bfloat16().requires_grad_()
    do = torch.randn(tot, heads, d, device=dev, generator=g).bfloat16()

    def step():
        q.grad = k.grad = v.grad = None
        varlen_linear_attention(q, k, v, cu, mx).backward(do)

    for _ in range(3):
        step()
    blocks = timed_blocks(lambda: step(), 10, barrier, world, dev, min_blocks=5, min_total_s=0.1, max_blocks=40)
    ms = statistics.median(blocks) / 10
    nbytes = 11 * tot * heads * d * 2                      # this rank's share (the slowest rank sets the time)
    out = {"workload": f"varlen_linear_attention fwd+bwd bf16 H{heads}-D{d}, 32 packed sequences of 256..16384 tokens "
                       f"({sum(lengths)} in all), {len(mine)} sequences / {tot} tokens on rank 0"
                       + (", whole sequences dealt to the ranks, no communication" if world > 1 else ""),
           "scaling": "strong", "ms_per_step": ms, "value": sum(lengths) / (ms * 1e-3), "unit": UNIT,
           "algo_gbs_rank0": nbytes / (ms * 1e-3) / 1e9, "frac_of_peak_rank0": nbytes / (ms * 1e-3) / 1e9 / peak,
           "blocks": {"n": len(blocks), "steps_each": 10, "min_ms": min(blocks) / 10, "max_ms": max(blocks) / 10}}
    del q, k, v, do
    torch.cuda.empty_cache()
    return out


def run_cfg5(world, rank, dev, barrier):
    """piecewise_sparse_attention bf16 B2-H24-T4608-D128, block 64, density 0.1: the 48 (batch, head) pairs are
    independent, each rank takes its share (no communication); forward + backward of the whole operator
    (block statistics, first-order state, selection, attention)."""
    from flash_bla.ops.piecewise_attn.kernel import piecewise_sparse_attention
    from flash_bla.ops.sharded import shard_units
    c = CFG5
    units = shard_units(c["B"] * c["H"], world, rank)
    if len(units) == 0:
        return {"skipped": f"{c['B'] * c['H']} (batch, head) pairs do not cover {world} ranks"}
    g = torch.Generator(device=dev).manual_seed(5000 + rank)
    # this rank's pairs as a (1, n, T, D) problem: pairs do not interact, so the split is free
    q, k, v, do = (torch.randn(1, len(units), c["T"], c["D"], device=dev, generator=g).bfloat16() for _ in range(4))
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()

    def step():
        q.grad = k.grad = v.grad = None
        o = piecewise_sparse_attention(q, k, v, density=c["density"], block_size=c["block"])
        o.backward(do)

    def fwd_only():
        with torch.no_grad():
            piecewise_sparse_attention(q, k, v, density=c["density"], block_size=c["block"])

    for _ in range(3):
        step()
    blocks = timed_blocks(lambda: step(), 10, barrier, world, dev, min_blocks=5, min_total_s=0.1, max_blocks=40)
    fblocks = timed_blocks(lambda: fwd_only(), 10, barrier, world, dev, min_blocks=5, min_total_s=0.05, max_blocks=40)
    ms, fms = statistics.median(blocks) / 10, statistics.median(fblocks) / 10
    out = {"workload": f"piecewise_sparse_attention fwd+bwd bf16 B{c['B']}-H{c['H']}-T{c['T']}-D{c['D']}, block {c['block']}, "
                       f"density {c['density']}; {len(units)} (batch, head) pairs per GPU, no communication",
           "scaling": "strong", "ms_per_step": ms, "fwd_ms": fms, "value": c["B"] * c["T"] / (ms * 1e-3), "unit": UNIT,
           "kernels": "tcgen05 (attention forward, backward query side, backward key side)",
           "blocks": {"n": len(blocks), "steps_each": 10, "min_ms": min(blocks) / 10, "max_ms": max(blocks) / 10}}
    del q, k, v, do
    torch.cuda.empty_cache()
    return out


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

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    parity = None
    if world > 1:
        parity, all_ok = parity_check(world, rank, dev)
        if not all_ok:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "n_gpus": world, "parity": parity,
                                  "error": "sharded results differ from the single-GPU operator"}), flush=True)
            dist.destroy_process_group()
            raise SystemExit(3)

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

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    if world > 1:
        # the collectives the timing itself uses, once before anything is timed: a library that sets up
        # buffers or connections on first use must not do so next to a timed kernel
        warm = torch.zeros(1, device=dev, dtype=torch.float64)
        dist.all_reduce(warm, op=dist.ReduceOp.MAX)
        barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = _C.lib().fbla_launch_count()
    blocks = timed_blocks(step, args.steps, barrier, world, dev)
    launches = (_C.lib().fbla_launch_count() - launches0) // len(blocks)
    clocks = sampler.stop()
    ms_per_step = statistics.median(blocks) / args.steps
    value = tokens / (ms_per_step * 1e-3)
    block_info = {"n": len(blocks), "steps_each": args.steps, "reported": "median",
                  "min_ms_per_step": min(blocks) / args.steps, "max_ms_per_step": max(blocks) / args.steps,
                  "timed_s": sum(blocks) * 1e-3}

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
    traffic = NCU_DRAM_BYTES_T32768[dom] if (B, H, D, T) == (8, 16, 64, 32768) else None
    roofline = {"bound": "hbm", "kernel": dom, "achieved": passes[dom]["gbs"], "peak": peak, "unit": "GB/s",
                "frac": passes[dom]["gbs"] / peak, "traffic": traffic, "peak_kind": f"of {peak_kind}",
                "all_passes_gbs": total_gbs, "all_passes_frac": total_gbs / peak,
                "step_gbs": 11 * tensor_bytes / (ms_per_step * 1e-3) / 1e9,
                "step_frac": 11 * tensor_bytes / (ms_per_step * 1e-3) / 1e9 / peak,
                "frac_of_nominal_8000": total_gbs / 8000.0}
    del o_buf, dq, dk, dv

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
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(e2e_steps):
        e2e_step(i + 1)
    cur.wait_stream(s_out)
    e1.record()
    barrier()
    ms2_local = e0.elapsed_time(e1)
    ms2 = torch.tensor([ms2_local], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
    e2e_value = tokens / (ms2.item() / e2e_steps * 1e-3)
    # what limits it: bytes each rank moves per direction over its own PCIe link per second
    link_gbs = 4 * tensor_bytes / (ms2.item() / e2e_steps * 1e-3) / 1e9
    e2e = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * tensor_bytes * world,
           "d2h_bytes_per_step": 4 * tensor_bytes * world, "steps": e2e_steps,
           "per_rank_h2d_gbs": link_gbs, "per_rank_d2h_gbs": link_gbs,
           "limiter": "host<->device copies: %.0f GB/s in each direction at once per rank against %.2f ms of kernels "
                      "per step; summed over ranks %.0f GB/s each way through the host's memory and PCIe root"
                      % (link_gbs, ms_per_step, link_gbs * world)}
    del sets, keep, host_in, host_out
    torch.cuda.empty_cache()

    exchange_kind = None
    if world > 1:
        from flash_bla.ops import sharded
        kinds = {type(e).__name__ for e in sharded._exchanges.values() if e is not None}
        exchange_kind = ("by one kernel per direction over the per-segment pieces (owner sums, peer loads over NVLink)"
                         if "_FusedExchange" in kinds
                         else "by one peer-memory kernel per direction" if kinds
                         else "by NCCL all-reduce (the default beyond four ranks: measured faster than the "
                              "library's own exchange kernel there)")

    peak_now = peak
    cfg3 = None if args.no_cfg3 else run_cfg3(world, rank, dev, barrier, peak_now)
    cfg4 = None if args.no_cfg4 else run_cfg4(world, rank, dev, barrier, peak_now)
    cfg5 = None if args.no_cfg5 else run_cfg5(world, rank, dev, barrier)

    cpu = None
    triton = None
    if rank == 0 and world == 1:
        if not args.no_cpu:
            cv, _, kind = time_cpu(T, 3, 1)
            cpu = cpu_baseline_dict(cv, T, kind)
        if not args.no_triton:
            triton = triton_reference(T, ms_per_step)

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"linear_attn fwd+bwd bf16 B{B}-H{H}-D{D} T={T} per GPU"
                                       + (f", T-sharded global T={T_global}, state summed over ranks "
                                          + exchange_kind if world > 1 else ""),
                           "l2": "inputs larger than L2 (4 x %d MB per step)" % (tensor_bytes // 2 ** 20),
                           "kernel_path": "tcgen05+TMA" if path == 1 else "cuda-core"},
                "blocks": block_info, "roofline": roofline, "passes": passes, "cpu_baseline": cpu, "e2e": e2e,
                "gpu_launches": int(launches), "clocks": clocks}
        if parity is not None:
            line["parity"] = parity
        if cfg3 is not None:
            line["cfg3"] = cfg3
        if cfg4 is not None:
            line["cfg4"] = cfg4
        if cfg5 is not None:
            line["cfg5"] = cfg5
        if triton is not None:
            line["triton_reference"] = triton
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--seq-len", type=int, default=32768)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-cfg3", action="store_true", help="skip the simple_la T=262144 block")
    ap.add_argument("--no-cfg4", action="store_true", help="skip the packed variable-length block")
    ap.add_argument("--no-cfg5", action="store_true", help="skip the piecewise_sparse_attention block")
    ap.add_argument("--no-triton", action="store_true", help="skip the run of the reference's Triton kernels")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
