#!/usr/bin/env python
"""Benchmark of stick-breaking attention forward+backward (packed variable-length layout, bf16).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c4|c5]

One step = one forward and one backward over one synthetic batch through the public API
(``sb_attn_varlen`` + autograd).  At N GPUs every rank runs its own batch of the same shape (independent
sequences, no collective on the data path: weak scaling); the time is the maximum over ranks.
Prints ONE JSON line on rank 0.

Workloads (seeded synthetic data, N(0,1) inputs rounded to bf16, inv_temp = 1/sqrt(D)):
  c2  32 heads, head_dim 128, 16384 tokens packed from lengths drawn uniformly in [256, 4096]  (default)
  c3  32 heads, head_dim 128, 8 sequences of 4096 tokens
  c4   8 heads, head_dim 128, one sequence of 65536 tokens, inputs 0.5*N(0,1)
  c5  64 heads, head_dim 128, 131072 tokens packed from log-normal lengths; heads are SPLIT over the ranks
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np
import torch

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture summarised in profiles/tc_kernels_c2.md
NCU_TRAFFIC_BYTES = {"c2-varlen-h32-d128-t16384": {"fwd": 618e6, "bwd_dq": 895e6, "bwd_dkdv": 1002e6}}

METRIC = "fwd+bwd TFLOP/s (varlen, bf16)"
UNIT = "TFLOP/s"
NOMINAL_BF16_TFLOPS = 2250.0


# ------------------------------------------------------------------------------------------------ workloads
def lengths_uniform(total, lo, hi, seed):
    g = torch.Generator().manual_seed(seed)
    out, tot = [], 0
    while tot < total:
        l = min(int(torch.randint(lo, hi + 1, (1,), generator=g)), total - tot)
        out.append(l)
        tot += l
    return out


def lengths_lognormal(total, median, sigma, lo, hi, seed):
    g = torch.Generator().manual_seed(seed)
    out, tot = [], 0
    while tot < total:
        z = float(torch.randn(1, generator=g))
        l = int(min(max(round(math.exp(math.log(median) + sigma * z)), lo), hi))
        l = min(l, total - tot)
        out.append(l)
        tot += l
    return out


def workload(name):
    if name == "c2":
        return dict(name="c2-varlen-h32-d128-t16384", H=32, D=128, lengths=lengths_uniform(16384, 256, 4096, 0),
                    scale=1.0, split_heads=False)
    if name == "c3":
        return dict(name="c3-train-h32-d128-8x4096", H=32, D=128, lengths=[4096] * 8, scale=1.0, split_heads=False)
    if name == "c4":
        return dict(name="c4-long-h8-d128-1x65536", H=8, D=128, lengths=[65536], scale=0.5, split_heads=False)
    if name == "c5":
        return dict(name="c5-sweep-h64-d128-t131072", H=64, D=128,
                    lengths=lengths_lognormal(131072, 1024, 1.0, 64, 16384, 0), scale=1.0, split_heads=True)
    raise SystemExit(f"unknown workload {name}")


def pairs(lengths):
    return sum(l * (l - 1) // 2 for l in lengths)


def flops_fwd_bwd(H, D, lengths):
    """Algorithmic work: 4*D per valid (query,key) pair forward (QK^T, PV), 10*D backward (S, dO V^T, dQ, dK, dV)."""
    return 14.0 * D * pairs(lengths) * H


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        rows = [r for t, r in self.rows if t0 - 0.05 <= t <= t1 + 0.15] or [r for _, r in self.rows]
        for r in rows:
            parts = [x.strip() for x in r.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ peaks
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "hbm_gbs": d["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------ CPU baseline
def cpu_reference_step(wl, heads, seqs, seed=0):
    """One bounded pass of the CPU oracle (float32, the reference's triangular-matmul suffix sum) over ``heads`` heads
    of the sequences listed in ``seqs``.  Returns (seconds, algorithmic flops)."""
    from oracle import sb_oracle as orc
    D = wl["D"]
    rng = np.random.RandomState(seed)
    it = 1.0 / math.sqrt(D)
    t = 0.0
    fl = 0.0
    for L in seqs:
        q, k, v, do = (rng.standard_normal((heads, L, D)).astype(np.float32) * wl["scale"] for _ in range(4))
        drem = rng.standard_normal((heads, L)).astype(np.float32)
        t0 = time.perf_counter()
        orc.sb_dense_fwd(q, k, v, it, dtype=np.float32, faithful=True)
        orc.sb_dense_bwd(q, k, v, do, drem, it, dtype=np.float32)
        t += time.perf_counter() - t0
        fl += 14.0 * D * (L * (L - 1) // 2) * heads
    return t, fl


def cpu_sample_of(wl):
    """A sample of the workload the host finishes in roughly 10-30 s: one head, sequences capped at 4096 tokens."""
    seqs = [min(l, 4096) for l in wl["lengths"]]
    room, out = 6.0e10 * 3, []   # sum of L^3 the sample may hold
    for l in seqs:
        if room - float(l) ** 3 < 0 and out:
            break
        out.append(l)
        room -= float(l) ** 3
    return out


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    seqs = cpu_sample_of(wl)
    cpu_reference_step(wl, 1, seqs[:1])
    times, fl = [], 0.0
    for i in range(args.warmup + args.steps):
        t, fl = cpu_reference_step(wl, 1, seqs, seed=i)
        if i >= args.warmup:
            times.append(t)
    sec = sum(times) / len(times)
    val = fl / sec / 1e12
    sample = (f"1 of {wl['H']} heads, sequences {seqs} of the workload (lengths capped at 4096), float32 numpy port of "
              f"sb_ref.py with its O(L^3) triangular-matmul suffix sum, closed-form backward")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["name"], "lengths": wl["lengths"], "sample": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tokens_per_s": sum(seqs) / sec, "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ sharding
def shard_of(wl, world, rank):
    """What rank `rank` of `world` processes works on: (heads of its batch, first head, whole batches in the job).

    Every (head, sequence) pair is independent, so there is no collective on the data path.  Default workloads give
    every rank a whole batch of its own (weak scaling: `world` batches in the job); a workload with `split_heads`
    is ONE batch whose heads are cut into `world` contiguous slices (strong scaling)."""
    H = wl["H"]
    if wl["split_heads"]:
        if H % world:
            raise SystemExit("heads must divide over the ranks")
        return H // world, rank * (H // world), 1
    return H, 0, world


def max_over_ranks(ms, world, device):
    """Device time of the job = the slowest rank's."""
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ------------------------------------------------------------------------------------------------ GPU arm
def run_ours(args, wl):
    import torch.distributed as dist
    from stickbreaking_attention_b200 import check_status, ops, sb_attn_varlen

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU implementation of the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # keep stdout to the one JSON line: NCCL prints its version banner there at the VERSION level
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)

    D, lengths = wl["D"], wl["lengths"]
    H, _, n_jobs = shard_of(wl, world, rank)
    T = sum(lengths)
    it = 1.0 / math.sqrt(D)
    g = torch.Generator().manual_seed(1000 + rank)

    def host(*shape):
        return (torch.randn(*shape, generator=g) * wl["scale"]).to(torch.bfloat16).pin_memory()

    hq, hk, hv = host(H, T, D), host(H, T, D), host(H, T, D)
    hdo = torch.randn(H, T, D, generator=g).to(torch.bfloat16).pin_memory()
    cu = torch.tensor(np.cumsum(lengths), dtype=torch.int32, device=dev)
    max_len = max(lengths)
    q, k, v = (x.to(dev, non_blocking=True).requires_grad_() for x in (hq, hk, hv))
    do = hdo.to(dev, non_blocking=True)
    drem = torch.zeros(H, T, dtype=torch.bfloat16, device=dev)

    def step():
        o, rem = sb_attn_varlen(q, k, v, cu, max_len, inv_temp=it, zero_start=False)
        return torch.autograd.grad([o, rem], [q, k, v], [do, drem])

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sync_all()
    check_status()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    t_wall0 = time.time()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    sync_all()
    t_wall1 = time.time()
    ms = ev0.elapsed_time(ev1)
    check_status()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    ms_step = max_over_ranks(ms, world, dev) / args.steps

    # ---- per-kernel times (forward / backward-dq / backward-dk,dv), events on the launching stream
    def time_kernel(fn, reps):
        fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    kernels = {}
    if rank == 0:
        with torch.no_grad():
            reps = max(3, min(args.steps, 10))
            o_, rem_, nla_, ws = ops.varlen_fwd(q, k, v, cu, max_len, it)
            outs = (torch.empty_like(q), torch.empty_like(k), torch.empty_like(v))
            _, bwd_bytes = ops._workspace_sizes(ops._base_params(q, False, cu, max_len, it, False, True))
            bws = torch.empty(bwd_bytes, dtype=torch.uint8, device=dev)
            kernels["fwd"] = time_kernel(lambda: ops.varlen_fwd(q, k, v, cu, max_len, it), reps)
            kernels["bwd_dq"] = time_kernel(
                lambda: ops.varlen_bwd(do, drem, q, k, v, cu, max_len, ws, it, phases=1, out=outs, bwd_workspace=bws), reps)
            kernels["bwd_dkdv"] = time_kernel(
                lambda: ops.varlen_bwd(do, drem, q, k, v, cu, max_len, ws, it, phases=2, out=outs, bwd_workspace=bws), reps)
            del o_, rem_, nla_, ws, outs, bws

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region
    ho = torch.empty(H, T, D, dtype=torch.bfloat16).pin_memory()
    hrem = torch.empty(H, T, dtype=torch.bfloat16).pin_memory()
    hdq, hdk, hdv = (torch.empty(H, T, D, dtype=torch.bfloat16).pin_memory() for _ in range(3))
    dq_, dk_, dv_ = (torch.empty(H, T, D, dtype=torch.bfloat16, device=dev) for _ in range(3))
    h2d = sum(x.numel() * x.element_size() for x in (hq, hk, hv, hdo))
    d2h = sum(x.numel() * x.element_size() for x in (ho, hrem, hdq, hdk, hdv))

    # Every step copies its inputs in and its five results out.  Three streams and two sets of device input buffers:
    # the inputs of step i + 1 arrive and the results of step i - 1 leave while step i computes (PCIe is full duplex).
    s_comp = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ins = [(q, k, v, do)]
    ins.append(tuple(torch.empty_like(x).requires_grad_(x.requires_grad) for x in ins[0]))
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_out = torch.cuda.Event()

    def e2e_step(i):
        b = i & 1
        bq, bk, bv, bdo = ins[b]
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_comp[b])  # step i - 2 has finished reading this set of buffers
            bq.data.copy_(hq, non_blocking=True)
            bk.data.copy_(hk, non_blocking=True)
            bv.data.copy_(hv, non_blocking=True)
            bdo.data.copy_(hdo, non_blocking=True)
            ev_in[b].record(s_in)
        s_comp.wait_event(ev_in[b])
        o, rem = sb_attn_varlen(bq, bk, bv, cu, max_len, inv_temp=it, zero_start=False)
        gq, gk, gv = torch.autograd.grad([o, rem], [bq, bk, bv], [bdo, drem])
        ev_comp[b].record(s_comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[b])
            for src, dst in ((o.detach(), ho), (rem.detach(), hrem), (gq, hdq), (gk, hdk), (gv, hdv)):
                src.record_stream(s_out)
                dst.copy_(src, non_blocking=True)
            ev_out.record(s_out)

    e2e_steps = max(2, min(args.steps, 10))
    e2e_step(0)
    e2e_step(1)
    sync_all()
    ev0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    s_comp.wait_event(ev_out)  # the last results are on the host
    ev1.record()
    sync_all()
    e2e_ms = max_over_ranks(ev0.elapsed_time(ev1), world, dev) / e2e_steps

    if rank == 0:
        flops_job = flops_fwd_bwd(wl["H"], D, lengths) * n_jobs
        tokens_job = T * n_jobs
        value = flops_job / (ms_step * 1e-3) / 1e12
        peaks = measured_peaks()
        fl_rank = flops_fwd_bwd(H, D, lengths)
        dom = max(kernels, key=kernels.get)
        share = {"fwd": 4.0 / 14.0, "bwd_dq": 5.0 / 14.0, "bwd_dkdv": 5.0 / 14.0}
        # the backward's 10*D flops per pair are split evenly over its two kernels (S and dO V^T are recomputed in both)
        achieved = fl_rank * share[dom] / (kernels[dom] * 1e-3) / 1e12
        peak = peaks["bf16_tflops"]
        roofline = {
            "bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak, "peak_source": f"of {peaks['source']} (burst cuBLAS bf16)",
            "frac_of_nominal_2250": achieved / NOMINAL_BF16_TFLOPS,
            "traffic": (NCU_TRAFFIC_BYTES.get(wl["name"], {}).get(dom) if world == 1 else None), "traffic_unit": "bytes",
            "kernel_ms": kernels,
            "kernel_tflops": {kk: fl_rank * share[kk] / (vv * 1e-3) / 1e12 for kk, vv in kernels.items()},
        }
        cpu_seqs = cpu_sample_of(wl)
        cpu_reference_step(wl, 1, cpu_seqs[:1])
        csec, cfl = cpu_reference_step(wl, 1, cpu_seqs)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if wl["split_heads"] else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl["name"], "heads": wl["H"], "head_dim": D, "tokens": T, "lengths": lengths,
                       "inputs": "N(0,1)*%g bf16, dO N(0,1), drem 0" % wl["scale"],
                       "l2": "inputs larger than L2 (q,k,v,dO %d MB per rank)" % (h2d >> 20),
                       "sharding": ("heads split over ranks" if wl["split_heads"] else "one batch per rank, no collective")},
            "tokens_per_s": tokens_job / (ms_step * 1e-3),
            "frac_of_nominal_bf16_peak": value / (NOMINAL_BF16_TFLOPS * world),
            "frac_of_measured_bf16_peak": value / (peaks["bf16_tflops_sustained"] * world),
            "roofline": roofline,
            "cpu_baseline": {"value": cfl / csec / 1e12, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                             "sample": f"1 head, sequences {cpu_seqs}, float32 numpy port of sb_ref.py (O(L^3) suffix sum)"},
            "e2e": {"value": flops_job / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": 4 * args.steps,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4", "c5"])
    args = ap.parse_args()
    wl = workload(args.workload)
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
