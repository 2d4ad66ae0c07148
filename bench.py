#!/usr/bin/env python
"""Benchmark of stick-breaking attention forward+backward (packed variable-length layout, bf16).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
                    [--heads H] [--skip kernels,e2e,cpu,sustained,c5,short,graph]

One step = one forward and one backward over one synthetic batch through the public API (``sb_attn_varlen`` +
autograd).  Prints ONE JSON line on rank 0.

``value`` is measured on the chosen workload (default c2).  At N GPUs every rank runs its own batch of that shape
(independent sequences, no collective on the data path: weak scaling); the time is the maximum over ranks.  The same
line carries three further records, each timed the same way (CUDA events, max over ranks):

  c5_strong  ONE batch of workload c5 whose 64 heads are cut into N contiguous shards (strong scaling: the lines of
             N = 1, 2, 4, 8 give the head-sharded curve), inputs generated on the device.  After the timed region
             every rank sends one short sequence of one head of its shard (inputs and all five results) to rank 0
             over NCCL, where it is compared with the CPU oracle: ``verified_ranks``.
  sustained  the default step repeated for at least two seconds, with the SM clock sampled meanwhile
  short      a pack of 128-token sequences (memory-bound): achieved HBM GB/s against the measured copy bandwidth

and, for the two small workloads c1 and b500, ``graph_replay``: the step captured once into a CUDA graph and replayed.
``cpu_baseline`` (the reference's sb_ref.py on the host cores, a bounded sample) is timed at N = 1 only.

Workloads (seeded synthetic data, N(0,1) inputs rounded to bf16, inv_temp = 1/sqrt(D)):
  c2     32 heads, head_dim 128, 16384 tokens packed from lengths drawn uniformly in [256, 4096]  (default)
  c3     32 heads, head_dim 128, 8 sequences of 4096 tokens
  c4      8 heads, head_dim 128, one sequence of 65536 tokens, inputs 0.5*N(0,1)
  c5     64 heads, head_dim 128, 131072 tokens packed from log-normal lengths; heads are SPLIT over the ranks
  short  32 heads, head_dim 128, 512 sequences of 128 tokens
  c1     4 heads, head_dim 64, 512 tokens in sequences of 128/192/192, float32 (the fp32-arithmetic kernels)
  b500   batched layout of the reference's tests: 4 x 8 heads x 500 tokens x head_dim 50, bf16 (fp32-arithmetic kernels)
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

# dram__bytes_read.sum + dram__bytes_write.sum per launch of each kernel, from one ncu capture of
#   python bench.py --workload c2 --heads 16 --steps 1 --warmup 1 --skip kernels,e2e,cpu,sustained,c5,short
# (16 of the 32 heads, so that the capture stays small), scaled to the workload's 32 heads: traffic grows in
# proportion to the heads, which are independent.
NCU_TRAFFIC_BYTES = {"c2-varlen-h32-d128-t16384": {"fwd": 2 * 295.5e6, "bwd_dq": 2 * 433.0e6, "bwd_dkdv": 2 * 488.7e6}}

METRIC = "fwd+bwd TFLOP/s (varlen, bf16)"
UNIT = "TFLOP/s"
NOMINAL_BF16_TFLOPS = 2250.0
TOL_BF16 = 2e-2


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
    base = dict(scale=1.0, split_heads=False, dtype="bf16", batch=0)
    if name == "c2":
        return dict(base, name="c2-varlen-h32-d128-t16384", H=32, D=128, lengths=lengths_uniform(16384, 256, 4096, 0))
    if name == "c3":
        return dict(base, name="c3-train-h32-d128-8x4096", H=32, D=128, lengths=[4096] * 8)
    if name == "c4":
        return dict(base, name="c4-long-h8-d128-1x65536", H=8, D=128, lengths=[65536], scale=0.5)
    if name == "c5":
        return dict(base, name="c5-sweep-h64-d128-t131072", H=64, D=128,
                    lengths=lengths_lognormal(131072, 1024, 1.0, 64, 16384, 0), split_heads=True)
    if name == "short":
        return dict(base, name="short-h32-d128-512x128", H=32, D=128, lengths=[128] * 512)
    if name == "c1":
        return dict(base, name="c1-f32-h4-d64-t512", H=4, D=64, lengths=[128, 192, 192], dtype="f32")
    if name == "b500":
        return dict(base, name="b500-batched-4x8x500x50", H=8, D=50, lengths=[500] * 4, batch=4)
    raise SystemExit(f"unknown workload {name}")


def pairs(lengths):
    return sum(l * (l - 1) // 2 for l in lengths)


def flops_fwd_bwd(H, D, lengths):
    """Algorithmic work: 4*D per valid (query,key) pair forward (QK^T, PV), 10*D backward (S, dO V^T, dQ, dK, dV)."""
    return 14.0 * D * pairs(lengths) * H


def bytes_fwd_bwd(H, D, T, elem):
    """Algorithmic HBM bytes: the forward reads q, k, v and writes o; the backward reads q, k, v, dO and writes
    dq, dk, dv (11 matrices of H*T*D elements), plus 12 bytes of per-row vectors per (head, token)."""
    return 11.0 * H * T * D * elem + 12.0 * H * T


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed regions run."""
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

    def stop(self):
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()

    def result(self, t0, t1):
        """Median SM clock and the throttle reasons seen between the wall-clock times t0 and t1."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
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
def cpu_threads():
    """All host cores, set explicitly: a launcher (torch.distributed.run) may have put OMP_NUM_THREADS=1 into the
    environment, which would make this arm depend on how the script was started."""
    n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return torch.get_num_threads()


def cpu_sample_of(wl):
    """A sample of the workload the host finishes in a few seconds: one head, sequences capped at 4096 tokens,
    as many of them (in order) as fit a budget on the sum of L^3 (the reference's suffix sum is a dense
    L x L x L contraction, sb_ref.py:21-22)."""
    seqs = [min(l, 4096) for l in wl["lengths"]]
    room, out = 1.8e11, []
    for l in seqs:
        if room - float(l) ** 3 < 0 and out:
            break
        out.append(l)
        room -= float(l) ** 3
    return out


def cpu_reference_step(wl, seqs, seed=0):
    """One pass of the reference's CPU implementation (float32) over one head of the sequences ``seqs``:
    forward and autograd backward of ``stickbreaking`` from the reference's own sb_ref.py when oracle/_ref holds it
    (kind "reference"), else the numpy restatement of it (kind "port").  Returns (seconds, algorithmic flops, kind)."""
    from oracle import ref_drive
    D = wl["D"]
    g = torch.Generator().manual_seed(seed)
    T = sum(seqs)
    q, k, v, do = (torch.randn(1, T, D, generator=g) * wl["scale"] for _ in range(4))
    drem = torch.randn(1, T, generator=g)
    fl = sum(14.0 * D * (L * (L - 1) // 2) for L in seqs)
    if ref_drive.available():
        sb = ref_drive.load()
        t0 = time.perf_counter()
        ref_drive.fwd_bwd(sb, q, k, v, do, drem, seqs)
        return time.perf_counter() - t0, fl, "reference"
    from oracle import sb_oracle as orc
    it = 1.0 / math.sqrt(D)
    t = 0.0
    start = 0
    for L in seqs:
        a = [x[:, start:start + L].numpy() for x in (q, k, v, do)]
        dr = drem[:, start:start + L].numpy()
        t0 = time.perf_counter()
        orc.sb_dense_fwd(a[0], a[1], a[2], it, dtype=np.float32, faithful=True)
        orc.sb_dense_bwd(a[0], a[1], a[2], a[3], dr, it, dtype=np.float32)
        t += time.perf_counter() - t0
        start += L
    return t, fl, "port"


def cpu_sample_text(wl, seqs, kind):
    what = ("the reference's sb_ref.py (torch, float32, autograd backward)" if kind == "reference" else
            "float32 numpy port of sb_ref.py with its O(L^3) triangular-matmul suffix sum, closed-form backward")
    return f"1 of {wl['H']} heads, sequences {seqs} of the workload (lengths capped at 4096), {what}"


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = cpu_threads()
    seqs = cpu_sample_of(wl)
    cpu_reference_step(wl, seqs[:1])
    times, fl, kind = [], 0.0, "port"
    for i in range(args.warmup + args.steps):
        t, fl, kind = cpu_reference_step(wl, seqs, seed=i)
        if i >= args.warmup:
            times.append(t)
    sec = sum(times) / len(times)
    val = fl / sec / 1e12
    sample = cpu_sample_text(wl, seqs, kind)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["name"], "lengths": wl["lengths"], "sample": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "host_cores": os.cpu_count(), "kind": kind,
                         "sample": sample},
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


def verify_pick(lengths, lo=64, hi=640):
    """The sequence of a pack that the cross-rank check uses: the shortest one of at least `lo` tokens (at most `hi`,
    so that the CPU oracle needs milliseconds).  Returns (index, start, length)."""
    best = None
    start = 0
    for i, l in enumerate(lengths):
        if lo <= l <= hi and (best is None or l < best[2]):
            best = (i, start, l)
        start += l
    if best is None:
        i = int(np.argmin(lengths))
        best = (i, int(sum(lengths[:i])), int(lengths[i]))
    return best


CHECK_FIELDS = ("q", "k", "v", "do", "drem", "o", "dq", "dk", "dv", "rem")


def pack_for_check(tensors):
    """Flattens the slices a rank contributes to the cross-rank check (CHECK_FIELDS order) into one float32 vector."""
    return torch.cat([t.detach().float().reshape(-1) for t in tensors])


def unpack_check(flat, L, D):
    """Inverse of pack_for_check: q, k, v, do [L, D]; drem [L]; o, dq, dk, dv [L, D]; rem [L]."""
    shapes = [(L, D)] * 4 + [(L,)] + [(L, D)] * 4 + [(L,)]
    out, pos = {}, 0
    for name, s in zip(CHECK_FIELDS, shapes):
        n = int(np.prod(s))
        out[name] = flat[pos:pos + n].reshape(s)
        pos += n
    return out


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
    from stickbreaking_attention_b200 import check_status, launch_count, ops, sb_attn, sb_attn_varlen

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU implementation of the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # keep stdout to the one JSON line: NCCL prints its version banner there at the VERSION level (and above);
        # a level somebody asked for explicitly (WARN, INFO ...) is left alone
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            del os.environ["NCCL_DEBUG"]
        dist.init_process_group("nccl", device_id=dev)
    skip = args.skip
    peaks = measured_peaks()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        """(ms per step as the max over ranks, wall-clock window) of `steps` calls after `warmup` untimed ones."""
        for _ in range(warmup):
            fn()
        sync_all()
        check_status()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        t1 = time.time()
        check_status()
        return max_over_ranks(e0.elapsed_time(e1), world, dev) / steps, (t0, t1)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)

    # ---------------------------------------------------------------- the main workload: one batch per rank
    D, lengths = wl["D"], wl["lengths"]
    H, _, n_jobs = shard_of(wl, world, rank)
    T = sum(lengths)
    it = 1.0 / math.sqrt(D)
    tdtype = torch.float32 if wl["dtype"] == "f32" else torch.bfloat16
    batched = wl["batch"] > 0
    shape = (wl["batch"], H, lengths[0], D) if batched else (H, T, D)
    g = torch.Generator().manual_seed(1000 + rank)

    def host(*s, scale=1.0):
        return (torch.randn(*s, generator=g) * scale).to(tdtype).pin_memory()

    hq, hk, hv = (host(*shape, scale=wl["scale"]) for _ in range(3))
    hdo = host(*shape)
    cu = torch.tensor(np.cumsum(lengths), dtype=torch.int32, device=dev)
    max_len = max(lengths)
    q, k, v = (x.to(dev, non_blocking=True).requires_grad_() for x in (hq, hk, hv))
    do = hdo.to(dev, non_blocking=True)
    drem = torch.zeros(shape[:-1], dtype=tdtype, device=dev)

    def attn(q_, k_, v_):
        if batched:
            return sb_attn(q_, k_, v_, inv_temp=it)
        return sb_attn_varlen(q_, k_, v_, cu, max_len, inv_temp=it, zero_start=False)

    def step():
        o, rem = attn(q, k, v)
        return torch.autograd.grad([o, rem], [q, k, v], [do, drem])

    step()
    torch.cuda.synchronize()
    n0 = launch_count()
    step()
    launches_per_step = launch_count() - n0  # kernels the library launched, counted inside the library
    ms_step, win_main = timed(step, args.steps, max(args.warmup, 3))

    # ---------------------------------------------------------------- the same step replayed from a CUDA graph
    # (the launch-bound workloads only: the launchers enqueue kernels on the caller's stream and nothing else, so forward and
    # backward replay from one graph launch without the Python layer and the per-kernel launch cost)
    graph_rec = None
    if "graph" not in skip and rank == 0 and world == 1 and wl["name"].split("-")[0] in ("c1", "b500"):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg):
            step()
        ms_graph, _ = timed(cg.replay, args.steps, max(args.warmup, 3))
        graph_rec = {"ms_per_step": ms_graph, "eager_ms_per_step": ms_step,
                     "what": "forward + backward captured once with torch.cuda.graph, one replay per step"}

    # ---------------------------------------------------------------- per-kernel times, events on the launching stream
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
    if rank == 0 and "kernels" not in skip and not batched:
        with torch.no_grad():
            reps = max(3, min(args.steps, 10))
            o_, rem_, nla_, ws = ops.varlen_fwd(q, k, v, cu, max_len, it)
            outs = (torch.empty_like(q), torch.empty_like(k), torch.empty_like(v))
            _, bwd_bytes = ops._workspace_sizes(ops._base_params(q, False, cu, max_len, it, False, True))
            bws = torch.empty(bwd_bytes, dtype=torch.uint8, device=dev)
            # the three launchers in the order of a step, an event between them: every kernel is timed under the conditions
            # of the step (clocks, power state, cache contents), and the three times add up to it
            calls = (("fwd", lambda: ops.varlen_fwd(q, k, v, cu, max_len, it)),
                     ("bwd_dq", lambda: ops.varlen_bwd(do, drem, q, k, v, cu, max_len, ws, it, phases=1, out=outs,
                                                       bwd_workspace=bws)),
                     ("bwd_dkdv", lambda: ops.varlen_bwd(do, drem, q, k, v, cu, max_len, ws, it, phases=2, out=outs,
                                                         bwd_workspace=bws)))
            for _, fn in calls:
                fn()
            evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(reps)]
            torch.cuda.synchronize()
            for ev in evs:
                ev[0].record()
                for i, (_, fn) in enumerate(calls):
                    fn()
                    ev[i + 1].record()
            torch.cuda.synchronize()
            for i, (name, _) in enumerate(calls):
                kernels[name] = sum(ev[i].elapsed_time(ev[i + 1]) for ev in evs) / reps
            del o_, rem_, nla_, ws, outs, bws

    # ---------------------------------------------------------------- sustained: the same step for at least two seconds
    sustained = None
    if "sustained" not in skip:
        n_sus = max(args.steps, int(math.ceil(2200.0 / max(ms_step, 1e-3))))
        ms_sus, win_sus = timed(step, n_sus, 0)
        sustained = {"steps": n_sus, "ms_per_step": ms_sus, "seconds": ms_sus * n_sus * 1e-3,
                     "value": flops_fwd_bwd(wl["H"], D, lengths) * n_jobs / (ms_sus * 1e-3) / 1e12, "unit": UNIT,
                     "window": win_sus}

    # ---------------------------------------------------------------- end to end: host buffers in, host buffers out
    e2e = None
    h2d = sum(x.numel() * x.element_size() for x in (hq, hk, hv, hdo))
    if "e2e" not in skip:
        ho = torch.empty(shape, dtype=tdtype).pin_memory()
        hrem = torch.empty(shape[:-1], dtype=tdtype).pin_memory()
        hdq, hdk, hdv = (torch.empty(shape, dtype=tdtype).pin_memory() for _ in range(3))
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
            o, rem = attn(bq, bk, bv)
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
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(e2e_steps):
            e2e_step(i)
        s_comp.wait_event(ev_out)  # the last results are on the host
        ev1.record()
        sync_all()
        e2e_ms = max_over_ranks(ev0.elapsed_time(ev1), world, dev) / e2e_steps
        e2e = {"value": flops_fwd_bwd(wl["H"], D, lengths) * n_jobs / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
               "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
        del ins, ho, hrem, hdq, hdk, hdv
    del q, k, v, do, drem, hq, hk, hv, hdo
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- short sequences: the memory-bound end
    short = None
    if "short" not in skip and rank == 0 and wl["name"].startswith("c2"):
        sw = workload("short")
        sl, sH, sD = sw["lengths"], sw["H"], sw["D"]
        sT = sum(sl)
        gd = torch.Generator(device=dev).manual_seed(7)
        sq, sk, sv = (torch.randn(sH, sT, sD, generator=gd, device=dev).bfloat16().requires_grad_() for _ in range(3))
        sdo = torch.randn(sH, sT, sD, generator=gd, device=dev).bfloat16()
        sdr = torch.zeros(sH, sT, dtype=torch.bfloat16, device=dev)
        scu = torch.tensor(np.cumsum(sl), dtype=torch.int32, device=dev)

        def short_step():
            o, rem = sb_attn_varlen(sq, sk, sv, scu, 128, inv_temp=1.0 / math.sqrt(sD), zero_start=False)
            return torch.autograd.grad([o, rem], [sq, sk, sv], [sdo, sdr])

        for _ in range(3):
            short_step()
        ms_short = time_kernel(short_step, 20)
        check_status()
        by = bytes_fwd_bwd(sH, sD, sT, 2)
        short = {"workload": sw["name"], "ms_per_step": ms_short, "algorithmic_bytes": by,
                 "achieved_gbs": by / (ms_short * 1e-3) / 1e9, "peak_gbs": peaks["hbm_gbs"],
                 "frac": by / (ms_short * 1e-3) / 1e9 / peaks["hbm_gbs"], "peak_source": f"of {peaks['source']} (copy)",
                 "value": flops_fwd_bwd(sH, sD, sl) / (ms_short * 1e-3) / 1e12, "unit": UNIT,
                 "l2": "q, k, v, dO and the results are 1.2 GB per step: larger than L2"}
        del sq, sk, sv, sdo, sdr
        torch.cuda.empty_cache()

    # ---------------------------------------------------------------- c5: ONE batch, heads split over the ranks
    c5 = None
    if "c5" not in skip and wl["name"].startswith("c2") and 64 % world == 0:
        w5 = workload("c5")
        l5, D5 = w5["lengths"], w5["D"]
        H5, h0, _ = shard_of(w5, world, rank)
        T5 = sum(l5)
        it5 = 1.0 / math.sqrt(D5)
        gd = torch.Generator(device=dev).manual_seed(500 + h0)  # a shard's data depends on its first head only
        q5, k5, v5 = (torch.randn(H5, T5, D5, generator=gd, device=dev).bfloat16().requires_grad_() for _ in range(3))
        do5 = torch.randn(H5, T5, D5, generator=gd, device=dev).bfloat16()
        dr5 = torch.randn(H5, T5, generator=gd, device=dev).bfloat16()
        cu5 = torch.tensor(np.cumsum(l5), dtype=torch.int32, device=dev)
        res5 = []

        def step5():
            o, rem = sb_attn_varlen(q5, k5, v5, cu5, max(l5), inv_temp=it5, zero_start=False)
            res5[:] = [o, rem, *torch.autograd.grad([o, rem], [q5, k5, v5], [do5, dr5])]

        steps5 = max(3, min(args.steps, 5))
        ms5, win5 = timed(step5, steps5, 3)
        # cross-rank check: one short sequence of the first head of every shard goes to rank 0 over NCCL
        _, vs, vl = verify_pick(l5)
        o5, rem5, dq5, dk5, dv5 = res5
        mine = pack_for_check([x[0, vs:vs + vl] for x in (q5, k5, v5, do5, dr5, o5, dq5, dk5, dv5, rem5)])
        if world > 1:
            allv = torch.empty(world * mine.numel(), dtype=torch.float32, device=dev)
            dist.all_gather_into_tensor(allv, mine)
        else:
            allv = mine
        verified, worst = 0, {}
        if rank == 0:
            from oracle import sb_oracle as orc  # the checker, on rank 0 only; nothing timed goes through it
            allv = allv.cpu().numpy().reshape(world, -1)
            for r in range(world):
                a = unpack_check(allv[r], vl, D5)
                want = orc.sb_varlen_fwd_bwd(a["q"][None], a["k"][None], a["v"][None], a["do"][None], a["drem"][None],
                                             np.array([vl]), it5)
                ok = True
                for name, ww in zip(("o", "rem", "dq", "dk", "dv"), want):
                    err = float(np.abs(a[name] - ww[0]).max())
                    worst[name] = max(worst.get(name, 0.0), err)
                    ok &= bool(np.isfinite(a[name]).all()) and err <= TOL_BF16
                verified += int(ok)
        fl5 = flops_fwd_bwd(w5["H"], D5, l5)
        c5 = {"workload": w5["name"], "scaling": "strong", "heads": w5["H"], "heads_per_rank": H5, "tokens": T5,
              "sequences": len(l5), "steps": steps5, "ms_per_step": ms5, "value": fl5 / (ms5 * 1e-3) / 1e12, "unit": UNIT,
              "tokens_per_s": T5 / (ms5 * 1e-3),
              "frac_of_nominal_bf16_peak": fl5 / (ms5 * 1e-3) / 1e12 / (NOMINAL_BF16_TFLOPS * world),
              "inputs": "N(0,1) bf16 generated on the device, dO and drem N(0,1)", "window": win5,
              "verified_ranks": verified,
              "verify": {"sequence_tokens": vl, "tolerance": TOL_BF16, "max_abs_err": worst,
                         "against": "CPU oracle (float64) on rank 0; one sequence of the first head of every shard, "
                                    "gathered over NCCL"}}
        del q5, k5, v5, do5, dr5, res5, o5, rem5, dq5, dk5, dv5
        torch.cuda.empty_cache()

    sampler.stop()
    if rank == 0:
        flops_job = flops_fwd_bwd(wl["H"], D, lengths) * n_jobs
        tokens_job = T * n_jobs
        value = flops_job / (ms_step * 1e-3) / 1e12
        fl_rank = flops_fwd_bwd(H, D, lengths)
        clocks = sampler.result(*win_main)
        for rec in (sustained, c5):
            if rec is not None:
                rec["clocks"] = sampler.result(*rec.pop("window"))
        if sustained is not None:
            sustained["frac_of_measured_sustained_bf16_peak"] = sustained["value"] / (peaks["bf16_tflops_sustained"] * world)
        roofline = None
        if kernels:
            dom = max(kernels, key=kernels.get)
            share = {"fwd": 4.0 / 14.0, "bwd_dq": 5.0 / 14.0, "bwd_dkdv": 5.0 / 14.0}
            # the backward's 10*D flops per pair are split evenly over its two kernels (S and dO V^T are recomputed in both)
            achieved = fl_rank * share[dom] / (kernels[dom] * 1e-3) / 1e12
            peak = peaks["bf16_tflops"]
            roofline = {
                "bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "peak_source": f"of {peaks['source']} (burst cuBLAS bf16)",
                "frac_of_nominal_2250": achieved / NOMINAL_BF16_TFLOPS,
                "traffic": NCU_TRAFFIC_BYTES.get(wl["name"], {}).get(dom),
                "traffic_unit": "bytes per launch on one GPU (ncu: dram read + write)",
                "kernel_ms": kernels,
                "kernel_tflops": {kk: fl_rank * share[kk] / (vv * 1e-3) / 1e12 for kk, vv in kernels.items()},
            }
        cpu = None  # timed at N = 1 only: with more ranks the other processes' polling threads share the host cores
        if "cpu" not in skip and world == 1:
            threads = cpu_threads()
            cpu_seqs = cpu_sample_of(wl)
            cpu_reference_step(wl, cpu_seqs[:1])
            csec, cfl, kind = cpu_reference_step(wl, cpu_seqs)
            cpu = {"value": cfl / csec / 1e12, "unit": UNIT, "cores": threads, "host_cores": os.cpu_count(), "kind": kind,
                   "sample": cpu_sample_text(wl, cpu_seqs, kind)}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if wl["split_heads"] else "weak",
            "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
            "config": {"workload": wl["name"], "heads": wl["H"], "head_dim": D, "tokens": T, "lengths": lengths,
                       "layout": "batched [B,H,T,D]" if batched else "packed [H,T,D]",
                       "inputs": "N(0,1)*%g %s, dO N(0,1), drem 0" % (wl["scale"], wl["dtype"]),
                       "l2": "q,k,v,dO are %d MB per rank (L2 is 126 MB)" % (h2d >> 20),
                       "sharding": ("heads split over ranks" if wl["split_heads"] else "one batch per rank, no collective")},
            "tokens_per_s": tokens_job / (ms_step * 1e-3),
            "frac_of_nominal_bf16_peak": value / (NOMINAL_BF16_TFLOPS * world),
            "frac_of_measured_bf16_peak": value / (peaks["bf16_tflops"] * world),
            "frac_of_measured_bf16_peak_divides_by": "burst cuBLAS bf16 %.0f TFLOP/s per GPU (of %s)" % (
                peaks["bf16_tflops"], peaks["source"]),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps, "gpu_launches_per_step": launches_per_step,
            "clocks": clocks, "sustained": sustained, "short": short, "c5_strong": c5, "graph_replay": graph_rec,
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
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4", "c5", "short", "c1", "b500"])
    ap.add_argument("--heads", type=int, default=0, help="run a subset of the workload's heads (profiling runs)")
    ap.add_argument("--skip", default="", help="comma list of parts to leave out: kernels,e2e,cpu,sustained,c5,short,graph")
    args = ap.parse_args()
    args.skip = set(x for x in args.skip.split(",") if x)
    wl = workload(args.workload)
    if args.heads > 0:
        wl["H"] = args.heads
        wl["name"] += "-heads%d" % args.heads
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
