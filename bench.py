#!/usr/bin/env python
"""Benchmark of the BTP forward+backward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one forward + one backward of the btp op over one batch of
synthetic input at the workload BASELINE.json quotes its metric on
(B=1024, H=32, L=128, head_dim 16, bf16; per GPU - weak scaling, the batch is
sharded over ranks and nothing is exchanged on the data path).  Rank 0 prints
one JSON line.

`value`     tokens/s with inputs resident in HBM (CUDA events around K steps).
`e2e`       the same metric with pinned HOST buffers in and out, through the package's
            host-buffer entry `btp_fwd_bwd_host` (batch slices on three streams so that
            upload, kernels and download overlap); H2D of coeff/x/dy and D2H of y/dx/dA are
            inside the timed region.  `via_btp_autograd` is the same through `btp()` +
            autograd with plain copies on one stream.
            `pcie_floor_ms` is the same byte count as plain pinned copies on all ranks at once.
`roofline`  backward kernel (the dominant one): algorithmic bytes / its launch duration,
            measured live with CUDA events (200 back-to-back launches of the kernel between
            two events, median of 5 repeats, right after the headline region).
`extra`     the same kernels at the long-sequence configuration (B=16, H=64, L=8192, float32
            log decays), at the BTP part of the sharded layer configuration (B=64, H=128,
            L=2048) and with the headline's global batch split over the ranks (strong scaling).
`cpu_baseline` the reference's own CPU path (spear/ops/btp/reference.py, staged under
            oracle/_ref; the oracle port only where that is absent) timed on this box's
            host cores, rank 0, N=1 only.

`--impl reference` times that CPU path instead, on host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# workload: BASELINE.json configs[1]/[2]
B, H, L, D = 1024, 32, 128, 16
FWD_BYTES_PER_HT = 66    # x 32 + coeff 2 + y 32          (per head-token, bf16)
BWD_BYTES_PER_HT = 102   # coeff 2 + x 32 + dy 32 + dx 32 + dA 4
NOMINAL_HBM_GBS = 8000.0  # the peak BASELINE.json's north star names
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one backward launch at this workload, from an ncu capture of
# this command with one input set: 276.9 MB read + 114.0 MB written (the remaining 37 MB of the 151 MB of
# output were still in L2 when the single profiled launch ended).
BWD_TRAFFIC_BYTES = 390_839_040
METRIC = "btp_fwd_bwd_tokens_per_s"
UNIT = "tokens/s"


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


COEFF_KIND = "bf16"


def workload_string() -> str:
    """One string for both arms, so that the two JSON lines name the same configuration."""
    which = " (configs[2])" if (B, H, L, COEFF_KIND) == (1024, 32, 128, "bf16") else ""
    coeff = "coeff=exp(-softplus(N(0,1))) bf16" if COEFF_KIND == "bf16" else "coeff=log a~U(-1e-3,0) float32"
    return f"btp fwd+bwd B={B} H={H} L={L} head_dim={D} block=16 per GPU{which}; x~N(0,1/16) bf16, {coeff}, dy~N(0,1) bf16"


def load_cpu_reference():
    """-> (fwd_bwd(a, x, dy), kind, what).

    kind "reference": the reference's own spear/ops/btp/reference.py, staged unmodified under oracle/_ref by
    oracle/stage_reference.py and loaded by file path (the package itself would import the compiled
    extension); block_two_pass_log with autograd, as spear/ops/btp/runners.py:151-163 drives it.
    kind "port": oracle/btp_oracle.py, only where the reference has not been staged."""
    ref_py = os.path.join(ROOT, "oracle", "_ref", "spear", "ops", "btp", "reference.py")
    if os.path.exists(ref_py):
        import importlib.util

        spec = importlib.util.spec_from_file_location("spear_reference_math", ref_py)
        R = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(R)

        def fwd_bwd(a, x, dy):
            a = a.detach().clone().requires_grad_(True)
            x = x.detach().clone().requires_grad_(True)
            y = R.block_two_pass_log(a, x, 16)
            (y * dy).sum().backward()
            return y.detach(), a.grad, x.grad

        return fwd_bwd, "reference", "spear/ops/btp/reference.py block_two_pass_log + autograd (the reference's own code)"
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import btp_oracle as O

    return (lambda a, x, dy: O.btp_forward_backward_autograd(a, x, dy, "log")), "port", \
        "oracle/btp_oracle.py (restatement of block_two_pass_log) + autograd"


def cpu_reference_times(batch: int, reps: int, warm: int):
    """Seconds per fwd+bwd of the CPU path over `batch` batch entries of the workload -> (times, kind, what)."""
    fwd_bwd, kind, what = load_cpu_reference()
    # all the host threads this process may use (torchrun presets OMP_NUM_THREADS=1)
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    g = torch.Generator().manual_seed(0)
    a = torch.exp(-torch.nn.functional.softplus(torch.randn(batch, H, L, generator=g))).bfloat16().float()
    x = (torch.randn(batch, H, D, L, generator=g) * 0.25).bfloat16().float()
    dy = torch.randn(batch, H, D, L, generator=g).bfloat16().float()
    times = []
    for i in range(warm + reps):
        t0 = time.perf_counter()
        fwd_bwd(a, x, dy)
        t1 = time.perf_counter()
        if i >= warm:
            times.append(t1 - t0)
    return times, kind, what


def run_reference_arm(args, rank):
    """The reference's CPU path on this box's host cores; rank 0 only."""
    if rank != 0:
        return
    # size the per-step sample so that the whole run stays within about two minutes
    probe = min(cpu_reference_times(8, 1, 1)[0])
    per_seq = probe / 8
    seconds_per_step = 120.0 / max(1, args.steps + args.warmup)
    batch = int(max(1, min(B, seconds_per_step / per_seq)))
    times, kind, what = cpu_reference_times(batch, args.steps, args.warmup)
    threads = torch.get_num_threads()
    total = sum(times)
    value = batch * L * len(times) / total
    line = {
        "impl": "reference",
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_string(),
                   "step": f"CPU fwd+bwd over a sample of {batch} of the {B} batch entries; {what}"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind,
                         "sample": f"{batch}/{B} batch entries per step, {len(times)} steps, float32 (bf16-rounded inputs), torch CPU autograd"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    global B, H, L, COEFF_KIND
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the other configurations and the strong-scaling line")
    ap.add_argument("--batch", type=int, default=B, help="batch entries per GPU (default: the benchmark workload)")
    ap.add_argument("--heads", type=int, default=H, help="heads (default: the benchmark workload)")
    ap.add_argument("--length", type=int, default=L, help="tokens per sequence (default: the benchmark workload)")
    ap.add_argument("--coeff", default="bf16", choices=["bf16", "f32log"],
                    help="bf16: a = exp(-softplus(N(0,1))) in bf16; f32log: log a ~ U(-1e-3, 0) in float32")
    ap.add_argument("--sets", type=int, default=3, help="rotating input/output sets")
    ap.add_argument("--seam", default="recompute", choices=["recompute", "handoff"],
                    help="how the forward gets the carry across the seams between warps' stretches of a long sequence")
    ap.add_argument("--kernel-launches", type=int, default=200, help="launches per per-kernel timing loop")
    ap.add_argument("--kernel-repeats", type=int, default=5, help="repeats of each per-kernel timing loop")
    args = ap.parse_args()

    B, H, L = args.batch, args.heads, args.length
    COEFF_KIND = args.coeff
    log_coeff = args.coeff == "f32log"
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the BTP path has no CPU fallback)")
    if args.warmup < 3:
        args.warmup = 3
    torch.cuda.set_device(local_rank)
    dist = None
    # Rank 0's stdout carries exactly one JSON line.  Libraries write banners to file descriptor 1 (NCCL
    # prints its version there), so everything else that lands on it during the run is sent to stderr.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from spear_b200 import _btp, _lib
    from spear_b200.ops.btp import btp
    from spear_b200.sharding import batch_shard, bind_to_gpu_numa_node, max_over_ranks, sum_over_ranks

    _lib.load()
    if args.seam == "handoff":
        _lib.set_seam_mode(_lib.SEAM_HANDOFF)
    dev = torch.device("cuda", local_rank)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def over_ranks_max(values):
        return max_over_ranks(values, device=dev) if dist is not None else [float(v) for v in values]

    def make_sets(nb, heads, length, nsets, coeff="bf16"):
        """nsets rotating (coeff, x, dy, y, dx, dA) tuples in the benchmark's distributions."""
        out = []
        for _ in range(nsets):
            x = (torch.randn(nb, heads, D, length, device=dev, generator=gen) * 0.25).bfloat16()
            if coeff == "bf16":  # a = exp(-softplus(N(0,1))), the linear 16-bit form the reference op takes
                a = torch.exp(-torch.nn.functional.softplus(torch.randn(nb, heads, length, device=dev, generator=gen))).bfloat16()
            else:                # "f32log": log a ~ U(-1e-3, 0) in float32 (decays bf16 cannot hold)
                a = -1e-3 * torch.rand(nb, heads, length, device=dev, generator=gen)
            dy = torch.randn(nb, heads, D, length, device=dev, generator=gen).bfloat16()
            out.append((a, x, dy, torch.empty_like(x), torch.empty_like(x), torch.empty(nb, heads, length, device=dev)))
        return out

    def loop_us(launch, n, repeats, idle_s=0.0):
        """n back-to-back launches between two CUDA events on the launching stream, `repeats` times ->
        us per launch of every repeat.  This is the kernel's launch duration the way it runs in a step loop
        (launch latency hidden behind the previous kernel).  With `idle_s` the GPU idles that long before every
        repeat: the kernel timed alone, as a burst, rather than at the clock the loops before it left behind."""
        res = []
        for i in range(3):
            launch(i)
        for _ in range(repeats):
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            if idle_s > 0:
                time.sleep(idle_s)
                for i in range(20):  # a millisecond or two of untimed launches: clocks back up, caches as in the loop
                    launch(i)
                torch.cuda.synchronize()
            g0.record()
            for i in range(n):
                launch(i)
            g1.record()
            torch.cuda.synchronize()
            res.append(g0.elapsed_time(g1) / n * 1e3)
        return res

    # ---- inputs resident in HBM; NSETS rotating sets (each step touches 705 MB, the L2 holds 126 MB)
    NSETS = max(1, args.sets)
    sets = make_sets(B, H, L, NSETS, args.coeff)

    def step(i):
        a, x, dy, y, dx, dA = sets[i % NSETS]
        _btp.forward(a, x, y, None, 2, 32, log_coeff=log_coeff)
        _btp.backward(a, x, dy, None, dx, dA, 2, 32, log_coeff=log_coeff)

    for i in range(args.warmup):
        step(i)
    barrier()

    # ---- timed region 1: K steps back to back (the headline `value`)
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    launches = _lib.launch_count() - launches0
    total_ms = e0.elapsed_time(e1)

    # ---- per-kernel durations, live (a second pass, so that no event record sits inside the headline region):
    #      a fixed number of launches per loop whatever --steps is, several repeats, median and best reported.
    nk, reps = max(1, args.kernel_launches), max(1, args.kernel_repeats)

    def launch_fwd(i):
        a, x, dy, y, dx, dA = sets[i % NSETS]
        _btp.forward(a, x, y, None, 2, 32, log_coeff=log_coeff)

    def launch_bwd(i):
        a, x, dy, y, dx, dA = sets[i % NSETS]
        _btp.backward(a, x, dy, None, dx, dA, 2, 32, log_coeff=log_coeff)

    fwd_runs = loop_us(launch_fwd, nk, reps)
    bwd_runs = loop_us(launch_bwd, nk, reps)
    fwd_us, bwd_us = statistics.median(fwd_runs), statistics.median(bwd_runs)
    # an event on either side of every single launch: includes the launch latency that the records expose
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(nk)]
    for i in range(nk):
        evs[i][0].record()
        launch_fwd(i)
        evs[i][1].record()
        launch_bwd(i)
        evs[i][2].record()
    barrier()
    clocks = sampler.stop()
    # the same loops as bursts: 0.3 s of idle before each repeat (extra keys; `frac` stays on the loops above, and
    # the clock record, which ends here, covers those and the timed steps)
    fwd_burst = statistics.median(loop_us(launch_fwd, nk, reps, idle_s=0.3))
    bwd_burst = statistics.median(loop_us(launch_bwd, nk, reps, idle_s=0.3))
    fwd_single_us = statistics.mean(e[0].elapsed_time(e[1]) for e in evs) * 1e3
    bwd_single_us = statistics.mean(e[1].elapsed_time(e[2]) for e in evs) * 1e3
    _lib.device_status()

    # ---- timed region 2: end to end with pinned host buffers.  With several ranks on the box each rank first moves
    #      to the cores next to its GPU, so that the pinned pages it is about to touch land on that socket's memory.
    numa_cores = bind_to_gpu_numa_node(local_rank) if world > 1 else []
    ha = sets[0][0].cpu().pin_memory()
    hx = sets[0][1].cpu().pin_memory()
    hdy = sets[0][2].cpu().pin_memory()
    hy = torch.empty_like(hx).pin_memory()
    hdx = torch.empty_like(hx).pin_memory()
    hdA = torch.empty(B, H, L, dtype=torch.float32).pin_memory()
    h2d = ha.numel() * 2 + hx.numel() * 2 + hdy.numel() * 2
    d2h = hy.numel() * 2 + hdx.numel() * 2 + hdA.numel() * 4

    def e2e_step():
        a = ha.to(dev, non_blocking=True).requires_grad_(True)
        x = hx.to(dev, non_blocking=True).requires_grad_(True)
        dy = hdy.to(dev, non_blocking=True)
        y = btp(a, x, k=2, output_dtype=torch.bfloat16)
        y.backward(dy)
        hy.copy_(y.detach(), non_blocking=True)
        hdx.copy_(x.grad, non_blocking=True)
        hdA.copy_(a.grad, non_blocking=True)

    from spear_b200.ops.btp import btp_fwd_bwd_host

    def e2e_step_pipelined():  # the host-buffer entry of the package
        btp_fwd_bwd_host(ha, hx, hdy, hy, hdx, hdA, k=2)

    # the floor the link sets: the step's bytes as plain pinned copies, both directions at once on two streams,
    # on every rank at the same time (no kernels)
    s_up, s_down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    d_in = [torch.empty_like(t, device=dev) for t in (ha, hx, hdy)]
    d_out = [torch.empty_like(t, device=dev) for t in (hy, hdx, hdA)]

    def copies_only():
        cur = torch.cuda.current_stream(dev)
        s_up.wait_stream(cur)
        s_down.wait_stream(cur)
        with torch.cuda.stream(s_up):
            for d, h in zip(d_in, (ha, hx, hdy)):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s_down):
            for d, h in zip(d_out, (hy, hdx, hdA)):
                h.copy_(d, non_blocking=True)
        cur.wait_stream(s_up)
        cur.wait_stream(s_down)

    def time_e2e(fn):
        for _ in range(3):
            fn()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(args.e2e_steps):
            fn()
        f1.record()
        barrier()
        return f0.elapsed_time(f1)

    e2e_ms = e2e_autograd_ms = floor_ms = float("nan")
    if log_coeff:
        args.e2e_steps = 0  # the host-buffer entry takes linear coefficients
    if args.e2e_steps > 0:
        e2e_autograd_ms = time_e2e(e2e_step)
        e2e_ms = time_e2e(e2e_step_pipelined)
        floor_ms = time_e2e(copies_only)
    del d_in, d_out

    # ---- the other benchmark configurations and the strong-scaling line (extra keys; the headline stays as it is)
    extra = {}
    if not args.no_extra:
        del sets
        torch.cuda.empty_cache()
        n_x = max(20, nk // 2)

        def plain_pair(nb, heads, length, coeff, log_coeff, forward_only=False):
            ss = make_sets(nb, heads, length, 2, coeff)

            def f(i):
                a, x, dy, y, dx, dA = ss[i % 2]
                _btp.forward(a, x, y, None, 2, 32, log_coeff=log_coeff)

            def b(i):
                a, x, dy, y, dx, dA = ss[i % 2]
                _btp.backward(a, x, dy, None, dx, dA, 2, 32, log_coeff=log_coeff)

            def fb(i):
                f(i)
                b(i)

            r = [statistics.median(loop_us(fn, n_x, 3)) for fn in ((f,) if forward_only else (f, b, fb))]
            r.extend(_lib.last_launch())  # CTAs and cluster size of the last launch (the forward's when forward_only)
            del ss
            torch.cuda.empty_cache()
            return r

        # what a launch of the forward kernel's size can reach at all: a plain device copy of x-sized tensors
        # (read 2 B, write 2 B per element) in the same kind of loop
        cs = [(torch.randn(1024, 32, D, 128, device=dev, generator=gen).bfloat16(),
               torch.empty(1024, 32, D, 128, device=dev, dtype=torch.bfloat16)) for _ in range(3)]
        copy_us = over_ranks_max([statistics.median(loop_us(lambda i: cs[i % 3][1].copy_(cs[i % 3][0]), nk, 3))])[0]
        copy_bytes = 2 * cs[0][0].numel() * 2
        del cs
        torch.cuda.empty_cache()
        # configs[3]: long sequences, near-unit decays given as float32 log a (4 more bytes per head-token)
        _lib.set_seam_mode(_lib.SEAM_RECOMPUTE)  # the extras are quoted on the default kernels whatever --seam says
        f3, b3, s3 = over_ranks_max(plain_pair(16, 64, 8192, "f32log", True)[:3])
        # the same forward with the carry handed over between CTAs of a cluster instead of recomputed at the seams
        f3r, grid_r, _ = plain_pair(16, 64, 8192, "f32log", True, forward_only=True)
        _lib.set_seam_mode(_lib.SEAM_HANDOFF)
        try:
            f3h, grid_h, cluster_h = plain_pair(16, 64, 8192, "f32log", True, forward_only=True)
        finally:
            _lib.set_seam_mode(_lib.SEAM_RECOMPUTE)
        f3r, f3h = over_ranks_max([f3r, f3h])
        # the BTP part of configs[4] (Phalanx layer, dim 2048, L 2048, global batch 64) in the plain layout
        nb4 = 64
        f4, b4, s4 = over_ranks_max(plain_pair(nb4, 128, 2048, "bf16", False)[:3])
        # strong scaling of the headline workload: the global batch of 1024 split over the ranks
        lo, hi = batch_shard(1024, rank, world)
        fs, bs, ss_ = over_ranks_max(plain_pair(hi - lo, H, L, "bf16", False)[:3])
        _lib.device_status()
        extra = {"world": world, "loop": f"{n_x} launches between two CUDA events, median of 3, slowest rank; 2 rotating sets"}

        def cfg_line(label, nb, heads, length, fb_, bb_, f_us, b_us, s_us):
            ht_ = nb * heads * length
            return {"workload": label, "fwd_us": f_us, "bwd_us": b_us, "fwd_bwd_us": s_us,
                    "fwd_gbs": fb_ * ht_ / f_us / 1e3, "bwd_gbs": bb_ * ht_ / b_us / 1e3,
                    "fwd_bwd_gbs": (fb_ + bb_) * ht_ / s_us / 1e3,
                    "tokens_per_s_per_gpu": nb * length / (s_us * 1e-6)}

        extra["same_size_copy"] = {
            "what": "torch copy_ of a [1024,32,16,128] bf16 tensor (268 MB read + written), the practical ceiling for a launch "
                    "of the forward kernel's size; the roofline peak is the rate of a 4 GiB copy",
            "us_per_launch": copy_us, "gbs": copy_bytes / copy_us / 1e3}
        extra["configs3"] = cfg_line("btp fwd+bwd B=16 H=64 L=8192 per GPU, float32 log a ~ U(-1e-3,0), bf16 x/dy",
                                     16, 64, 8192, FWD_BYTES_PER_HT + 2, BWD_BYTES_PER_HT + 2, f3, b3, s3)
        extra["configs3"]["seam"] = {
            "what": "forward alone, the carry across the seams between warps' stretches recomputed from the block to the "
                    "left (default) against handed over through distributed shared memory in a thread-block cluster",
            "recompute_fwd_us": f3r, "recompute_grid": grid_r,
            "handoff_fwd_us": f3h, "handoff_grid": grid_h, "handoff_cluster": cluster_h}
        extra["configs4_btp_part"] = cfg_line("btp fwd+bwd B=64 H=128 L=2048 per GPU, bf16 (plain layout)",
                                              nb4, 128, 2048, FWD_BYTES_PER_HT, BWD_BYTES_PER_HT, f4, b4, s4)
        extra["strong_scaling"] = {
            "workload": f"btp fwd+bwd global B=1024 H={H} L={L} split over {world} GPU(s)", "batch_per_gpu": hi - lo,
            "fwd_us": fs, "bwd_us": bs, "fwd_bwd_us": ss_, "tokens_per_s": 1024 * L / (ss_ * 1e-6),
            "limiter": "per-launch host cost and launch latency once a rank's share drops below a few hundred sequences per SM wave",
        }

    # ---- max over ranks
    if dist is not None:
        (total_ms, e2e_ms, e2e_autograd_ms, floor_ms, fwd_us, bwd_us, fwd_single_us, bwd_single_us, fwd_burst,
         bwd_burst) = max_over_ranks([total_ms, e2e_ms, e2e_autograd_ms, floor_ms, fwd_us, bwd_us, fwd_single_us,
                                      bwd_single_us, fwd_burst, bwd_burst], device=dev)
        launches = int(sum_over_ranks([launches], device=dev)[0])

    if rank == 0:
        peak, peak_kind = measured_peak()
        ht = B * H * L
        fwd_b, bwd_b = FWD_BYTES_PER_HT + (2 if log_coeff else 0), BWD_BYTES_PER_HT + (2 if log_coeff else 0)
        bwd_gbs = bwd_b * ht / (bwd_us * 1e-6) / 1e9
        fwd_gbs = fwd_b * ht / (fwd_us * 1e-6) / 1e9
        step_us = total_ms * 1e3 / args.steps
        step_gbs = (fwd_b + bwd_b) * ht / (step_us * 1e-6) / 1e9
        value = world * B * L * args.steps / (total_ms * 1e-3)
        for v in extra.values():
            if isinstance(v, dict) and "fwd_gbs" in v:
                for key in ("fwd", "bwd", "fwd_bwd"):
                    v[key + "_frac_of_measured"] = v[key + "_gbs"] / peak
        e2e_value = world * B * L * args.e2e_steps / (e2e_ms * 1e-3)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": workload_string(),
                "l2": f"each step touches {(fwd_b + bwd_b) * B * H * L / 1e6:.0f} MB (L2 holds 126 MB) and {NSETS} input/output sets rotate",
                "parallelism": f"batch sharded over {world} GPU(s), no data-path collective",
                "seam": args.seam,
            },
            "e2e": {"value": e2e_value, "unit": UNIT, "per_gpu": e2e_value / world,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / max(1, args.e2e_steps),
                    "pcie_floor_ms": floor_ms / max(1, args.e2e_steps),
                    "pcie_floor": f"the same bytes as plain pinned copies, both directions at once, on all {world} rank(s) at the same time",
                    "frac_of_pcie_floor": floor_ms / e2e_ms,
                    "host_placement": (f"rank 0 bound to {len(numa_cores)} cores next to its GPU before pinning its buffers"
                                       if numa_cores else "default placement"),
                    "api": "spear_b200.ops.btp.btp_fwd_bwd_host (pinned host tensors in and out, batch slices on 3 streams)",
                    "via_btp_autograd": {"value": world * B * L * args.e2e_steps / (e2e_autograd_ms * 1e-3), "unit": UNIT,
                                         "api": "tensor.to(device) + btp() + backward() + copy_ to host, one stream"}},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "btp_backward_kernel", "achieved": bwd_gbs, "peak": peak,
                         "unit": "GB/s", "frac": bwd_gbs / peak,
                         "traffic": BWD_TRAFFIC_BYTES if (B, H, L) == (1024, 32, 128) else None,
                         "peak_kind": f"of {peak_kind}", "us_per_launch": bwd_us, "us_per_launch_best": min(bwd_runs),
                         "frac_best_repeat": bwd_b * ht / (min(bwd_runs) * 1e-6) / 1e9 / peak,
                         "us_per_launch_burst": bwd_burst, "frac_burst": bwd_b * ht / (bwd_burst * 1e-6) / 1e9 / peak,
                         "us_per_launch_runs": bwd_runs,
                         "us_per_launch_between_event_records": bwd_single_us,
                         "method": f"{nk} back-to-back launches of the kernel between two CUDA events on the launching stream, "
                                   f"median of {reps} repeats (frac_best_repeat: the best of them, the way the measured "
                                   "peak is the best of 10 copies; frac_burst: the same loops, median, each after 0.3 s of idle)",
                         "algorithmic_bytes_per_launch": bwd_b * ht},
            "roofline_forward": {"bound": "hbm", "kernel": "btp_forward_kernel", "achieved": fwd_gbs, "peak": peak,
                                 "unit": "GB/s", "frac": fwd_gbs / peak, "us_per_launch": fwd_us,
                                 "us_per_launch_best": min(fwd_runs), "us_per_launch_runs": fwd_runs,
                                 "frac_best_repeat": fwd_b * ht / (min(fwd_runs) * 1e-6) / 1e9 / peak,
                                 "us_per_launch_burst": fwd_burst,
                                 "frac_burst": fwd_b * ht / (fwd_burst * 1e-6) / 1e9 / peak,
                                 "us_per_launch_between_event_records": fwd_single_us,
                                 "algorithmic_bytes_per_launch": fwd_b * ht},
            "step_hbm": {"achieved_gbs": step_gbs, "frac_of_measured": step_gbs / peak,
                         "frac_of_nominal_8TBs": step_gbs / NOMINAL_HBM_GBS, "us_per_step": step_us},
        }
        if extra:
            line["extra"] = extra
        if world == 1 and not args.no_cpu_baseline:
            nb = B  # the full batch: a few seconds of CPU work per repetition
            times, kind, what = cpu_reference_times(nb, 3, 1)
            line["cpu_baseline"] = {
                "value": nb * L / min(times), "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
                "sample": f"{nb}/{B} batch entries, fwd+bwd float32 torch CPU autograd, best of 3 after 1 warm-up; {what}",
            }
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
