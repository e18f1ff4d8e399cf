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
`roofline`  backward kernel (the dominant one): algorithmic bytes / its mean launch
            duration, measured live with CUDA events (200 back-to-back launches of the
            kernel between two events, right after the headline region).
`cpu_baseline` the CPU oracle (a restatement of the reference's PyTorch path)
            timed on this box's host cores, rank 0, N=1 only.

`--impl reference` times the reference's CPU path instead (the oracle port:
the reference is Python and cannot travel to the GPU box), on host cores.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one backward launch at this workload
# (ncu capture summarised in profiles/btp_fwd_bwd_B1024_H32_L128_ncu_full.md: 276.9 MB read + 117.5 MB written;
# the remaining 33.5 MB of the 151 MB of output were still in L2 when the single profiled launch ended).
BWD_TRAFFIC_BYTES = 394_406_144
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


def cpu_reference_tokens_per_s(batch: int, reps: int, warm: int):
    """fwd+bwd of the CPU oracle (restatement of spear/ops/btp/reference.py block_two_pass_log with
    autograd, as spear/ops/btp/runners.py:151-163 uses it) on `batch` sequences-batches of the workload."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import btp_oracle as O

    # all the host threads this process may use (torchrun presets OMP_NUM_THREADS=1)
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    g = torch.Generator().manual_seed(0)
    a = torch.sigmoid(torch.randn(batch, H, L, generator=g))
    x = torch.randn(batch, H, D, L, generator=g) * 0.25
    dy = torch.randn(batch, H, D, L, generator=g)
    times = []
    for i in range(warm + reps):
        t0 = time.perf_counter()
        O.btp_forward_backward_autograd(a, x, dy, "log")
        t1 = time.perf_counter()
        if i >= warm:
            times.append(t1 - t0)
    return times


def run_reference_arm(args, rank):
    """The reference's CPU path (oracle port) on this box's host cores; rank 0 only."""
    if rank != 0:
        return
    # size the per-step sample so that the whole run stays within about two minutes
    probe = min(cpu_reference_tokens_per_s(8, 1, 1))
    per_seq = probe / 8
    seconds_per_step = 120.0 / max(1, args.steps + args.warmup)
    batch = int(max(1, min(B, seconds_per_step / per_seq)))
    times = cpu_reference_tokens_per_s(batch, args.steps, args.warmup)
    threads = torch.get_num_threads()
    total = sum(times)
    value = batch * L * len(times) / total
    line = {
        "impl": "reference",
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"btp fwd+bwd B={B} H={H} L={L} head_dim={D} block=16 (configs[2])",
                   "step": f"CPU fwd+bwd over a sample of {batch} of the {B} batch entries"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{batch}/{B} batch entries per step, {len(times)} steps, float32, torch CPU autograd"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    global B
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=B, help="batch entries per GPU (default: the benchmark workload)")
    ap.add_argument("--sets", type=int, default=3, help="rotating input/output sets")
    args = ap.parse_args()

    B = args.batch
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

    _lib.load()
    dev = torch.device("cuda", local_rank)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)

    # ---- inputs resident in HBM; NSETS rotating sets (each step touches 705 MB, the L2 holds 126 MB)
    NSETS = max(1, args.sets)
    sets = []
    for _ in range(NSETS):
        x = (torch.randn(B, H, D, L, device=dev, generator=gen) * 0.25).bfloat16()
        a = torch.exp(-torch.nn.functional.softplus(torch.randn(B, H, L, device=dev, generator=gen))).bfloat16()
        dy = torch.randn(B, H, D, L, device=dev, generator=gen).bfloat16()
        sets.append((a, x, dy, torch.empty_like(x), torch.empty_like(x), torch.empty(B, H, L, device=dev)))

    def step(i):
        a, x, dy, y, dx, dA = sets[i % NSETS]
        _btp.forward(a, x, y, None, 2, 32)
        _btp.backward(a, x, dy, None, dx, dA, 2, 32)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

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

    # ---- per-kernel durations, live (a second pass, so that no event record sits inside the headline region).
    #      (a) nk launches of ONE kernel back to back between two events: total / nk is that kernel's average
    #          launch duration the way it runs in the step loop (launch latency hidden behind the previous kernel);
    #      (b) an event on either side of every single launch: includes the launch latency that the event records
    #          expose, reported beside (a) for reference.
    nk = min(args.steps, 200)

    def same_kernel_loop(launch):
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(3):
            launch(i)
        g0.record()
        for i in range(nk):
            launch(i)
        g1.record()
        torch.cuda.synchronize()
        return g0.elapsed_time(g1) / nk * 1e3

    def launch_fwd(i):
        a, x, dy, y, dx, dA = sets[i % NSETS]
        _btp.forward(a, x, y, None, 2, 32)

    def launch_bwd(i):
        a, x, dy, y, dx, dA = sets[i % NSETS]
        _btp.backward(a, x, dy, None, dx, dA, 2, 32)

    fwd_us = same_kernel_loop(launch_fwd)
    bwd_us = same_kernel_loop(launch_bwd)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(nk)]
    for i in range(nk):
        evs[i][0].record()
        launch_fwd(i)
        evs[i][1].record()
        launch_bwd(i)
        evs[i][2].record()
    barrier()
    clocks = sampler.stop()
    fwd_single_us = statistics.mean(e[0].elapsed_time(e[1]) for e in evs) * 1e3
    bwd_single_us = statistics.mean(e[1].elapsed_time(e[2]) for e in evs) * 1e3
    _lib.device_status()

    # ---- timed region 2: end to end through btp() with pinned host buffers
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

    def e2e_step_pipelined():  # the host-buffer entry of the package: three streams, batch in slices
        btp_fwd_bwd_host(ha, hx, hdy, hy, hdx, hdA, k=2)

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

    e2e_ms = e2e_autograd_ms = float("nan")
    if args.e2e_steps > 0:
        e2e_autograd_ms = time_e2e(e2e_step)
        e2e_ms = time_e2e(e2e_step_pipelined)

    # ---- max over ranks
    if dist is not None:
        from spear_b200.sharding import max_over_ranks, sum_over_ranks

        total_ms, e2e_ms, e2e_autograd_ms, fwd_us, bwd_us, fwd_single_us, bwd_single_us = max_over_ranks(
            [total_ms, e2e_ms, e2e_autograd_ms, fwd_us, bwd_us, fwd_single_us, bwd_single_us], device=dev)
        launches = int(sum_over_ranks([launches], device=dev)[0])

    if rank == 0:
        peak, peak_kind = measured_peak()
        ht = B * H * L
        bwd_gbs = BWD_BYTES_PER_HT * ht / (bwd_us * 1e-6) / 1e9
        fwd_gbs = FWD_BYTES_PER_HT * ht / (fwd_us * 1e-6) / 1e9
        step_us = total_ms * 1e3 / args.steps
        step_gbs = (FWD_BYTES_PER_HT + BWD_BYTES_PER_HT) * ht / (step_us * 1e-6) / 1e9
        value = world * B * L * args.steps / (total_ms * 1e-3)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": f"btp fwd+bwd B={B} H={H} L={L} head_dim={D} block=16 per GPU (configs[2]); "
                            "x~N(0,1/16) bf16, coeff=exp(-softplus(N(0,1))) bf16, dy~N(0,1) bf16",
                "l2": f"each step touches {168 * B * H * L / 1e6:.0f} MB (L2 holds 126 MB) and {NSETS} input/output sets rotate",
                "parallelism": f"batch sharded over {world} GPU(s), no data-path collective",
            },
            "e2e": {"value": world * B * L * args.e2e_steps / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": "spear_b200.ops.btp.btp_fwd_bwd_host (pinned host tensors in and out, 8 batch slices on 3 streams)",
                    "via_btp_autograd": {"value": world * B * L * args.e2e_steps / (e2e_autograd_ms * 1e-3), "unit": UNIT,
                                         "api": "tensor.to(device) + btp() + backward() + copy_ to host, one stream"}},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "btp_backward_kernel", "achieved": bwd_gbs, "peak": peak,
                         "unit": "GB/s", "frac": bwd_gbs / peak,
                         "traffic": BWD_TRAFFIC_BYTES if (B, H, L) == (1024, 32, 128) else None,
                         "peak_kind": f"of {peak_kind}", "us_per_launch": bwd_us,
                         "us_per_launch_between_event_records": bwd_single_us,
                         "method": f"{nk} back-to-back launches of the kernel between two CUDA events on the launching stream",
                         "algorithmic_bytes_per_launch": BWD_BYTES_PER_HT * ht},
            "roofline_forward": {"bound": "hbm", "kernel": "btp_forward_kernel", "achieved": fwd_gbs, "peak": peak,
                                 "unit": "GB/s", "frac": fwd_gbs / peak, "us_per_launch": fwd_us,
                                 "us_per_launch_between_event_records": fwd_single_us,
                                 "algorithmic_bytes_per_launch": FWD_BYTES_PER_HT * ht},
            "step_hbm": {"achieved_gbs": step_gbs, "frac_of_measured": step_gbs / peak,
                         "frac_of_nominal_8TBs": step_gbs / NOMINAL_HBM_GBS, "us_per_step": step_us},
        }
        if world == 1 and not args.no_cpu_baseline:
            nb = B  # the full batch: a few seconds of CPU work per repetition
            times = cpu_reference_tokens_per_s(nb, 3, 1)
            line["cpu_baseline"] = {
                "value": nb * L / min(times), "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                "sample": f"{nb}/{B} batch entries, fwd+bwd float32 torch CPU autograd, best of 3 after 1 warm-up",
            }
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
