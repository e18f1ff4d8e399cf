"""Runs the REFERENCE's own CUDA kernels (built by oracle/build_reference_kernel.sh into oracle/_ref/_btp.so)
next to this repository's kernels on the same seeded inputs: time per launch and relative L2 error against
the float32/float64 oracle.  Test infrastructure, not a product path.

Only shapes whose sequences fit one CTA of the reference kernel (L/16 <= wpb) are run: there its cluster has
one CTA and none of its unbounded cluster-barrier waits is ever entered (csrc/btp/btp-forward.cu:340-347).

    python oracle/compare_reference_kernel.py [--out reference_kernel.json]
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

import btp_oracle as O  # noqa: E402


def load_reference_extension():
    path = os.path.join(HERE, "_ref", "_btp.so")
    if not os.path.exists(path):
        raise SystemExit(f"{path} is missing: run oracle/build_reference_kernel.sh where the reference is mounted")
    spec = importlib.util.spec_from_file_location("_btp", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def timed(fn, iters=30, warm=5):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3  # us


def run(B, H, L, wpb, ref, ours, nsets=3):
    g = torch.Generator(device="cuda").manual_seed(2024)
    sets = []
    for _ in range(nsets):
        x = (torch.randn(B, H, 16, L, device="cuda", generator=g) * 0.25).bfloat16()
        a = torch.sigmoid(torch.randn(B, H, L, device="cuda", generator=g)).bfloat16()
        dy = torch.randn(B, H, 16, L, device="cuda", generator=g).bfloat16()
        sets.append((a, x, dy))
    y = torch.empty_like(sets[0][1])
    dx = torch.empty_like(y)
    dA = torch.zeros(B, H, L, device="cuda")
    ck = torch.empty(B, H, L // 16, 16, device="cuda")
    res = {"B": B, "H": H, "L": L, "wpb": wpb}
    cnt = [0]

    def pick():
        cnt[0] += 1
        return sets[cnt[0] % nsets]

    # ---- errors on a sample of batch entries (same inputs for both kernels)
    a, x, dy = sets[0]
    idx = torch.arange(0, B, max(1, B // 4))[:4]
    a_s, x_s, dy_s = a[idx].float().cpu(), x[idx].float().cpu(), dy[idx].float().cpu()
    y_w = O.btp_forward(a_s.double(), x_s.double(), 2, "product").float()
    dA_w, dx_w = O.btp_backward(a_s.double(), x_s.double(), dy_s.double(), 2, "product")
    for name, mod in (("reference_kernel", ref), ("this_repo", ours)):
        dA.zero_()
        mod.forward(a, x, y, ck, 2, wpb)
        mod.backward(a, x, dy, ck, dx, dA, 2, wpb)
        torch.cuda.synchronize()
        res[name] = {
            "rel_l2_y": O.rel_l2(y[idx].float().cpu(), y_w),
            "rel_l2_dx": O.rel_l2(dx[idx].float().cpu(), dx_w.float()),
            "rel_l2_dA": O.rel_l2(dA[idx].cpu(), dA_w.float()),
        }
    # ---- time per launch
    for name, mod in (("reference_kernel", ref), ("this_repo", ours)):
        def fwd():
            a, x, _ = pick()
            mod.forward(a, x, y, ck, 2, wpb)

        def bwd():
            a, x, dy = pick()
            mod.backward(a, x, dy, ck, dx, dA, 2, wpb)

        res[name]["fwd_us"] = timed(fwd)
        res[name]["bwd_us"] = timed(bwd)
        res[name]["fwd_bwd_tokens_per_s"] = B * L / ((res[name]["fwd_us"] + res[name]["bwd_us"]) * 1e-6)
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    ref = load_reference_extension()
    from spear_b200 import _btp as ours

    results = []
    for B, H, L, wpb in ((1024, 32, 128, 32), (1024, 32, 128, 8), (2, 8, 512, 32)):
        assert L // 16 <= wpb
        r = run(B, H, L, wpb, ref, ours)
        results.append(r)
        print(json.dumps(r), flush=True)
    if args.out:
        json.dump(results, open(args.out, "w"), indent=1)


if __name__ == "__main__":
    main()
