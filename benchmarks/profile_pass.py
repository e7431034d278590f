#!/usr/bin/env python
"""Run single tile passes of the native FFT backend on one GPU, for profiling.

    python benchmarks/profile_pass.py --size 512 --reps 3
    ncu --set full --clock-control none -k regex:fft_fast -s 2 -c 2 -o prof python benchmarks/profile_pass.py --size 512

Launch order per repetition: one rotating pass (FFT along the last axis +
rotated store), one plain pass (FFT along the last axis, same layout), then
one full pfft3d (rotating, rotating, plain).  Prints CUDA-event timings.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import jaxdecomp_b200 as jd  # noqa: E402
from jaxdecomp_b200.ops import b200_backend, plan  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", type=int, default=512)
    ap.add_argument("--dtype", default="c64", choices=["c64", "c128"])
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--shape", type=int, nargs=3, default=None, help="block shape instead of size^3 "
                    "(the passes transform the last axis)")
    args = ap.parse_args()
    n = args.size
    dt = torch.complex64 if args.dtype == "c64" else torch.complex128
    mesh = jd.single_rank_mesh()
    x = torch.randn(tuple(args.shape) if args.shape else (n, n, n), device="cuda", dtype=dt)
    rot = [plan.Fft(2), plan.Perm(plan.ROT_FWD)]
    pln = [plan.Fft(2)]
    nbytes = 2 * x.numel() * x.element_size()

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    for r in range(args.reps):
        t_rot = timed(lambda: b200_backend.run_steps(x, rot, mesh, False, 1.0))
        t_pln = timed(lambda: b200_backend.run_steps(x, pln, mesh, False, 1.0))
        t_fft = timed(lambda: jd.pfft3d(x, backend="b200"))
        print(f"rep {r}: rotating pass {t_rot:.3f} ms ({nbytes / t_rot / 1e6:.0f} GB/s)  plain pass {t_pln:.3f} ms "
              f"({nbytes / t_pln / 1e6:.0f} GB/s)  pfft3d {t_fft:.3f} ms")
    b200_backend.check_status(mesh, sync=True)


if __name__ == "__main__":
    main()
