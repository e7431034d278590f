#!/usr/bin/env python
"""Run the particle-mesh kernels of the LPT step on one GPU, for profiling.

    python benchmarks/profile_lpt.py --size 256 --reps 3
    ncu --set full --clock-control none -k regex:cic_paint -s 2 -c 2 -o prof python benchmarks/profile_lpt.py --size 256

Launch order per repetition: tiled CIC paint of size^3 lattice particles (shared-memory bricks), the plain
atomic paint of the same particles, then the batched inverse transform with the fused i k / k^2 multiplier
(three passes; the first one applies the multiplier while it reads).  Prints CUDA-event timings and, for the
paint kernels, particles per second and the bytes the mesh and the displacements account for.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import jaxdecomp_b200 as jd  # noqa: E402
from jaxdecomp_b200.ops import b200_backend, kspace  # noqa: E402
from jaxdecomp_b200.ops.cic import cic_paint  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", type=int, default=256)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--amplitude", type=float, default=1.5, help="rms displacement in cells")
    args = ap.parse_args()
    n = args.size
    mesh = jd.single_rank_mesh()
    gen = torch.Generator(device="cuda").manual_seed(0)
    disp = torch.randn((3, n, n, n), device="cuda", generator=gen) * args.amplitude
    delta = torch.randn((n, n, n), device="cuda", generator=gen)
    k = jd.pfft3d(jd.ShardedTensor(delta, mesh), backend="b200")

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), out

    def paint():
        return cic_paint(disp, (n, n, n), wrap=(True, True, True), lattice=(n, n, n), planar=True)

    nbytes = 4 * n ** 3 * (3 + 2)          # three displacement components read, every mesh cell read and written once
    for r in range(args.reps):
        os.environ["JD_B200_CIC_TILED"] = "1"
        t_tiled, a = timed(paint)
        os.environ["JD_B200_CIC_TILED"] = "0"
        t_plain, b = timed(paint)
        os.environ.pop("JD_B200_CIC_TILED")
        t_disp, _ = timed(lambda: kspace.inverse_displacements(k, (float(n),) * 3, backend="b200"))
        err = float((a - b).abs().max())
        print(f"rep {r}: tiled paint {t_tiled:.3f} ms ({n ** 3 / t_tiled / 1e6:.2f} G particles/s, {nbytes / t_tiled / 1e6:.0f} GB/s "
              f"of displacement + mesh traffic)  plain paint {t_plain:.3f} ms  max diff {err:.2e}  "
              f"fused inverse displacements {t_disp:.3f} ms")
    b200_backend.check_status(mesh, sync=True)


if __name__ == "__main__":
    main()
