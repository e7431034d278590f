#!/usr/bin/env python
"""Solve the periodic Poisson equation  laplace(phi) = rho  with distributed FFTs.

    python examples/spectral_poisson.py                      # one process (CPU or one GPU)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 examples/spectral_poisson.py --pdims 2x4 --size 64

Shows the pieces a spectral solver needs: `pfft3d` (output in the rotated layout), the wave numbers of that
layout from `fftfreq3d`, a pointwise operation on the local block, and `pifft3d` back to the input layout.
The result is checked against the analytic solution of a plane-wave source.
"""
import argparse
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import jaxdecomp_b200 as jd  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", type=int, default=32)
    ap.add_argument("--pdims", default=None, help="process grid P0xP1 (default 1xWORLD_SIZE)")
    args = ap.parse_args()
    device = jd.init_distributed()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    pdims = tuple(int(v) for v in args.pdims.split("x")) if args.pdims else (1, world)
    mesh = jd.make_mesh(pdims, ("z", "y")) if world > 1 else jd.single_rank_mesh()
    n = args.size

    # rho(x) = cos(2 pi (2 x0 + 3 x1 + x2) / n): the solution is -rho / |k|^2 with k = 2 pi (2, 3, 1) / n
    idx = [torch.arange(n, dtype=torch.float64) for _ in range(3)]
    phase = 2 * math.pi / n * (2 * idx[0][:, None, None] + 3 * idx[1][None, :, None] + idx[2][None, None, :])
    rho_global = torch.cos(phase).to(torch.complex128)
    rho = jd.shard(rho_global.to(device), mesh)

    rho_k = jd.pfft3d(rho)
    k0, k1, k2 = jd.fftfreq3d(rho_k)               # wave numbers of the original axes 0, 1, 2 (grid spacing 1)
    k2sum = k0 ** 2 + k1 ** 2 + k2 ** 2
    inv = torch.where(k2sum > 0, -1.0 / k2sum.clamp_min(1e-30), torch.zeros_like(k2sum))
    phi_k = jd.ShardedTensor(rho_k.local * inv, mesh, rho_k.spec)
    phi = jd.pifft3d(phi_k)

    kk = (2 * math.pi / n) ** 2 * (4 + 9 + 1)
    want = jd.shard((-rho_global / kk).to(device), mesh)
    err = (phi.local - want.local).abs().max().item()
    if mesh.rank == 0:
        print(f"max abs error against the analytic solution: {err:.3e}")
    assert err < 1e-10
    jd.finalize()


if __name__ == "__main__":
    main()
