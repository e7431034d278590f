#!/usr/bin/env python
"""Distributed first-order LPT (Zel'dovich) simulation: white noise -> coloured
initial conditions -> displacements -> cloud-in-cell density, with one `.npy`
per rank for the initial conditions and the final field.

Single GPU or CPU:      python examples/lpt_nbody_demo.py --nc 128
Several GPUs (torchrun): python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
                             examples/lpt_nbody_demo.py --nc 512 --pdims 2x4 --halo-size 32

Counterpart of the reference's examples/lpt_nbody_demo.py (argparse at lines
265-271, per-rank dumps at 256-257); files written here can be assembled with
jaxdecomp_b200.utils.checkpoint.assemble().
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import jaxdecomp_b200 as jd  # noqa: E402
from jaxdecomp_b200.models.lpt import LPTConfig, LPTModel  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--pdims", default=None, help="process grid P0xP1 (default 1xWORLD)")
    ap.add_argument("--nc", type=int, default=128)
    ap.add_argument("--box-size", type=float, default=None)
    ap.add_argument("--halo-size", type=int, default=16)
    ap.add_argument("--output", default="out_lpt")
    ap.add_argument("--grad", action="store_true", help="also compute d sum(density^2) / d noise")
    args = ap.parse_args()

    device = jd.init_distributed()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    pdims = tuple(int(v) for v in args.pdims.lower().split("x")) if args.pdims else (1, world)
    mesh = jd.make_mesh(pdims, ("x", "y"))
    nc = args.nc
    cfg = LPTConfig(nc=nc, box_size=args.box_size or float(nc), halo=args.halo_size, amplitude=0.02)
    gen = torch.Generator(device=device).manual_seed(42 + mesh.rank)
    noise = jd.ShardedTensor(torch.randn((nc // pdims[0], nc // pdims[1], nc), generator=gen, device=device,
                                         requires_grad=args.grad), mesh)
    model = LPTModel(mesh, cfg)
    initial, final = model(noise, return_initial_conditions=True)
    jd.save_sharded(initial, args.output, "initial_conditions")
    jd.save_sharded(final, args.output, "field")
    total = jd.ShardedTensor(final.local, mesh).global_sum()
    if mesh.rank == 0:
        print(f"painted mass {float(total):.1f} (expected {nc ** 3}); wrote per-rank files to {args.output}/")
    if args.grad:
        loss = jd.ShardedTensor(final.local ** 2, mesh).global_sum()
        loss.backward()
        if mesh.rank == 0:
            print(f"loss {float(loss):.6e}, |grad| on rank 0 = {float(noise.local.grad.norm()):.4e}")
    jd.finalize()


if __name__ == "__main__":
    main()
