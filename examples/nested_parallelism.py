#!/usr/bin/env python
"""Nested parallelism: independent FFT groups on a 3-D mesh, on eight CPU ranks.

    python examples/nested_parallelism.py

A mesh may have leading axes in front of the two decomposition axes.  Ranks that share their leading
coordinates form a decomposition group of their own: each group transforms its own fields, exchanges data
only inside the group (its own process sub-groups on the baseline backend, its own peer-visible workspace
and barriers on the native one) and never waits for another group.  On top of that every op takes a local
batch dimension, and ``torch.func.vmap`` maps over it.  This is the ensemble / data-parallel pattern of
the reference's ``examples/03-nested-parallelism.ipynb`` (``vmap`` over a leading mesh axis 'c'; the HLO there
shows ``replica_groups={{0,1},{2,3},...}``); the printed output is reproduced in
``docs/examples/nested_parallelism.md``.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import jaxdecomp_b200 as jd  # noqa: E402
from jaxdecomp_b200.utils.testing import run_ranks  # noqa: E402


def work(rank, world):
    def everyone(msg):
        # print in rank order
        for r in range(world):
            if r == rank:
                print(msg, flush=True)
            dist.barrier()

    say = print if rank == 0 else (lambda *a, **k: None)

    say("=== 1. a 3-D mesh: 2 groups ('c') of 2 x 2 ranks ('z', 'y') ===")
    mesh = jd.Mesh((2, 2, 2), ("c", "z", "y"))
    group = mesh.coords[0]
    everyone(f"rank {rank}: mesh coordinates {mesh.coords} -> group {group}, pdims {mesh.pdims}, "
             f"ranks of my group {mesh.submesh_ranks()}, my row {mesh.axis_ranks('y')}, my column {mesh.axis_ranks('z')}")

    say("\n=== 2. every group owns a different ensemble member (a batch of 3 fields each) ===")
    fields = torch.randn((3, 16, 16, 16), generator=torch.Generator().manual_seed(100 + group))
    x = jd.shard(fields, mesh, (None, "z", "y", None))          # batch local, grid sharded inside the group
    say("x:", x)
    k = jd.pfft3d(x)
    say("pfft3d(x):", k)
    ref = torch.fft.fftn(fields.to(torch.complex64), dim=(1, 2, 3)).permute(0, 2, 3, 1)
    offs = k.offsets
    mine = ref[:, offs[1]:offs[1] + k.local.shape[1], offs[2]:offs[2] + k.local.shape[2], :]
    everyone(f"rank {rank} (group {group}): my block of my group's transform matches fftn of my group's fields: "
             f"{torch.allclose(k.local, mine, atol=1e-3)}")

    say("\n=== 3. the same as a vmap over the batch ===")
    with mesh:
        kv = torch.func.vmap(jd.pfft3d)(x.local)
    say("vmap(pfft3d)(x.local) equals the batched call:", torch.equal(kv, k.local))

    say("\n=== 4. groups are independent: only group 1 calls an op, group 0 does something else ===")
    if group == 1:
        y = jd.transposeXtoY(x)
        msg = f"transposed to {tuple(y.local.shape)} spec {tuple(y.spec)}"
    else:
        msg = f"computed a local reduction instead: {float(x.local.sum()):.3f}"
    everyone(f"rank {rank} (group {group}): {msg}")

    say("\n=== 5. halo exchange and a gradient inside the groups ===")
    h = jd.halo_exchange(jd.pad_halo(x, (1, 1)), (1, 1), (True, True))
    say("padded + exchanged:", h)
    xl = x.local.clone().requires_grad_(True)
    kk = jd.pfft3d(jd.ShardedTensor(xl, mesh, x.spec))
    loss = (kk.local.abs() ** 2).sum()
    dist.all_reduce(loss_all := loss.detach().clone(), group=mesh.submesh_group())   # sum over MY group only
    loss.backward()
    everyone(f"rank {rank} (group {group}): sum |F x|^2 over my group = {float(loss_all):.1f} "
             f"(Parseval: {float(16 ** 3 * (fields ** 2).sum()):.1f}); grad == 2 N x: "
             f"{torch.allclose(xl.grad, 2 * 16 ** 3 * x.local, rtol=1e-3, atol=1e-1)}")

    say("\n=== 6. round trip ===")
    back = jd.pifft3d(k)
    everyone(f"rank {rank}: round trip error {float((back.local.real - x.local).abs().max()):.2e}")


if __name__ == "__main__":
    run_ranks(work, 8)
