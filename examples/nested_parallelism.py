#!/usr/bin/env python
"""Independent FFT groups on a 3-D mesh: a leading mesh axis 'c' splits the
ranks into groups that each transform their own batch of fields, with a local
batch dimension on top.  Counterpart of the reference's
examples/03-nested-parallelism.ipynb (vmap over a leading mesh axis).

    python examples/nested_parallelism.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import jaxdecomp_b200 as jd  # noqa: E402
from jaxdecomp_b200.utils.testing import run_ranks  # noqa: E402


def work(rank, world):
    mesh = jd.Mesh((2, 2, 2), ("c", "z", "y"))             # 2 groups of 2x2 ranks
    group = mesh.coords[0]
    fields = torch.randn((3, 16, 16, 16), generator=torch.Generator().manual_seed(100 + group))
    x = jd.shard(fields, mesh, (None, "z", "y", None))      # batch of 3 per group, sharded inside the group
    k = jd.pfft3d(x)
    back = jd.pifft3d(k)
    ok = torch.allclose(back.local.real, x.local, atol=1e-4)
    print(f"rank {rank}: group {group}, submesh ranks {mesh.submesh_ranks()}, local k block {tuple(k.local.shape)}, "
          f"round trip ok: {ok}")


if __name__ == "__main__":
    run_ranks(work, 8)
