#!/usr/bin/env python
"""Feature tour on eight CPU ranks (gloo): sharded arrays, distributed FFT and
its output layout, wave numbers, pencil transposes, halo exchange, gradients.
The plain-script counterpart of the reference's examples/01-demo_features.ipynb.

    python examples/demo_features.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import jaxdecomp_b200 as jd  # noqa: E402
from jaxdecomp_b200.utils.testing import run_ranks  # noqa: E402


def tour(rank, world):
    say = print if rank == 0 else (lambda *a, **k: None)
    mesh = jd.make_mesh((2, 4), ("z", "y"))
    g = torch.randn((32, 32, 32), generator=torch.Generator().manual_seed(0))
    x = jd.shard(g, mesh)                                    # X-pencil: axis 0 over 'z', axis 1 over 'y'
    say("input    ", x)
    k = jd.pfft3d(x)                                         # forward transform, rotated layout (N1, N2, N0)
    say("pfft3d   ", k)
    say("matches fftn:", torch.allclose(k.gather(), torch.fft.fftn(g.to(torch.complex64)).permute(1, 2, 0), atol=1e-3))
    kz, ky, kx = jd.fftfreq3d(k)                             # wave numbers of original axes 0, 1, 2 for this block
    lap = jd.ShardedTensor(k.local * (-(kz ** 2 + ky ** 2 + kx ** 2)), mesh, k.spec)
    say("laplacian", jd.pifft3d(lap))
    y = jd.transposeXtoY(x)
    z = jd.transposeYtoZ(y)
    say("Y pencil ", y)
    say("Z pencil ", z)
    say("round trip exact:", torch.equal(jd.transposeYtoX(jd.transposeZtoY(z)).local, x.local))
    padded = jd.pad_halo(x, (2, 2))
    exch = jd.halo_exchange(padded, (2, 2), (True, True))
    say("halo     ", exch)
    xl = x.local.clone().requires_grad_(True)
    loss = jd.ShardedTensor(jd.pfft3d(jd.ShardedTensor(xl, mesh)).local.abs() ** 2, mesh).global_sum()
    loss.backward()
    say("d/dx sum|F x|^2 == 2 N x:", torch.allclose(xl.grad, 2 * 32 ** 3 * x.local, rtol=1e-3, atol=1e-1))
    jd.config.update("transpose_axis_contiguous", False)
    say("non-contiguous mode keeps the axis order:", jd.pfft3d(x))


if __name__ == "__main__":
    run_ranks(tour, 8)
