#!/usr/bin/env python
"""Feature tour on eight CPU ranks (gloo backend, no GPU needed).

    python examples/demo_features.py

Walks through everything the library offers, printing what rank 0 sees: meshes and sharded arrays, the
distributed FFT and its rotated output layout, output specs, wave numbers and a spectral derivative, the six
pencil transposes, halo exchange (periodic and not) with the accumulate/reduce variants, gradients and
``torch.func`` transforms, batches, the non-contiguous layout mode, the three normalisations, checkpoints.
The plain-script counterpart of the reference's ``examples/01-demo_features.ipynb``; the printed output is
reproduced in ``docs/examples/feature_tour.md``.  On a GPU box the same calls run the native kernels
(``torchrun --nproc-per-node 8 ...`` with ``jd.init_distributed()`` instead of ``run_ranks``).
"""
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import jaxdecomp_b200 as jd  # noqa: E402
from jaxdecomp_b200.utils.testing import run_ranks  # noqa: E402


def tour(rank, world, tmpdir):
    say = print if rank == 0 else (lambda *a, **k: None)

    def section(title):
        say(f"\n=== {title} " + "=" * max(0, 76 - len(title)))

    # ------------------------------------------------------------------------------------------
    section("1. mesh and sharded arrays")
    mesh = jd.make_mesh((2, 4), ("z", "y"))
    say("mesh:", mesh)
    say("pencil type:", jd.Decomposition(mesh.pencil_type).name, "| this rank's coordinates:", mesh.coords)
    g = torch.randn((32, 32, 32), generator=torch.Generator().manual_seed(0))       # the same array on every rank
    x = jd.shard(g, mesh)                                                           # X-pencil: axis 0 over 'z', axis 1 over 'y'
    say("x:", x)
    say("local block", tuple(x.local.shape), "of global", x.global_shape, "| first element at", x.offsets)
    say("gather() restores the global array:", torch.equal(x.gather(), g))

    # ------------------------------------------------------------------------------------------
    section("2. forward and inverse distributed FFT")
    k = jd.pfft3d(x)
    say("k = pfft3d(x):", k)
    ref = torch.fft.fftn(g.to(torch.complex64)).permute(1, 2, 0)                    # the output layout is (N1, N2, N0)
    say("k equals fftn(x).permute(1, 2, 0):", torch.allclose(k.gather(), ref, atol=1e-3))
    back = jd.pifft3d(k)
    say("pifft3d(k):", back)
    say("round trip error:", float((back.local.real - x.local).abs().max()))
    say("spec predicted without running anything:",
        jd.get_output_specs("fft", mesh.pencil_type, x.spec), "==", tuple(k.spec))
    for norm in ("backward", "ortho", "forward"):
        kn = jd.pfft3d(x, norm=norm)
        say(f"norm={norm!r:10s} |k|_max = {float(kn.local.abs().max()):.4f}")

    # ------------------------------------------------------------------------------------------
    section("3. wave numbers and a spectral derivative")
    k0, k1, k2 = jd.fftfreq3d(k)                                                    # original axes 0, 1, 2
    say("fftfreq3d shapes (broadcast against k.local", tuple(k.local.shape), "):",
        tuple(k0.shape), tuple(k1.shape), tuple(k2.shape))
    wave = torch.sin(2 * torch.pi * 3 * torch.arange(32) / 32).view(32, 1, 1).expand(32, 32, 32).contiguous()
    kw = jd.pfft3d(jd.shard(wave, mesh))
    q0, _, _ = jd.fftfreq3d(kw)
    d_wave = jd.pifft3d(jd.ShardedTensor(kw.local * (1j * q0), mesh, kw.spec)).gather().real
    exact = (2 * torch.pi * 3 / 32) * torch.cos(2 * torch.pi * 3 * torch.arange(32) / 32).view(32, 1, 1).expand(32, 32, 32)
    say("d/dx0 of sin(2 pi 3 x0 / 32): max error", float((d_wave - exact).abs().max()))

    # ------------------------------------------------------------------------------------------
    section("4. pencil transposes")
    y = jd.transposeXtoY(x)
    z = jd.transposeYtoZ(y)
    say("X pencil:", x)
    say("Y pencil:", y)
    say("Z pencil:", z)
    say("Y pencil equals the global permute(2, 0, 1):", torch.equal(y.gather(), g.permute(2, 0, 1)))
    say("Z -> Y -> X restores x exactly:", torch.equal(jd.transposeYtoX(jd.transposeZtoY(z)).local, x.local))
    say("X -> Z in one exchange:", jd.transposeXtoZ(x))
    dest = jd.empty_sharded(mesh, tuple(y.local.shape), y.local.dtype, spec=y.spec)   # peer-visible on GPUs
    jd.transposeXtoY(x, out=dest)
    say("out= writes into a preallocated block (on GPUs the exchange stores straight into it):",
        torch.equal(dest.local, y.local))

    # ------------------------------------------------------------------------------------------
    section("5. halo exchange")
    ranks = jd.ShardedTensor(torch.full((4, 4, 1), float(rank)), mesh)              # every block holds its rank number
    padded = jd.pad_halo(ranks, (1, 1))
    say("padded block of rank 0 before the exchange (zeros in the pads):")
    say(padded.local[:, :, 0])
    ex = jd.halo_exchange(padded, (1, 1), (True, True))
    say("after halo_exchange, periodic: faces and corners hold the neighbours' rank numbers")
    say(ex.local[:, :, 0])
    ex_np = jd.halo_exchange(padded, (1, 1), (False, False))
    say("non-periodic: halos at the edge of the domain are zero")
    say(ex_np.local[:, :, 0])
    ones = jd.ShardedTensor(torch.ones((6, 6, 1)), mesh)
    acc = jd.halo_accumulate(ones, (1, 1), (True, True))
    say("halo_accumulate of a block of ones: pads are folded into the neighbours' interior edges")
    say(acc.local[:, :, 0])
    say("halo_reduce = accumulate + crop:", tuple(jd.halo_reduce(ones, (1, 1), (True, True)).local.shape),
        "| mass conserved:", float(jd.halo_reduce(ones, (1, 1), (True, True)).global_sum()), "==", 36.0 * world)

    # ------------------------------------------------------------------------------------------
    section("6. gradients")
    xl = x.local.clone().requires_grad_(True)
    kk = jd.pfft3d(jd.ShardedTensor(xl, mesh))
    loss = jd.ShardedTensor(kk.local.abs() ** 2, mesh, kk.spec).global_sum()        # a global scalar
    loss.backward()
    say("loss = sum |F x|^2 =", float(loss.detach()), "| Parseval: N * sum x^2 =", float(32 ** 3 * (g ** 2).sum()))
    say("d loss / d x == 2 N x:", torch.allclose(xl.grad, 2 * 32 ** 3 * x.local, rtol=1e-3, atol=1e-1))
    with mesh:
        batch = torch.stack([x.local, 2 * x.local, 3 * x.local])
        kb = torch.func.vmap(jd.pfft3d)(batch)                                      # vmap over a stack of local blocks
    say("vmap(pfft3d) over 3 blocks:", tuple(kb.shape), "| linear in the input:", torch.allclose(kb[2], 3 * kb[0], atol=1e-2))

    # ------------------------------------------------------------------------------------------
    section("7. batches and the non-contiguous layout mode")
    xb = jd.shard(torch.stack([g, -g]), mesh, (None, "z", "y", None))
    say("batched input :", xb)
    say("batched output:", jd.pfft3d(xb))
    jd.config.update("transpose_axis_contiguous", False)
    kn = jd.pfft3d(x)
    say("non-contiguous mode keeps the axis order, the sharded dimensions migrate:", kn)
    say("equals fftn(x) without permutation:", torch.allclose(kn.gather(), torch.fft.fftn(g.to(torch.complex64)), atol=1e-3))
    jd.config.update("transpose_axis_contiguous", True)

    # ------------------------------------------------------------------------------------------
    section("8. slabs, autotuned grid, pencil geometry")
    slab = jd.make_mesh((1, 8), ("z", "y"))
    say("slab mesh:", slab, "->", jd.pfft3d(jd.shard(g, slab)))
    info = jd.get_pencil_info(jd.make_config((32, 32, 32), (2, 4)), 0, coords=mesh.coords)
    say("X-pencil geometry of this rank:", info)

    # ------------------------------------------------------------------------------------------
    section("9. checkpoints")
    jd.save_sharded(k, tmpdir, "delta_k")
    torch.distributed.barrier()
    k_again = jd.load_sharded(tmpdir, mesh, "delta_k")
    say("saved and reloaded:", torch.equal(k_again.local, k.local), "| files:", sorted(os.listdir(tmpdir))[:3], "...")


if __name__ == "__main__":
    with tempfile.TemporaryDirectory() as d:
        run_ranks(tour, 8, d)
