"""Particle-mesh and k-space kernels, and the LPT step, on one GPU: native
kernels against the plain PyTorch restatements (run on the CPU in float64)."""
import math

import pytest
import torch

import jaxdecomp_b200 as jd
from jaxdecomp_b200.models.lpt import LPTConfig, LPTModel, lpt_loss
from jaxdecomp_b200.ops import kspace
from jaxdecomp_b200.ops.cic import cic_paint, cic_readout

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_cic_kernels_match_cpu_reference():
    g = torch.Generator().manual_seed(0)
    shape = (20, 24, 16)
    pos = (torch.rand((5000, 3), generator=g) * torch.tensor([21.0, 25.0, 18.0]) - 0.5)
    w = torch.rand(5000, generator=g)
    field = torch.rand(shape, generator=g)
    for wrap in ((False, False, True), (True, True, True)):
        ref = cic_paint(pos.double(), shape, weight=w.double(), wrap=wrap)
        pd = pos.to(DEV).requires_grad_(True)
        wd = w.to(DEV).requires_grad_(True)
        out = cic_paint(pd, shape, weight=wd, wrap=wrap)
        torch.testing.assert_close(out.cpu().double(), ref, atol=2e-5, rtol=1e-4)
        # gradients of a scalar functional
        fd = field.to(DEV)
        (out * fd).sum().backward()
        pr = pos.double().requires_grad_(True)
        wr = w.double().requires_grad_(True)
        (cic_paint(pr, shape, weight=wr, wrap=wrap) * field.double()).sum().backward()
        torch.testing.assert_close(pd.grad.cpu().double(), pr.grad, atol=2e-4, rtol=1e-3)
        torch.testing.assert_close(wd.grad.cpu().double(), wr.grad, atol=2e-5, rtol=1e-4)
        ro = cic_readout(pos.to(DEV), fd, wrap=wrap)
        torch.testing.assert_close(ro.cpu().double(), cic_readout(pos.double(), field.double(), wrap=wrap), atol=2e-5, rtol=1e-4)
    # grid mode
    lat = (10, 12, 16)
    disp = torch.rand((*lat, 3), generator=g) * 1.5 - 0.75
    a = cic_paint(disp.to(DEV), shape, wrap=(False, False, True), lattice=lat, origin=(5.0, 6.0, 0.0))
    b = cic_paint(disp.double(), shape, wrap=(False, False, True), lattice=lat, origin=(5.0, 6.0, 0.0))
    torch.testing.assert_close(a.cpu().double(), b, atol=2e-5, rtol=1e-4)
    assert abs(float(a.sum()) - 10 * 12 * 16) < 1e-2


def test_tiled_cic_paint_matches_the_plain_kernel_and_the_cpu(monkeypatch):
    """Lattices that split into whole 8 x 8 x 32 bricks take the shared-memory kernel: small displacements
    stay inside a brick's apron, large ones (up to 9 cells here) leave it and go to global memory directly,
    and both wrap and drop at the block edge."""
    g = torch.Generator().manual_seed(3)
    lat = (16, 24, 64)
    for scale, wrap, shape, origin in ((1.5, (False, False, True), (24, 32, 64), (4.0, 4.0, 0.0)),
                                       (18.0, (True, True, True), (16, 24, 64), (0.0, 0.0, 0.0)),
                                       (18.0, (False, False, True), (20, 28, 64), (2.0, 2.0, 0.0))):
        disp = (torch.rand((*lat, 3), generator=g) - 0.5) * scale
        w = torch.rand(lat, generator=g)
        ref = cic_paint(disp.double(), shape, weight=w.double().reshape(-1), wrap=wrap, lattice=lat, origin=origin)
        monkeypatch.setenv("JD_B200_CIC_TILED", "1")
        tiled = cic_paint(disp.to(DEV), shape, weight=w.to(DEV).reshape(-1), wrap=wrap, lattice=lat, origin=origin)
        monkeypatch.setenv("JD_B200_CIC_TILED", "0")
        plain = cic_paint(disp.to(DEV), shape, weight=w.to(DEV).reshape(-1), wrap=wrap, lattice=lat, origin=origin)
        monkeypatch.delenv("JD_B200_CIC_TILED")
        torch.testing.assert_close(tiled.cpu().double(), ref, atol=5e-5, rtol=1e-4)
        torch.testing.assert_close(tiled, plain, atol=5e-5, rtol=1e-4)


def test_kspace_kernels_match_torch():
    mesh = jd.single_rank_mesh()
    x = torch.randn((16, 24, 32), generator=torch.Generator().manual_seed(1))
    box = (16.0, 12.0, 64.0)
    kd = jd.pfft3d(jd.ShardedTensor(x.to(DEV), mesh))
    kc = jd.ShardedTensor(kd.local.cpu().to(torch.complex128), mesh, kd.spec)
    a = kspace.apply_power_law(kd, box, 2.0, -1.7, 1.3, 0.25)
    b = kspace.apply_power_law(kc, box, 2.0, -1.7, 1.3, 0.25)
    torch.testing.assert_close(a.local.cpu().to(torch.complex128), b.local, atol=1e-3, rtol=2e-4)
    for pa, pb in zip(kspace.displacement_potentials(kd, box), kspace.displacement_potentials(kc, box)):
        torch.testing.assert_close(pa.local.cpu().to(torch.complex128), pb.local, atol=1e-3, rtol=2e-4)
    a = kspace.inverse_laplacian(kd, box)
    b = kspace.inverse_laplacian(kc, box)
    torch.testing.assert_close(a.local.cpu().to(torch.complex128), b.local, atol=1e-3, rtol=2e-4)
    tab = torch.linspace(0.5, 2.5, 32)
    a = kspace.apply_power_table(kd, box, math.log(0.05), 0.15, tab, 2.0)
    b = kspace.apply_power_table(kc, box, math.log(0.05), 0.15, tab.double(), 2.0)
    torch.testing.assert_close(a.local.cpu().to(torch.complex128), b.local, atol=1e-3, rtol=5e-4)
    # gradient of the displacement operator uses the adjoint kernel
    xl = kd.local.detach().clone().requires_grad_(True)
    pots = kspace.displacement_potentials(jd.ShardedTensor(xl, mesh, kd.spec), box)
    wts = [torch.randn(xl.shape, device=DEV, dtype=torch.complex64, generator=torch.Generator(device=DEV).manual_seed(i)) for i in range(3)]
    sum((p.local * w).real.sum() for p, w in zip(pots, wts)).backward()
    xr = kc.local.detach().clone().requires_grad_(True)
    potr = kspace.displacement_potentials(jd.ShardedTensor(xr, mesh, kd.spec), box)
    sum((p.local * w.cpu().to(torch.complex128)).real.sum() for p, w in zip(potr, wts)).backward()
    torch.testing.assert_close(xl.grad.cpu().to(torch.complex128), xr.grad, atol=1e-3, rtol=5e-4)


def test_lpt_step_and_gradient_on_gpu():
    mesh = jd.single_rank_mesh()
    cfg = LPTConfig(nc=32, box_size=32.0, halo=4, amplitude=0.05)
    noise_c = torch.randn((32, 32, 32), dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    nd = jd.ShardedTensor(noise_c.float().to(DEV).requires_grad_(True), mesh)
    nc_ = jd.ShardedTensor(noise_c.clone().requires_grad_(True), mesh)
    model = LPTModel(mesh, cfg)
    ld = lpt_loss(model, nd)
    lc = lpt_loss(model, nc_)
    ld.backward()
    lc.backward()
    assert abs(float(ld.detach()) - float(lc.detach())) < 1e-3 * abs(float(lc.detach()))
    g_ref = nc_.local.grad
    err = (nd.local.grad.cpu().double() - g_ref).abs().max() / g_ref.abs().max()
    assert err < 5e-3, float(err)
    dens = model(jd.ShardedTensor(noise_c.float().to(DEV), mesh))
    assert abs(float(dens.local.sum()) - 32 ** 3) < 1.0


def test_fused_inverse_displacements_match_the_unfused_sequence():
    """One batched inverse plan with the multiplier applied in its first pass against potentials formed by
    the k-space kernel and transformed one by one; values and the gradient with respect to delta_k."""
    from jaxdecomp_b200.ops import b200_backend

    mesh = jd.single_rank_mesh()
    box = (16.0, 12.0, 64.0)
    x = torch.randn((32, 16, 128), device=DEV, generator=torch.Generator(device=DEV).manual_seed(4))
    k = jd.pfft3d(jd.ShardedTensor(x, mesh), backend="b200")
    kl = k.local.detach().clone().requires_grad_(True)
    before = b200_backend.launches(mesh)
    psi = kspace.inverse_displacements(jd.ShardedTensor(kl, mesh, k.spec), box, backend="b200")
    assert b200_backend.launches(mesh) - before == 3          # three passes, no separate multiplier kernel
    assert psi.local.shape == (3, 32, 16, 128)
    kr = k.local.detach().clone().requires_grad_(True)
    pots = kspace.displacement_potentials(jd.ShardedTensor(kr, mesh, k.spec), box)
    ref = torch.stack([jd.pifft3d(p, backend="b200").local for p in pots])
    torch.testing.assert_close(psi.local, ref, atol=2e-5, rtol=1e-4)
    w = torch.randn(psi.local.shape, device=DEV, generator=torch.Generator(device=DEV).manual_seed(5))
    (psi.local.real * w).sum().backward()
    (ref.real * w).sum().backward()
    torch.testing.assert_close(kl.grad, kr.grad, atol=2e-5, rtol=1e-4)
    b200_backend.check_status(mesh, sync=True)
