"""CIC, k-space operators and the LPT step on CPU: single-process oracles and
eight gloo ranks against the single-process result."""
import math

import pytest
import torch

import jaxdecomp_b200 as jd
from jaxdecomp_b200.models.lpt import LPTConfig, LPTModel, lpt_loss
from jaxdecomp_b200.ops import kspace
from jaxdecomp_b200.ops.cic import cic_paint, cic_readout
from jaxdecomp_b200.utils.testing import run_ranks


def _brute_paint(pos, w, shape, wrap):
    mesh = torch.zeros(shape, dtype=torch.float64)
    for p, ww in zip(pos.tolist(), w.tolist()):
        i = [math.floor(v) for v in p]
        d = [v - math.floor(v) for v in p]
        for c in range(8):
            b = [(c >> k) & 1 for k in range(3)]
            idx, ok, f = [], True, 1.0
            for k in range(3):
                j = i[k] + b[k]
                if wrap[k]:
                    j %= shape[k]
                elif not (0 <= j < shape[k]):
                    ok = False
                idx.append(j)
                f *= d[k] if b[k] else 1 - d[k]
            if ok:
                mesh[tuple(idx)] += ww * f
    return mesh


def test_cic_paint_and_readout_against_brute_force():
    g = torch.Generator().manual_seed(0)
    shape = (6, 5, 7)
    pos = torch.rand((40, 3), generator=g, dtype=torch.float64) * torch.tensor([7.0, 6.0, 9.0]) - 0.5
    w = torch.rand(40, generator=g, dtype=torch.float64)
    for wrap in ((False, False, True), (True, True, True), (False, True, False)):
        mesh = cic_paint(pos, shape, weight=w, wrap=wrap)
        torch.testing.assert_close(mesh, _brute_paint(pos, w, shape, wrap))
        field = torch.rand(shape, generator=g, dtype=torch.float64)
        # paint and read-out are adjoint: <paint(w), field> == <w, readout(field)>
        lhs = (mesh * field).sum()
        rhs = (w * cic_readout(pos, field, wrap=wrap)).sum()
        torch.testing.assert_close(lhs, rhs)
    # mass conservation with full wrap
    torch.testing.assert_close(cic_paint(pos, shape, weight=w, wrap=(True, True, True)).sum(), w.sum())


def test_cic_gradients():
    g = torch.Generator().manual_seed(1)
    shape = (5, 6, 4)
    pos = (torch.rand((12, 3), generator=g, dtype=torch.float64) * 3 + 1.2).requires_grad_(True)
    w = torch.rand(12, generator=g, dtype=torch.float64).requires_grad_(True)
    field = torch.rand(shape, generator=g, dtype=torch.float64).requires_grad_(True)
    assert torch.autograd.gradcheck(lambda p, ww: cic_paint(p, shape, weight=ww, wrap=(False, False, True)), (pos, w))
    assert torch.autograd.gradcheck(lambda p, f: cic_readout(p, f, wrap=(False, True, True)), (pos, field))
    lat = (2, 3, 2)
    disp = (torch.rand((2, 3, 2, 3), generator=g, dtype=torch.float64) * 0.8).requires_grad_(True)
    assert torch.autograd.gradcheck(
        lambda d: cic_paint(d, shape, wrap=(False, False, True), lattice=lat, origin=(1.0, 1.0, 0.0)), (disp,))


def test_kspace_operators_single_rank():
    mesh = jd.single_rank_mesh()
    x = torch.randn((8, 12, 16), dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    k = jd.pfft3d(jd.ShardedTensor(x, mesh))
    box = (8.0, 12.0, 16.0)
    k0, k1, k2 = kspace.wave_numbers(k, box)
    assert k1.shape == (12, 1, 1) and k2.shape == (1, 16, 1) and k0.shape == (1, 1, 8)
    # spectral derivative along original axis 0 equals the analytic one for a single mode
    mode = torch.cos(2 * math.pi * 2 * torch.arange(8, dtype=torch.float64) / 8).view(8, 1, 1).expand(8, 12, 16).contiguous()
    km = jd.pfft3d(jd.ShardedTensor(mode, mesh))
    pots = kspace.displacement_potentials(km, box)
    d0 = jd.pifft3d(pots[0]).local.real
    kval = 2 * math.pi * 2 / 8.0
    want = -torch.sin(2 * math.pi * 2 * torch.arange(8, dtype=torch.float64) / 8).view(8, 1, 1).expand(8, 12, 16) / kval
    torch.testing.assert_close(d0, want, atol=1e-10, rtol=1e-10)
    assert jd.pifft3d(pots[1]).local.abs().max() < 1e-10
    # inverse Laplacian of the Laplacian
    lap = jd.ShardedTensor(k.local * (-(k0 ** 2 + k1 ** 2 + k2 ** 2)), mesh, k.spec)
    back = kspace.inverse_laplacian(lap, box)
    ref = k.local.clone()
    ref[0, 0, 0] = 0
    torch.testing.assert_close(back.local, ref, atol=1e-9, rtol=1e-9)
    # gradcheck of the operators (complex inputs)
    xs = torch.randn((4, 4, 4), dtype=torch.complex128, generator=torch.Generator().manual_seed(3), requires_grad=True)
    ks = jd.ShardedTensor(xs, mesh)
    assert torch.autograd.gradcheck(lambda t: kspace.apply_power_law(jd.ShardedTensor(t, mesh), (4.0,) * 3, 2.0, -1.5, 2.0, 0.5).local, (xs,))
    assert torch.autograd.gradcheck(lambda t: torch.stack([p.local for p in kspace.displacement_potentials(jd.ShardedTensor(t, mesh), (4.0,) * 3)]), (xs,))
    tab = torch.linspace(1.0, 3.0, 16, dtype=torch.float64)
    y = kspace.apply_power_table(ks, (4.0,) * 3, math.log(0.5), 0.2, tab, 1.0)
    assert y.local.shape == xs.shape and torch.isfinite(y.local).all()


def _lpt_reference(noise, cfg):
    """Single-process restatement with torch.fft and a periodic global paint."""
    nc = cfg.nc
    dk = torch.fft.fftn(noise.to(torch.complex128))
    f = torch.fft.fftfreq(nc, d=1.0 / nc, dtype=torch.float64) * (2 * math.pi / cfg.box_size)
    k0, k1, k2 = f.view(-1, 1, 1), f.view(1, -1, 1), f.view(1, 1, -1)
    kk = k0 ** 2 + k1 ** 2 + k2 ** 2
    kabs = kk.sqrt()
    k_nyq = math.pi * nc / cfg.box_size
    p = cfg.amplitude * kabs.clamp_min(1e-30) ** cfg.index * torch.exp(-(kabs / k_nyq) ** 2)
    p = torch.where(kk > 0, p, torch.zeros_like(p))
    dk = dk * (p * (nc / cfg.box_size) ** 3).sqrt()
    inv = torch.where(kk > 0, 1 / kk.clamp_min(1e-30), torch.zeros_like(kk))
    psi = [torch.fft.ifftn(dk * 1j * kd * inv).real * (nc / cfg.box_size) * cfg.growth for kd in (k0, k1, k2)]
    disp = torch.stack(psi, dim=-1)
    return cic_paint(disp, (nc, nc, nc), wrap=(True, True, True), lattice=(nc, nc, nc))


def _lpt_worker(rank, world, pdims):
    mesh = jd.make_mesh(pdims, ("z", "y"))
    cfg = LPTConfig(nc=16, box_size=16.0, halo=4, amplitude=0.05)
    noise_g = torch.randn((16, 16, 16), dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    noise = jd.shard(noise_g, mesh)
    noise.local.requires_grad_(True)
    model = LPTModel(mesh, cfg)
    density = model(noise)
    ng = noise_g.clone().requires_grad_(True)
    ref = _lpt_reference(ng, cfg)
    torch.testing.assert_close(density.gather(), ref.detach(), atol=1e-9, rtol=1e-9)
    assert abs(float(density.gather().sum()) - 16 ** 3) < 1e-6  # mass conservation
    loss = lpt_loss(model, noise)
    loss.backward()
    (ref ** 2).sum().backward()
    torch.testing.assert_close(loss.detach(), (ref ** 2).sum().detach(), atol=1e-8, rtol=1e-10)
    torch.testing.assert_close(noise.local.grad, jd.shard(ng.grad, mesh).local, atol=1e-8, rtol=1e-7)


@pytest.mark.parametrize("pdims", [(2, 4), (1, 8), (8, 1)])
def test_lpt_step_matches_single_process(pdims):
    run_ranks(_lpt_worker, 8, pdims)
