"""Distributed ops on eight CPU ranks (gloo), baseline backend, checked against
single-process torch: forward FFT, round trip, transposes, halos, gradients."""

import pytest
import torch

import jaxdecomp_b200 as jd
from jaxdecomp_b200.utils.testing import run_ranks

PDIMS8 = [(2, 4), (4, 2), (1, 8), (8, 1)]


def _global(shape, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g, dtype=torch.float64)
    if dtype.is_complex:
        x = torch.complex(x, torch.randn(shape, generator=g, dtype=torch.float64))
    return x.to(dtype)


def _fft_worker(rank, world, pdims, shape, contiguous, dtype):
    jd.config.update("transpose_axis_contiguous", contiguous)
    mesh = jd.make_mesh(pdims, ("z", "y"))
    xg = _global(shape, dtype)
    x = jd.shard(xg, mesh)
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.complex64 else dict(rtol=1e-10, atol=1e-10)
    ref = torch.fft.fftn(xg)
    if contiguous:
        ref = ref.permute(1, 2, 0)
    for norm in ("backward", "ortho", "forward"):
        k = jd.pfft3d(x, norm=norm)
        assert k.global_shape == tuple(ref.shape)
        n = xg.numel()
        s = {"backward": 1.0, "ortho": n ** -0.5, "forward": 1.0 / n}[norm]
        torch.testing.assert_close(k.gather(), ref * s, **tol)
        back = jd.pifft3d(k, norm=norm)
        assert back.global_shape == tuple(shape) and tuple(back.spec) == tuple(x.spec)
        torch.testing.assert_close(back.gather(), xg, **tol)
    want = jd.get_output_specs("fft", mesh.pencil_type, x.spec)
    assert tuple(k.spec) == tuple(want), (k.spec, want)
    assert tuple(jd.get_fft_output_sharding(x.sharding).spec) == tuple(want)


@pytest.mark.parametrize("pdims", PDIMS8)
@pytest.mark.parametrize("contiguous", [True, False])
def test_fft_matches_fftn(pdims, contiguous):
    run_ranks(_fft_worker, 8, pdims, (16, 8, 32), contiguous, torch.complex64)


def test_fft_c128_nonpow2_and_real_input():
    run_ranks(_fft_worker, 8, (2, 4), (2 * 6, 4 * 5, 8 * 3), True, torch.complex128)
    run_ranks(_real_worker, 8)


def _real_worker(rank, world):
    mesh = jd.make_mesh((2, 4), ("z", "y"))
    xg = _global((64, 64, 64), torch.float32)
    x = jd.shard(xg, mesh)
    k = jd.pfft3d(x)
    assert k.dtype == torch.complex64
    torch.testing.assert_close(k.gather(), torch.fft.fftn(xg.to(torch.complex64)).permute(1, 2, 0), rtol=1e-4, atol=2e-3)
    back = jd.pifft3d(k)
    torch.testing.assert_close(back.gather().real, xg, rtol=1e-4, atol=1e-4)


def _transpose_worker(rank, world, pdims, contiguous):
    jd.config.update("transpose_axis_contiguous", contiguous)
    mesh = jd.make_mesh(pdims, ("z", "y"))
    for dtype in (torch.float32, torch.float64, torch.complex64, torch.complex128):
        xg = _global((8, 16, 32), dtype, seed=3)
        x = jd.shard(xg, mesh)
        y = jd.transposeXtoY(x)
        z = jd.transposeYtoZ(y)
        y2 = jd.transposeZtoY(z)
        x2 = jd.transposeYtoX(y2)
        if contiguous:
            assert torch.equal(y.gather(), xg.permute(2, 0, 1))
            assert torch.equal(z.gather(), xg.permute(1, 2, 0))
        else:
            assert torch.equal(y.gather(), xg) and torch.equal(z.gather(), xg)
        assert torch.equal(y2.gather(), y.gather())
        assert torch.equal(x2.gather(), xg) and tuple(x2.spec) == tuple(x.spec)
        if pdims[0] > 1 and pdims[1] > 1:
            zz = jd.transposeXtoZ(x)
            assert torch.equal(zz.gather(), xg.permute(1, 2, 0) if contiguous else xg)
            xx = jd.transposeZtoX(zz)
            assert torch.equal(xx.gather(), xg)
        # out=: the result lands in the given tensor (plain or sharded), without autograd
        dest = jd.empty_sharded(mesh, tuple(y.local.shape), dtype, spec=y.spec, peer_visible=False)
        got = jd.transposeXtoY(x, out=dest)
        assert got.local.data_ptr() == dest.local.data_ptr() and torch.equal(dest.local, y.local)
        raw = torch.empty_like(z.local)
        jd.transposeYtoZ(y, out=raw)
        assert torch.equal(raw, z.local)
    xr = jd.ShardedTensor(x.local.real.clone().requires_grad_(True), mesh)
    with pytest.raises(RuntimeError, match="automatic differentiation"):
        jd.transposeXtoY(xr, out=torch.empty_like(jd.transposeXtoY(xr).local))


@pytest.mark.parametrize("pdims,contiguous", [((2, 4), True), ((4, 2), False), ((1, 8), True), ((8, 1), True)])
def test_transposes_chain(pdims, contiguous):
    run_ranks(_transpose_worker, 8, pdims, contiguous)


def _expected_halo(xg_blocks, mesh_shape, coords, h, periods):
    """Recompute one rank's halo result from the padded blocks of all ranks."""
    p0, p1 = mesh_shape
    me = xg_blocks[coords]
    out = me.clone()
    s0, s1 = me.shape[0], me.shape[1]
    h0, h1 = h

    def rng_send(d, hh, s):
        return slice(0, s) if d == 0 else (slice(s - 2 * hh, s - hh) if d > 0 else slice(hh, 2 * hh))

    def rng_recv(d, hh, s):
        return slice(0, s) if d == 0 else (slice(0, hh) if d > 0 else slice(s - hh, s))

    dirs = []
    if h0 and p0 > 1:
        dirs += [(1, 0), (-1, 0)]
    if h1 and p1 > 1:
        dirs += [(0, 1), (0, -1)]
    if h0 and h1 and p0 > 1 and p1 > 1:
        dirs += [(1, 1), (1, -1), (-1, 1), (-1, -1)]
    for d0, d1 in dirs:
        c0, c1 = coords[0] - d0, coords[1] - d1
        ok = True
        if not (0 <= c0 < p0):
            ok = ok and periods[0]
            c0 %= p0
        if not (0 <= c1 < p1):
            ok = ok and periods[1]
            c1 %= p1
        reg = (rng_recv(d0, h0, s0), rng_recv(d1, h1, s1))
        if ok:
            out[reg] = xg_blocks[(c0, c1)][rng_send(d0, h0, s0), rng_send(d1, h1, s1)]
        else:
            out[reg] = 0
    return out


def _halo_worker(rank, world, pdims, periods):
    mesh = jd.make_mesh(pdims, ("z", "y"))
    h = (2, 3)
    p0, p1 = pdims
    blocks = {}
    g = torch.Generator().manual_seed(11)
    for i in range(p0):
        for j in range(p1):
            blocks[(i, j)] = torch.randn((4 + 2 * h[0], 6 + 2 * h[1], 5), generator=g, dtype=torch.float32)
    mine = blocks[tuple(mesh.coords)]
    st = jd.ShardedTensor(mine.clone(), mesh)
    out = jd.halo_exchange(st, h, periods)
    want = _expected_halo(blocks, pdims, tuple(mesh.coords), h, periods)
    assert torch.equal(out.local, want)
    assert torch.equal(jd.halo_exchange_(jd.ShardedTensor(mine.clone(), mesh), h, periods).local, want)
    # exact adjoint: <L x, y> == <x, L^T y> summed over ranks
    y = torch.randn(mine.shape, generator=torch.Generator().manual_seed(100 + rank))
    lty = jd.halo_accumulate(jd.ShardedTensor(y, mesh), h, periods)
    a = (out.local * y).sum()
    b = (mine * lty.local).sum()
    tot = torch.stack([a, b]).double()
    torch.distributed.all_reduce(tot)
    assert abs(tot[0] - tot[1]) < 1e-3 * max(1.0, abs(tot[0])), tot
    # autograd uses that adjoint
    xl = mine.clone().requires_grad_(True)
    o = jd.halo_exchange(jd.ShardedTensor(xl, mesh), h, periods)
    (o.local * y).sum().backward()
    torch.testing.assert_close(xl.grad, lty.local)


@pytest.mark.parametrize("pdims,periods", [((2, 4), (True, True)), ((4, 2), (False, True)), ((2, 4), (False, False)),
                                           ((1, 8), (True, True)), ((8, 1), (True, False))])
def test_halo_exchange(pdims, periods):
    run_ranks(_halo_worker, 8, pdims, periods)


def _grad_worker(rank, world, pdims):
    mesh = jd.make_mesh(pdims, ("z", "y"))
    xg = _global((8, 16, 8), torch.complex128, seed=5)
    x = jd.shard(xg, mesh)
    x.local.requires_grad_(True)
    k = jd.pfft3d(x, norm="ortho")
    loss = (k.local.abs() ** 2 * (1 + rank)).sum()  # rank-dependent weights make the test sensitive to routing
    loss.backward()
    # reference: same loss on the gathered transform
    xr = xg.clone().requires_grad_(True)
    kr = torch.fft.fftn(xr, norm="ortho").permute(1, 2, 0)
    w = torch.zeros(kr.shape, dtype=torch.float64)
    for r in range(world):
        offs = jd.parallel.sharding.shard_offsets(k.global_shape, k.spec, mesh, rank=r)
        idx = tuple(slice(o, o + n) for o, n in zip(offs, k.local.shape))
        w[idx] = 1 + r
    ((kr.abs() ** 2) * w).sum().backward()
    want = jd.shard(xr.grad, mesh).local
    torch.testing.assert_close(x.local.grad, want, rtol=1e-9, atol=1e-9)
    # inverse transform
    k2 = jd.ShardedTensor(k.local.detach().clone().requires_grad_(True), mesh, k.spec)
    xb = jd.pifft3d(k2, norm="ortho")
    (xb.local.real ** 2).sum().backward()
    kr2 = kr.detach().clone().requires_grad_(True)
    xbr = torch.fft.ifftn(kr2.permute(2, 0, 1), norm="ortho")
    (xbr.real ** 2).sum().backward()
    want2 = jd.ShardedTensor(jd.shard(kr2.grad, mesh, k.spec).local, mesh, k.spec).local
    torch.testing.assert_close(k2.local.grad, want2, rtol=1e-9, atol=1e-9)


@pytest.mark.parametrize("pdims", [(2, 4), (1, 8), (8, 1)])
def test_fft_gradients(pdims):
    run_ranks(_grad_worker, 8, pdims)


def _batch_worker(rank, world):
    # nested parallelism: leading mesh axis = independent groups, plus a local batch dimension
    mesh = jd.Mesh((2, 2, 2), ("c", "z", "y"))
    grp = mesh.coords[0]
    xg = _global((3, 8, 8, 16), torch.complex64, seed=20 + grp)
    x_local = jd.shard(xg, mesh, (None, "z", "y", None))
    k = jd.pfft3d(x_local)
    assert k.local.shape == (3, 4, 8, 8)
    ref = torch.fft.fftn(xg, dim=(1, 2, 3)).permute(0, 2, 3, 1)
    offs = jd.parallel.sharding.shard_offsets(k.global_shape, k.spec, mesh)
    idx = tuple(slice(o, o + n) for o, n in zip(offs, k.local.shape))
    torch.testing.assert_close(k.local, ref[idx], rtol=1e-4, atol=1e-4)
    back = jd.pifft3d(k)
    torch.testing.assert_close(back.local, x_local.local, rtol=1e-4, atol=1e-4)


def test_batched_and_nested_mesh():
    run_ranks(_batch_worker, 8)


def _config1_worker(rank, world):
    """64^3 float32 N(0,1) from seed 0 cast to complex64, pdims (2,4)."""
    mesh = jd.make_mesh((2, 4), ("z", "y"))
    xg = torch.randn((64, 64, 64), generator=torch.Generator().manual_seed(0)).to(torch.complex64)
    x = jd.shard(xg, mesh)
    k = jd.pfft3d(x)
    torch.testing.assert_close(k.gather(), torch.fft.fftn(xg).permute(1, 2, 0), rtol=1e-4, atol=5e-3)
    torch.testing.assert_close(jd.pifft3d(k).gather(), xg, rtol=1e-4, atol=1e-4)
    y = jd.transposeXtoY(x)
    z = jd.transposeYtoZ(y)
    assert torch.equal(jd.transposeYtoX(jd.transposeZtoY(z)).gather(), xg)


def test_headline_config_on_cpu_ranks():
    run_ranks(_config1_worker, 8)


def test_fft_reference_shape_grid_with_large_prime_factors():
    """The reference's non-power-of-two test shape (29 N, 19 N, 17 N), here with N = 4."""
    for pdims in ((2, 4), (4, 2)):
        run_ranks(_fft_worker, 8, pdims, (29 * 4, 19 * 4, 17 * 4), True, torch.complex128)


def _spectral_worker(rank, world, pdims):
    mesh = jd.make_mesh(pdims, ("z", "y"))
    shape = (16, 8, 32)
    xg = _global(shape, torch.complex128, seed=3)
    x = jd.shard(xg, mesh)
    k = jd.pfft3d(x)
    k0, k1, k2 = jd.fftfreq3d(k)            # wave numbers of the original axes 0, 1, 2, broadcastable to k.local
    full = [2 * torch.pi * torch.fft.fftfreq(n, dtype=torch.float64) for n in shape]
    for axis, kv in enumerate((k0, k1, k2)):
        dk = jd.ShardedTensor(k.local * (1j * kv), mesh, k.spec)
        got = jd.pifft3d(dk).gather()
        view = [1, 1, 1]
        view[axis] = -1
        want = torch.fft.ifftn(torch.fft.fftn(xg) * (1j * full[axis].reshape(view)))
        torch.testing.assert_close(got, want, rtol=1e-10, atol=1e-10)


@pytest.mark.parametrize("pdims", [(2, 4), (1, 8)])
def test_spectral_derivative_with_fftfreq3d(pdims):
    run_ranks(_spectral_worker, 8, pdims)


def _jvp_worker(rank, world):
    import torch.autograd.forward_ad as fwAD

    mesh = jd.make_mesh((2, 4), ("z", "y"))
    xg, tg = _global((16, 8, 32), torch.complex128, seed=5), _global((16, 8, 32), torch.complex128, seed=6)
    x, t = jd.shard(xg, mesh), jd.shard(tg, mesh)
    with fwAD.dual_level():
        dual = jd.ShardedTensor(fwAD.make_dual(x.local, t.local), mesh, x.spec)
        y = jd.pfft3d(dual)
        primal, tangent = fwAD.unpack_dual(y.local)
        assert tangent is not None
        got = jd.ShardedTensor(tangent, mesh, y.spec).gather()
        torch.testing.assert_close(got, torch.fft.fftn(tg).permute(1, 2, 0), rtol=1e-10, atol=1e-10)
        z = jd.transposeXtoY(dual)
        _, tz = fwAD.unpack_dual(z.local)
        torch.testing.assert_close(tz, jd.transposeXtoY(t).local)


def test_forward_mode_derivatives():
    run_ranks(_jvp_worker, 8)
