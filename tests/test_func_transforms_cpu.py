"""``torch.func`` transforms through the distributed ops on CPU ranks: ``vmap`` over a stack of local
blocks, ``vmap`` with the batch sharded over a leading mesh axis (independent groups), ``jacfwd`` and
``jacrev``.  Counterparts of the reference's vmap / sharded-vmap / Jacobian tests
(``tests/test_fft.py:389-469, 507-560``, ``tests/test_transpose.py:281-321``,
``tests/test_halo.py:403-459``)."""
import torch
from torch.func import jacfwd, jacrev, vmap

import jaxdecomp_b200 as jd
from jaxdecomp_b200.utils.testing import run_ranks


def _global(shape, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g, dtype=torch.float64)
    if dtype.is_complex:
        x = torch.complex(x, torch.randn(shape, generator=g, dtype=torch.float64))
    return x.to(dtype)


def _vmap_worker(rank, world, pdims):
    mesh = jd.make_mesh(pdims, ("z", "y"))
    nb = 3
    xs = [_global((16, 16, 16), torch.complex128, seed=30 + i) for i in range(nb)]
    locals_ = torch.stack([jd.shard(x, mesh).local for x in xs])          # [batch, local block]
    with mesh:
        ks = vmap(lambda v: jd.pfft3d(v))(locals_)
        backs = vmap(lambda v: jd.pifft3d(v))(ks)
        ys = vmap(lambda v: jd.transposeXtoY(v))(locals_)
        hs = vmap(lambda v: jd.halo_exchange(v, (1, 1), (True, True)))(locals_.real.contiguous())
    for i, x in enumerate(xs):
        st = jd.shard(x, mesh)
        k1 = jd.pfft3d(st)
        assert torch.equal(ks[i], k1.local)
        torch.testing.assert_close(jd.ShardedTensor(ks[i], mesh, k1.spec).gather(), torch.fft.fftn(x).permute(1, 2, 0),
                                   rtol=1e-10, atol=1e-10)
        torch.testing.assert_close(backs[i], st.local, rtol=1e-10, atol=1e-10)
        assert torch.equal(ys[i], jd.transposeXtoY(st).local)
        assert torch.equal(hs[i], jd.halo_exchange(jd.ShardedTensor(st.local.real.contiguous(), mesh), (1, 1),
                                                   (True, True)).local)
    # mapping over a dimension that is not the first one
    with mesh:
        k_last = vmap(lambda v: jd.pfft3d(v), in_dims=3, out_dims=3)(locals_.permute(1, 2, 3, 0))
    assert torch.equal(k_last.permute(3, 0, 1, 2), ks)


def test_vmap_over_stacked_blocks_pencils_and_slabs():
    for pdims in ((2, 4), (1, 8), (8, 1)):
        run_ranks(_vmap_worker, 8, pdims)


def _sharded_vmap_worker(rank, world):
    # 3-D mesh: the leading axis 'c' splits the batch into independent groups of 2x2 ranks
    mesh = jd.Mesh((2, 2, 2), ("c", "z", "y"))
    grp = mesh.coords[0]
    nb = 4
    xg = _global((nb, 8, 8, 16), torch.complex128, seed=40)               # the whole batch, known to every rank
    mine = xg[grp * 2:(grp + 1) * 2]                                      # this group's half of the batch
    x = jd.shard(mine, mesh, (None, "z", "y", None))
    with mesh:
        k = vmap(lambda v: jd.pfft3d(v))(x.local)
        y = vmap(lambda v: jd.transposeXtoY(v))(x.local)
        h = vmap(lambda v: jd.halo_exchange(v, (1, 1), (True, True)))(x.local)
    kb = jd.pfft3d(x)                                                     # the explicit batch dimension, same result
    assert torch.equal(k, kb.local) and tuple(kb.spec) == (None, "z", "y", None)
    ref = torch.fft.fftn(mine, dim=(1, 2, 3)).permute(0, 2, 3, 1)
    offs = jd.parallel.sharding.shard_offsets(kb.global_shape, kb.spec, mesh)
    idx = tuple(slice(o, o + n) for o, n in zip(offs, kb.local.shape))
    torch.testing.assert_close(k, ref[idx], rtol=1e-10, atol=1e-10)
    assert torch.equal(y, jd.transposeXtoY(x).local)
    assert torch.equal(h, jd.halo_exchange(x, (1, 1), (True, True)).local)
    # round trip through the batched transposes on the nested mesh
    z = jd.transposeYtoZ(jd.transposeXtoY(x))
    assert torch.equal(jd.transposeYtoX(jd.transposeZtoY(z)).local, x.local)


def test_sharded_vmap_on_nested_mesh():
    run_ranks(_sharded_vmap_worker, 8)


def _jacobian_worker(rank, world):
    mesh = jd.make_mesh((2, 2), ("z", "y"))
    xg = _global((4, 4, 4), torch.float64, seed=50)
    x = jd.shard(xg, mesh).local                                          # 2 x 2 x 4 local block

    def roundtrip(v):
        with mesh:
            return jd.pifft3d(jd.pfft3d(v)).real

    jf, jr = jacfwd(roundtrip)(x), jacrev(roundtrip)(x)
    eye = torch.eye(x.numel(), dtype=torch.float64).reshape(x.shape + x.shape)
    torch.testing.assert_close(jf, eye, rtol=1e-12, atol=1e-12)
    torch.testing.assert_close(jr, eye, rtol=1e-12, atol=1e-12)

    # Under SPMD every rank differentiates with respect to its own block at the same time: forward mode
    # perturbs element i of every rank's block together, so column i of the local Jacobian of the
    # forward transform is the local part of the transform of that joint perturbation.
    def forward(v):
        with mesh:
            return torch.view_as_real(jd.pfft3d(v))                       # jacfwd wants real inputs and outputs

    jfwd = jacfwd(forward)(x)                                             # real input, complex output
    for i in (0, 5, 15):
        e = torch.zeros(x.numel(), dtype=torch.float64)
        e[i] = 1.0
        joint = jd.ShardedTensor(e.reshape(x.shape), mesh).gather()       # the same basis vector on every rank
        want = torch.view_as_real(jd.pfft3d(jd.shard(joint, mesh)).local)
        torch.testing.assert_close(jfwd.reshape(want.shape + (-1,))[..., i], want, rtol=1e-12, atol=1e-12)

    def through_transpose(v):
        with mesh:
            return jd.transposeYtoX(jd.transposeXtoY(v))

    jt = jacrev(through_transpose)(x)
    torch.testing.assert_close(jt, eye, rtol=0, atol=0)


def test_jacfwd_and_jacrev_through_the_ops():
    run_ranks(_jacobian_worker, 4)


def _unsharded_worker(rank, world):
    import pytest

    from jaxdecomp_b200.utils.errors import ShardingError

    x = torch.randn(4, 4, 4)
    with pytest.raises(ShardingError, match="no mesh is active"):
        jd.pfft3d(x)                                                      # several ranks, no mesh, no sharding: refuse
    with pytest.raises(ShardingError):
        jd.halo_exchange(x, (1, 1), (True, True))
    with jd.single_rank_mesh():                                           # the explicit way to transform a replica
        torch.testing.assert_close(jd.pfft3d(x), torch.fft.fftn(x.to(torch.complex64)).permute(1, 2, 0))


def test_plain_tensor_without_mesh_in_a_multi_rank_job_raises():
    run_ranks(_unsharded_worker, 2)


def _compat_grad_worker(rank, world):
    # the reference differentiates halo_exchange by exchanging the halos of the cotangent
    # (src/jaxdecomp/_src/jax/halo.py:401-420); reference_compat_halo_grad reproduces that rule,
    # the default is the exact adjoint (halo cotangents are added into the interior they came from)
    mesh = jd.make_mesh((2, 2), ("z", "y"))
    blk = torch.randn((6, 6, 3), generator=torch.Generator().manual_seed(60 + rank), dtype=torch.float64)
    w = torch.randn((6, 6, 3), generator=torch.Generator().manual_seed(70 + rank), dtype=torch.float64)
    grads = {}
    for compat in (False, True):
        jd.config.update("reference_compat_halo_grad", compat)
        x = blk.clone().requires_grad_(True)
        y = jd.halo_exchange(jd.ShardedTensor(x, mesh), (1, 1), (True, True))
        (y.local * w).sum().backward()
        grads[compat] = x.grad.clone()
    jd.config.update("reference_compat_halo_grad", False)
    want_compat = jd.halo_exchange(jd.ShardedTensor(w, mesh), (1, 1), (True, True)).local
    want_exact = jd.halo_accumulate(jd.ShardedTensor(w, mesh), (1, 1), (True, True)).local
    torch.testing.assert_close(grads[True], want_compat, rtol=0, atol=0)
    torch.testing.assert_close(grads[False], want_exact, rtol=0, atol=0)
    assert not torch.equal(grads[True], grads[False])
    # only the exact adjoint satisfies <L x, w> == <x, L^T w> summed over the ranks
    lhs = (jd.halo_exchange(jd.ShardedTensor(blk, mesh), (1, 1), (True, True)).local * w).sum()
    rhs = (blk * want_exact).sum()
    both = torch.stack([lhs, rhs])
    torch.distributed.all_reduce(both)
    torch.testing.assert_close(both[0], both[1], rtol=1e-12, atol=1e-12)


def test_reference_compatible_halo_gradient_rule():
    run_ranks(_compat_grad_worker, 4)


def test_gradcheck_and_double_backward_on_a_single_rank():
    """Numerical first and second derivatives of every differentiable op (float64, one rank)."""
    x = torch.randn((3, 4, 5), dtype=torch.float64, generator=torch.Generator().manual_seed(80), requires_grad=True)
    z = torch.randn((3, 4, 5), dtype=torch.complex128, generator=torch.Generator().manual_seed(81), requires_grad=True)
    for norm in ("backward", "ortho"):
        assert torch.autograd.gradcheck(lambda v: torch.view_as_real(jd.pfft3d(v, norm=norm)), (x,))
        assert torch.autograd.gradcheck(lambda v: jd.pifft3d(jd.pfft3d(v, norm=norm), norm=norm), (z,))
    assert torch.autograd.gradgradcheck(lambda v: torch.view_as_real(jd.pfft3d(v)).pow(2), (x,))
    for fn in (jd.transposeXtoY, jd.transposeYtoZ, jd.transposeZtoY, jd.transposeYtoX, jd.transposeXtoZ, jd.transposeZtoX):
        assert torch.autograd.gradcheck(fn, (x,))
        assert torch.autograd.gradgradcheck(lambda v: fn(v).pow(3), (x,))
    with jd.single_rank_mesh():
        assert torch.autograd.gradcheck(lambda v: jd.halo_exchange(v, (1, 1), (True, True)), (x,))
        assert torch.autograd.gradcheck(lambda v: jd.halo_accumulate(v, (1, 1), (True, True)), (x,))


def _halo_fit_worker(rank, world, pdims):
    # the reference's halo gradient test (tests/test_halo.py:313-398): a least-squares loss through
    # pad + halo_exchange has zero gradient at the observation; away from it the gradient is
    # 2 L^T (L x - obs), which is checked against a directional finite difference over all ranks
    mesh = jd.make_mesh(pdims, ("z", "y"))
    h = (2 if pdims[0] > 1 else 0, 2 if pdims[1] > 1 else 0)
    x0 = torch.randn((16 // pdims[0], 16 // pdims[1], 4), dtype=torch.float64, generator=torch.Generator().manual_seed(90 + rank))

    def forward(v):
        return jd.halo_exchange(jd.pad_halo(jd.ShardedTensor(v, mesh), h), h, (True, True)).local

    obs = forward(x0).detach()

    def loss(v):
        return ((forward(v) - obs) ** 2).sum()      # this rank's part; the global loss is the sum over ranks

    def global_loss(v):
        t = loss(v).detach().clone()
        torch.distributed.all_reduce(t)
        return float(t)

    x = x0.clone().requires_grad_(True)
    loss(x).backward()
    assert torch.equal(x.grad, torch.zeros_like(x0))
    x = (2 * x0).clone().requires_grad_(True)
    loss(x).backward()
    g = x.grad.clone()
    direction = torch.randn(x0.shape, dtype=torch.float64, generator=torch.Generator().manual_seed(190 + rank))
    eps = 1e-6
    fd = (global_loss(2 * x0 + eps * direction) - global_loss(2 * x0 - eps * direction)) / (2 * eps)
    an = (g * direction).sum()
    torch.distributed.all_reduce(an)
    assert abs(float(an) - fd) <= 1e-6 * max(1.0, abs(fd)), (float(an), fd)
    # every interior cell also appears in some neighbour's halo: the gradient is larger than the local term alone
    assert (g.abs() >= (2 * x0).abs() - 1e-12).all()


def test_least_squares_gradient_through_pad_and_halo_exchange():
    for pdims in ((2, 4), (1, 8), (4, 2)):
        run_ranks(_halo_fit_worker, 8, pdims)
