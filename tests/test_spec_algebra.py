"""Unit tests of the mesh / spec / geometry arithmetic (no ranks needed)."""
import pytest
import torch

import jaxdecomp_b200 as jd
from jaxdecomp_b200.ops import passes, plan
from jaxdecomp_b200.ops.fft import _fft_norm
from jaxdecomp_b200.parallel.mesh import Mesh, pencil_type_from_pdims
from jaxdecomp_b200.parallel.sharding import local_shape, pencil_info, shard_offsets


def _mesh(shape, names, rank=0):
    n = 1
    for s in shape:
        n *= s
    return Mesh(shape, names, rank=rank, world_size=n, create_groups=False)


def test_pencil_types():
    assert pencil_type_from_pdims((1, 1)) == jd.NO_DECOMP
    assert pencil_type_from_pdims((1, 4)) == jd.SLAB_YZ
    assert pencil_type_from_pdims((4, 1)) == jd.SLAB_XY
    assert pencil_type_from_pdims((2, 2)) == jd.PENCILS
    assert int(jd.SLAB_XY) == 0 and int(jd.SLAB_YZ) == 1 and int(jd.PENCILS) == 2 and int(jd.NO_DECOMP) == 3
    assert int(jd.HALO_COMM_NCCL) == 3 and int(jd.TRANSPOSE_COMM_NCCL) == 4 and int(jd.TRANSPOSE_COMM_MPI_P2P) == 1


def test_mesh_coordinates_and_neighbours():
    m = _mesh((2, 4), ("z", "y"), rank=5)
    assert m.coords == (1, 1) and m.pdims == (2, 4)
    assert m.axis_ranks(0) == [1, 5] and m.axis_ranks(1) == [4, 5, 6, 7]
    assert m.neighbor(1, 0) == 1 and m.neighbor(0, -1) == 4 and m.neighbor(1, 1) == 2
    assert m.neighbor(1, 0, (False, True)) is None
    b = _mesh((2, 2, 2), ("c", "z", "y"), rank=6)
    assert b.coords == (1, 1, 0) and b.pdims == (2, 2) and b.submesh_ranks() == [4, 5, 6, 7]
    assert b.batch_axis_names == ("c",)


def test_validate_spec_matches_mesh():
    m = _mesh((2, 4), ("z", "y"))
    jd.validate_spec_matches_mesh(("z", "y"), m)
    jd.validate_spec_matches_mesh(jd.P("z", "y", None), m)
    with pytest.raises(ValueError, match="position 0"):
        jd.validate_spec_matches_mesh(("y", "z"), m)
    with pytest.raises(ValueError, match="has size 4"):
        jd.validate_spec_matches_mesh(("z", None), m)
    s = _mesh((1, 8), ("z", "y"))
    jd.validate_spec_matches_mesh((None, "y"), s)
    jd.validate_spec_matches_mesh(("z", "y"), s)


@pytest.mark.parametrize("contig", [True, False])
@pytest.mark.parametrize("pdims", [(2, 4), (1, 8), (8, 1)])
def test_output_spec_table_matches_step_propagation(pdims, contig):
    jd.config.update("transpose_axis_contiguous", contig)
    names = ("z", "y")
    pt = pencil_type_from_pdims(pdims)
    spec = (names[0] if pdims[0] > 1 else None, names[1] if pdims[1] > 1 else None, None)
    lshape = (64 // pdims[0], 64 // pdims[1], 64)
    steps = plan.fft_steps(pt, False, contig)
    oshape, ospec = plan.propagate(steps, lshape, spec, pdims, names)
    assert tuple(jd.get_output_specs("fft", pt, spec)) == ospec
    isteps = plan.fft_steps(pt, True, contig)
    plan.check_input_spec(isteps, ospec, pdims, names)
    bshape, bspec = plan.propagate(isteps, oshape, ospec, pdims, names)
    assert bshape == lshape and bspec == spec
    assert tuple(jd.get_output_specs("ifft", pt, ospec)) == spec
    # the kernel-friendly list ends in the same layout
    assert plan.propagate(plan.fft_steps(pt, False, contig, native=True), lshape, spec, pdims, names) == (oshape, ospec)


def test_wrong_layout_is_reported():
    names = ("z", "y")
    with pytest.raises(ValueError, match="should be sharded"):
        plan.check_input_spec(plan.transpose_steps("y_z", True), ("z", "y", None), (2, 4), names)


def test_fft_norm():
    assert _fft_norm((4, 4, 4), False, "backward") == 1.0
    assert _fft_norm((4, 4, 4), True, "backward") == 1 / 64
    assert _fft_norm((4, 4, 4), False, "ortho") == pytest.approx(1 / 8)
    assert _fft_norm((4, 4, 4), False, "forward") == 1 / 64 and _fft_norm((4, 4, 4), True, "forward") == 1.0
    with pytest.raises(ValueError):
        _fft_norm((4, 4, 4), False, "bogus")


def test_fftfreq3d_shapes_and_values():
    k = torch.zeros((6, 8, 4), dtype=torch.complex64)
    kz, ky, kx = jd.fftfreq3d(k)
    assert kz.shape == (1, 1, 4) and ky.shape == (6, 1, 1) and kx.shape == (1, 8, 1)
    assert kz.dtype == torch.float32
    torch.testing.assert_close(ky.flatten(), torch.fft.fftfreq(6) * 2 * torch.pi)
    assert jd.fftfreq3d(k.to(torch.complex128))[0].dtype == torch.float64
    with pytest.raises(AssertionError):
        jd.fftfreq3d(torch.zeros(2, 2, 2))
    m = _mesh((2, 4), ("z", "y"), rank=5)
    st = jd.ShardedTensor(torch.zeros((3, 2, 4), dtype=torch.complex64), m)
    a, b, c = jd.fftfreq3d(st)
    assert b.shape == (3, 1, 1) and c.shape == (1, 2, 1)
    torch.testing.assert_close(b.flatten(), (torch.fft.fftfreq(6) * 2 * torch.pi)[3:6])
    assert jd.rfftfreq3d(k)[2].shape == (1, 5, 1)


def test_pencil_info_and_offsets():
    info = pencil_info((8, 16, 32), (2, 4), 0, (1, 2))
    assert info.shape == (4, 4, 32) and info.lo == (4, 8, 0) and info.hi == (7, 11, 31) and info.order == (0, 1, 2)
    y = pencil_info((8, 16, 32), (2, 4), 1, (1, 2), contiguous=True)
    assert y.shape == (8, 4, 16) and y.order == (2, 0, 1) and y.lo == (16, 4, 0)
    z = pencil_info((8, 16, 32), (2, 4), 2, (1, 2), contiguous=True)
    assert z.shape == (8, 8, 8) and z.order == (1, 2, 0) and z.size == 512
    h = pencil_info((8, 16, 32), (2, 4), 0, (0, 0), halo_extents=(2, 1, 0))
    assert h.shape == (8, 6, 32) and h.halo_extents == (2, 1, 0)
    cfg = jd.make_config((8, 16, 32), (2, 4))
    assert jd.get_pencil_info(cfg, 0, coords=(1, 2)) == info
    m = _mesh((2, 4), ("z", "y"), rank=6)
    assert local_shape((8, 16, 32), ("z", "y", None), m) == (4, 4, 32)
    assert shard_offsets((8, 16, 32), ("z", "y", None), m) == (4, 8, 0)
    with pytest.raises(jd.utils.errors.ShardingError):
        local_shape((9, 16, 32), ("z", "y", None), m)


def test_config_update_validates_keys():
    jd.config.update("transpose_axis_contiguous", False)
    assert jd.config.transpose_axis_contiguous is False
    with pytest.raises(ValueError):
        jd.config.update("no_such_key", 1)
    jd.config.update("backend", "JAX")
    assert jd.config.backend == "torch"
    with pytest.raises(ValueError):
        jd.pfft3d(torch.zeros(2, 2, 2), backend="bogus")


def test_pipeline_block_limit_setting():
    from jaxdecomp_b200.ops.b200_backend import auto_pipeline_ctas

    old = jd.config.pipeline_ctas
    try:
        jd.config.update("pipeline_ctas", -1)        # automatic: chosen per exchange from its number of peers
        jd.config.update("pipeline_ctas", 0)         # no limit
        jd.config.update("pipeline_ctas", "64")
        assert jd.config.pipeline_ctas == 64
        with pytest.raises(ValueError):
            jd.config.update("pipeline_ctas", -2)
        with pytest.raises(ValueError):
            jd.config.update("pipeline_chunks", -1)
    finally:
        jd.config.update("pipeline_ctas", old)
    assert 0 < auto_pipeline_ctas(2) <= auto_pipeline_ctas(8) <= 148


def test_pass_compiler_geometry():
    steps = plan.fft_steps(jd.PENCILS, False, True, native=True)
    specs, final = passes.compile_passes(steps, (4, 4, 32), (2, 4), (1, 2))
    assert final == (8, 8, 8) and len(specs) == 3
    p0 = specs[0]
    assert p0.fft and p0.npeers == 4 and p0.mesh_axis == 1 and p0.axes == (2, 1, 0)
    assert p0.chunks == (8, 4, 4) and p0.out_strides[1] == 1 and p0.out_base == 2 * 4
    assert specs[2].plain and not specs[1].plain
    t = passes.choose_tiling(p0, 8, True)
    assert t["fft_mode"] == 1 and t["store_t_contig"] == 1 and t["load_t_contig"] == 0 and t["pitch"] % 2 == 0
    odd, _ = passes.compile_passes([plan.Fft(2)], (2, 3, 29), (1, 1), (0, 0))
    t = passes.choose_tiling(odd[0], 8, False)
    assert t["fft_mode"] == 2 and t["M"] == 64 and t["vec_in"] == 0


def test_module_paths_of_the_reference():
    """``jaxdecomp.fft.pfft3d``, ``jaxdecomp.halo.halo_exchange`` and ``jaxdecomp.transpose.transposeXtoY`` have
    the same paths here; the real-input transforms exist and refuse, as in the reference
    (``src/jaxdecomp/fft.py:127-128, 214-284``)."""
    x = torch.randn(4, 6, 8)
    assert torch.equal(jd.fft.pfft3d(x), jd.pfft3d(x)) and jd.fft.pifft3d is jd.pifft3d
    assert jd.halo.halo_exchange is jd.halo_exchange and jd.transpose.transposeXtoY is jd.transposeXtoY
    assert jd.fft.fftfreq3d is jd.fftfreq3d and jd.fft.rfftfreq3d is jd.rfftfreq3d
    for fn in (jd.fft.prfft3d, jd.fft.pirfft3d, jd.prfft3d):
        with pytest.raises(NotImplementedError):
            fn(x)


def test_single_rank_plain_tensor_api():
    x = torch.randn(8, 4, 16)
    k = jd.pfft3d(x)
    torch.testing.assert_close(k, torch.fft.fftn(x.to(torch.complex64)).permute(1, 2, 0), rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(jd.pifft3d(k).real, x, rtol=1e-4, atol=1e-5)
    assert torch.equal(jd.transposeXtoY(x), x.permute(2, 0, 1))
    padded = jd.pad_halo(x, (1, 2))
    assert padded.shape == (10, 8, 16) and torch.equal(jd.unpad_halo(padded, (1, 2)), x)
    assert torch.equal(jd.halo_exchange(padded, (1, 2), (True, True)), padded)
    with pytest.raises(NotImplementedError):
        from jaxdecomp_b200.ops.fft import prfft3d

        prfft3d(x)


def test_workspace_queries_and_bounds_check():
    cfg = jd.make_config((1024, 1024, 1024), (2, 4))
    assert jd.get_fft_workspace_size(cfg) == 2 * (1 << 30)
    assert jd.get_fft_workspace_size(jd.make_config((64, 64, 64), (1, 1)), True) == 64 ** 3 * 16
    assert jd.get_transpose_workspace_size(cfg, 4) == (1 << 30) // 2
    assert jd.get_halo_workspace_size(cfg, (16, 16)) == (2 * 16 * 288 + 2 * 16 * 544 - 4 * 256) * 1024 * 4
    steps = plan.fft_steps(jd.PENCILS, False, True, native=True)
    specs, _ = passes.compile_passes(steps, (4, 4, 32), (2, 4), (1, 3))
    for sp in specs:
        passes.check_pass_bounds(sp)
    bad = specs[0]
    bad.out_base += bad.numel
    with pytest.raises(AssertionError):
        passes.check_pass_bounds(bad)
