"""Native sm_100a kernels on one GPU against plain PyTorch references."""
import os

import pytest
import torch

import jaxdecomp_b200 as jd

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _rel(a, b):
    return ((a - b).abs().max() / b.abs().max()).item()


@pytest.mark.parametrize("shape", [(64, 32, 128), (8, 16, 8), (256, 8, 1024), (16, 16, 2048), (24, 40, 58), (29, 19, 17),
                                   (4, 2, 4096), (128, 128, 128), (256, 64, 512), (32, 4096, 64), (2048, 32, 256),
                                   # mixed-radix lengths: every radix, ragged tiles, one and two blocks per SM
                                   (96, 60, 768), (100, 30, 1000), (12, 6, 2310), (77, 143, 26), (4, 2, 6),
                                   (1536, 8, 384), (7, 11, 13), (33, 21, 45), (20, 1365, 3072)])
@pytest.mark.parametrize("dtype", [torch.complex64, torch.complex128])
def test_fft_single_gpu(shape, dtype):
    x = torch.randn(shape, device=_dev(), dtype=dtype)
    k = jd.pfft3d(x, backend="b200")
    ref = torch.fft.fftn(x).permute(1, 2, 0)
    tol = 3e-6 if dtype == torch.complex64 else 1e-13
    assert k.shape == ref.shape
    assert _rel(k, ref) < tol
    back = jd.pifft3d(k, backend="b200")
    assert _rel(back, x) < 10 * tol
    for norm in ("ortho", "forward"):
        torch.testing.assert_close(jd.pfft3d(x, norm=norm, backend="b200"),
                                   torch.fft.fftn(x, norm=norm).permute(1, 2, 0),
                                   rtol=1e-4 if dtype == torch.complex64 else 1e-10,
                                   atol=1e-4 if dtype == torch.complex64 else 1e-10)


_STATIC_LENGTHS = [96, 192, 384, 768, 1536, 3072, 288, 576, 1152, 2304, 160, 320, 640, 1280, 2560, 200, 400, 800, 1600,
                   250, 500, 1000, 2000, 240, 480, 960, 1920, 448, 896, 1792]


@pytest.mark.parametrize("dtype", [torch.complex64, torch.complex128])
def test_mixed_radix_specialised_lengths(dtype, monkeypatch):
    """Every length with a specialised mixed-radix kernel, as the rotating first pass and as the plain last pass,
    against torch.fft and against the generic mixed-radix kernel."""
    tol = 3e-6 if dtype == torch.complex64 else 1e-13
    for n in _STATIC_LENGTHS:
        for shape in ((16, 32, n), (n, 16, 32)):
            x = torch.randn(shape, device=_dev(), dtype=dtype)
            k = jd.pfft3d(x, backend="b200")
            ref = torch.fft.fftn(x).permute(1, 2, 0)
            assert _rel(k, ref) < tol, (n, shape)
            assert _rel(jd.pifft3d(k, backend="b200"), x) < 10 * tol, (n, shape)
    monkeypatch.setenv("JD_B200_MIXED_STATIC", "0")
    x = torch.randn((16, 32, 768), device=_dev(), dtype=dtype)
    assert _rel(jd.pfft3d(x, backend="b200"), torch.fft.fftn(x).permute(1, 2, 0)) < tol


@pytest.mark.parametrize("bulk,tile", [("0", ""), ("1", "4"), ("1", "16"), ("0", "2")])
def test_fft_load_paths_and_tiles(bulk, tile, monkeypatch):
    monkeypatch.setenv("JD_B200_BULK", bulk)
    monkeypatch.setenv("JD_B200_TILE_T", tile)
    x = torch.randn((40, 24, 512), device=_dev(), dtype=torch.complex64)
    k = jd.pfft3d(x, backend="b200")
    assert _rel(k, torch.fft.fftn(x).permute(1, 2, 0)) < 3e-6
    assert _rel(jd.pifft3d(k, backend="b200"), x) < 3e-5


def test_fft_non_contiguous_mode_and_batch():
    jd.config.update("transpose_axis_contiguous", False)
    x = torch.randn((3, 16, 24, 64), device=_dev(), dtype=torch.complex64)
    k = jd.pfft3d(x, backend="b200")
    assert _rel(k, torch.fft.fftn(x, dim=(1, 2, 3))) < 3e-6
    assert _rel(jd.pifft3d(k, backend="b200"), x) < 3e-5
    jd.config.update("transpose_axis_contiguous", True)
    k = jd.pfft3d(x, backend="b200")
    assert _rel(k, torch.fft.fftn(x, dim=(1, 2, 3)).permute(0, 2, 3, 1)) < 3e-6
    # strided mixed-radix transforms
    jd.config.update("transpose_axis_contiguous", False)
    try:
        y = torch.randn((2, 48, 36, 60), device=_dev(), dtype=torch.complex128)
        k = jd.pfft3d(y, backend="b200")
        assert _rel(k, torch.fft.fftn(y, dim=(1, 2, 3))) < 1e-13
        assert _rel(jd.pifft3d(k, backend="b200"), y) < 1e-12
    finally:
        jd.config.update("transpose_axis_contiguous", True)


@pytest.mark.parametrize("shape", [(12, 20, 36), (64, 128, 192)])   # general copy kernel / 64x64-tile kernel
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.complex64, torch.complex128])
def test_transposes_single_gpu(dtype, shape):
    x = torch.randn(shape, device=_dev(), dtype=dtype)
    y = jd.transposeXtoY(x, backend="b200")
    assert torch.equal(y, x.permute(2, 0, 1))
    z = jd.transposeYtoZ(y, backend="b200")
    assert torch.equal(z, x.permute(1, 2, 0))
    assert torch.equal(jd.transposeYtoX(jd.transposeZtoY(z, backend="b200"), backend="b200"), x)
    assert torch.equal(jd.transposeZtoX(jd.transposeXtoZ(x, backend="b200"), backend="b200"), x)
    # out=: the rotation is written into the given tensor, also one that lives in a peer-visible block
    dest = torch.full_like(y, 7)
    assert jd.transposeXtoY(x, backend="b200", out=dest).data_ptr() == dest.data_ptr()
    assert torch.equal(dest, y)
    with jd.single_rank_mesh() as mesh:
        pv = jd.empty_peer_visible(mesh, tuple(z.shape), dtype)
        jd.transposeYtoZ(y, backend="b200", out=pv)
        assert torch.equal(pv, z)
        jd.free_peer_visible(mesh)
    with pytest.raises(ValueError):
        jd.transposeXtoY(x, backend="b200", out=torch.empty((3, 3, 3), device=_dev(), dtype=dtype))
    # a batch, and the tile kernels against the general one
    xb = torch.stack([x, 2 * x])
    assert torch.equal(jd.transposeXtoY(xb, backend="b200"), xb.permute(0, 3, 1, 2))


def test_rotating_copy_kernels_match_the_general_kernel(monkeypatch):
    for dtype in (torch.complex64, torch.complex128, torch.float64):
        x = torch.randn((128, 64, 256), device=_dev(), dtype=dtype)
        fast = [jd.transposeXtoY(x, backend="b200"), jd.transposeYtoX(x, backend="b200")]
        monkeypatch.setenv("JD_B200_COPY_FAST", "0")
        slow = [jd.transposeXtoY(x, backend="b200"), jd.transposeYtoX(x, backend="b200")]
        monkeypatch.delenv("JD_B200_COPY_FAST")
        assert torch.equal(fast[0], slow[0]) and torch.equal(fast[1], slow[1])
        assert torch.equal(fast[0], x.permute(2, 0, 1)) and torch.equal(fast[1], x.permute(1, 2, 0))


def test_fft_gradient_matches_torch():
    x = torch.randn((16, 8, 32), device=_dev(), dtype=torch.complex128, requires_grad=True)
    w = torch.rand((8, 32, 16), device=_dev(), dtype=torch.float64)
    (jd.pfft3d(x, norm="ortho", backend="b200").abs().pow(2) * w).sum().backward()
    xr = x.detach().clone().requires_grad_(True)
    (torch.fft.fftn(xr, norm="ortho").permute(1, 2, 0).abs().pow(2) * w).sum().backward()
    torch.testing.assert_close(x.grad, xr.grad, rtol=1e-10, atol=1e-10)
    xf = torch.randn((16, 8, 32), device=_dev(), dtype=torch.float32, requires_grad=True)
    jd.pifft3d(jd.pfft3d(xf, backend="b200") * 2.0, backend="b200").real.pow(2).sum().backward()
    torch.testing.assert_close(xf.grad, 8.0 * xf.detach(), rtol=1e-4, atol=1e-4)


def test_auto_backend_uses_native_kernels_on_cuda():
    from jaxdecomp_b200.ops import b200_backend

    mesh = jd.single_rank_mesh()
    before = b200_backend.launches(mesh)
    x = torch.randn((8, 8, 64), device=_dev(), dtype=torch.complex64)
    jd.pfft3d(x)
    assert b200_backend.launches(mesh) >= before + 3
    b200_backend.check_status(mesh, sync=True)


def test_bounded_wait_times_out_with_status_and_context_survives():
    """A wait on a flag that nothing sets must end by itself with a status
    record, leaving the CUDA context usable."""
    from jaxdecomp_b200 import native
    from jaxdecomp_b200.utils.errors import PeerTimeoutError

    nat = native.require()
    rt = nat.Runtime(1, 0)
    rt.create_arena(1 << 20)
    stream = torch.cuda.current_stream().cuda_stream
    rt.wait_only(2, 7, 50, stream)  # two slots, epoch 7, 50 ms budget
    torch.cuda.synchronize()
    code, peer, expected, seen, where = rt.read_status()
    assert nat.status_name(code) == "TIMEOUT_PEER_SIGNAL" and expected == 7 and seen == 0
    rt.clear_status()
    assert rt.read_status()[0] == 0
    # the context still works
    a = torch.ones(1024, device=_dev())
    assert float(a.sum()) == 1024.0
    rt.destroy_arena()
    assert issubclass(PeerTimeoutError, RuntimeError)


def test_wait_reports_a_slot_that_is_too_far_ahead_as_stale():
    """A slot more than one barrier ahead of the awaited epoch means the ranks stopped counting the
    same barriers; the wait returns at once with STALE_EPOCH (nothing waits, nothing faults)."""
    from jaxdecomp_b200 import native

    nat = native.require()
    rt = nat.Runtime(1, 0)
    rt.create_arena(1 << 20)
    rt.poke_flag(0, 40)  # this rank's own slot jumps to epoch 40
    stream = torch.cuda.current_stream().cuda_stream
    rt.wait_only(1, 7, 50, stream)
    torch.cuda.synchronize()
    code, peer, expected, seen, where = rt.read_status()
    assert nat.status_name(code) == "STALE_EPOCH" and peer == 0 and expected == 7 and seen == 40
    rt.clear_status()
    rt.poke_flag(0, 8)  # one ahead is legal: a peer may already have signalled the next barrier
    rt.wait_only(1, 7, 50, stream)
    torch.cuda.synchronize()
    assert rt.read_status()[0] == 0
    rt.destroy_arena()


def test_checked_build_reports_out_of_range_stores():
    """The library variant compiled with the per-store range check (JD_B200_BOUNDS=1) runs a correct plan
    cleanly and turns a descriptor that claims too small a destination into a BOUNDS status, skipping
    the stores instead of performing them."""
    import os
    import subprocess
    import sys

    code = r"""
import torch, jaxdecomp_b200 as jd
from jaxdecomp_b200 import native
from jaxdecomp_b200.ops import passes, plan
nat = native.require()
assert nat.BOUNDS_CHECK_BUILD
dev = torch.device('cuda', 0)
x = torch.randn(32, 64, 128, device=dev, dtype=torch.complex64)
k = jd.pfft3d(x, backend='b200')
ref = torch.fft.fftn(x).permute(1, 2, 0)
assert ((k - ref).abs().max() / ref.abs().max()).item() < 3e-6
from jaxdecomp_b200.ops import b200_backend
b200_backend.check_status(jd.single_rank_mesh(), sync=True)
steps = plan.fft_steps(jd.NO_DECOMP, False, True, native=True)
specs, _ = passes.compile_passes(steps, x.shape, (1, 1), (0, 0))
rt = nat.Runtime(1, 0)
rt.create_arena(1 << 20)
for sp in specs[:2]:
    d = passes.fill_desc(nat, sp, 8, False, 1.0, 1, False, True)
    out = torch.zeros(sp.out_shape, device=dev, dtype=torch.complex64)
    d.in_ptr = x.data_ptr(); d.set_out(0, out.data_ptr())
    d.out_limit = x.numel() // 2
    nat.launch_pass_checked(d, torch.cuda.current_stream().cuda_stream, rt.status_device_ptr())
    torch.cuda.synchronize()
    st = rt.read_status()
    assert nat.status_name(st[0]) == 'BOUNDS', st
    flat = out.reshape(-1)
    assert float(flat[: x.numel() // 2].abs().sum()) > 0 and float(flat[x.numel() // 2:].abs().sum()) == 0
    rt.clear_status()
print('checked build ok')
"""
    env = dict(os.environ, JD_B200_BOUNDS="1")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "checked build ok" in r.stdout, r.stdout + r.stderr


def test_large_offsets_use_64bit_indexing():
    # 2048 x 1024 x 1024 complex64 = 16 GiB: element offsets exceed 2^31
    free, _ = torch.cuda.mem_get_info()
    if free < 70 * (1 << 30):
        pytest.skip("needs ~64 GiB of free device memory")
    n0, n1, n2 = 2048, 1024, 1024
    x = torch.zeros((n0, n1, n2), device=_dev(), dtype=torch.complex64)
    x[n0 - 1, n1 - 1, 5] = 1.0  # a single impulse near the end of memory
    k = jd.pfft3d(x, backend="b200")
    # DFT of an impulse at (a,b,c): exp(-2 pi i (a k0/n0 + b k1/n1 + c k2/n2)); output layout (k1, k2, k0)
    k0 = torch.arange(0, n0, 397, device=_dev())
    want = torch.exp(-2j * torch.pi * ((n1 - 1) * 3 / n1 + 5 * 7 / n2 + (n0 - 1) * k0.double() / n0)).to(torch.complex64)
    torch.testing.assert_close(k[3, 7, k0], want, rtol=1e-4, atol=1e-4)
    assert abs(float(k.abs().max()) - 1.0) < 1e-4
    del k, x
    torch.cuda.empty_cache()


def test_cuda_graph_capture_of_native_round_trip():
    from jaxdecomp_b200.utils.graphs import capture

    x = torch.randn((32, 64, 128), device=_dev(), dtype=torch.complex64)
    g = capture(lambda v: jd.pifft3d(jd.pfft3d(v, backend="b200") * 2.0, backend="b200"), x)
    for seed in (1, 2):
        y = torch.randn((32, 64, 128), device=_dev(), dtype=torch.complex64, generator=torch.Generator(device=_dev()).manual_seed(seed))
        out = g(y)
        assert _rel(out, 2.0 * y) < 3e-5
