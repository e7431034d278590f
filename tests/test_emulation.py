"""Native tile passes on the CPU emulation: the planner, peer addressing and
FFT butterflies shared with the CUDA kernels, for every decomposition, both
layout modes, both precisions, power-of-two and arbitrary lengths."""
import pytest
import torch

from jaxdecomp_b200 import native
from jaxdecomp_b200.ops import emulate, passes, plan
from jaxdecomp_b200.parallel.mesh import pencil_type_from_pdims

pytestmark = pytest.mark.skipif(not native.available(), reason="native core could not be built (no nvcc)")


def _assemble(outs, pdims, spec, names, gshape):
    p0, p1 = pdims
    full = torch.zeros(gshape, dtype=outs[0].dtype)
    for r, o in enumerate(outs):
        c = (r // p1, r % p1)
        idx = [slice(None)] * 3
        for ax, s in enumerate(spec):
            if s is not None:
                m = names.index(s)
                n = o.shape[ax]
                idx[ax] = slice(c[m] * n, (c[m] + 1) * n)
        full[tuple(idx)] = o
    return full


def _xspec(pdims, names):
    return (names[0] if pdims[0] > 1 else None, names[1] if pdims[1] > 1 else None, None)


@pytest.mark.parametrize("pdims", [(1, 1), (2, 4), (4, 2), (1, 8), (8, 1)])
@pytest.mark.parametrize("contig", [True, False])
@pytest.mark.parametrize("dtype,shape", [(torch.complex64, (8, 16, 32)), (torch.complex128, (24, 40, 56)),
                                         (torch.complex128, (29 * 8, 19 * 8, 17 * 8))])
def test_fft_pipelines(pdims, contig, dtype, shape):
    names = ("a0", "a1")
    x = torch.randn(shape, dtype=dtype, generator=torch.Generator().manual_seed(0))
    pt = pencil_type_from_pdims(pdims)
    steps = plan.fft_steps(pt, False, contig, native=True)
    blocks = emulate.split_blocks(x, pdims)
    outs = emulate.emulate_steps(blocks, steps, pdims, False, 1.0)
    _, ospec = plan.propagate(steps, blocks[0].shape, _xspec(pdims, names), pdims, names)
    ref = torch.fft.fftn(x)
    if contig:
        ref = ref.permute(1, 2, 0)
    full = _assemble(outs, pdims, ospec, names, tuple(ref.shape))
    tol = 2e-6 if dtype == torch.complex64 else 1e-13
    assert (full - ref).abs().max() <= tol * ref.abs().max()
    isteps = plan.fft_steps(pt, True, contig, native=True)
    back = emulate.emulate_steps(outs, isteps, pdims, True, 1.0 / x.numel())
    xb = _assemble(back, pdims, _xspec(pdims, names), names, shape)
    assert (xb - x).abs().max() <= 10 * tol * x.abs().max()


def test_native_slab_xy_steps_equal_literal_ones():
    # the re-ordered forward slab-XY list used by the kernels must match the literal one
    names = ("a0", "a1")
    x = torch.randn((8, 8, 16), dtype=torch.complex128, generator=torch.Generator().manual_seed(1))
    ref = torch.fft.fftn(x).permute(1, 2, 0)
    for native_list in (True, False):
        steps = plan.fft_steps(pencil_type_from_pdims((4, 1)), False, True, native=native_list)
        _, ospec = plan.propagate(steps, (2, 8, 16), ("a0", None, None), (4, 1), names)
        assert ospec == (None, "a0", None)
        if native_list:
            outs = emulate.emulate_steps(emulate.split_blocks(x, (4, 1)), steps, (4, 1))
            full = _assemble(outs, (4, 1), ospec, names, tuple(ref.shape))
            assert (full - ref).abs().max() < 1e-12 * ref.abs().max()


@pytest.mark.parametrize("contig", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.complex64, torch.complex128])
def test_transposes(contig, dtype):
    names = ("a0", "a1")
    pdims = (2, 4)
    shape = (8, 16, 24)
    x = torch.randn(shape, dtype=dtype, generator=torch.Generator().manual_seed(2))
    cur = emulate.split_blocks(x, pdims)
    spec = _xspec(pdims, names)
    for kind, perm in (("x_y", (2, 0, 1)), ("y_z", (1, 2, 0)), ("z_y", (2, 0, 1)), ("y_x", (0, 1, 2)), ("x_z", (1, 2, 0)),
                       ("z_x", (0, 1, 2))):
        steps = plan.transpose_steps(kind, contig)
        lshape = cur[0].shape
        cur = emulate.emulate_steps(cur, steps, pdims)
        _, spec = plan.propagate(steps, lshape, spec, pdims, names)
        want = x.permute(perm) if contig else x
        full = _assemble(cur, pdims, spec, names, tuple(want.shape))
        assert torch.equal(full, want), kind


@pytest.mark.parametrize("pdims", [(1, 1), (1, 4), (4, 1), (2, 2), (2, 4), (4, 2)])
@pytest.mark.parametrize("dtype", [torch.complex64, torch.complex128, torch.float64])
def test_rotating_copy_kernels_addressing_on_every_mesh(pdims, dtype):
    """The rotating copy kernels (64 x 64 / 32 x 32 tiles, ``csrc/copy_fast.cu``) in their host restatement:
    the chain of all six transposes on slabs, pencils and a single rank, against the global permutation."""
    names = ("a0", "a1")
    n = 64 * max(pdims)          # every local extent of every pencil orientation is a multiple of the 64-wide tile
    shape = (n, n, n)
    x = torch.randn(shape, dtype=dtype, generator=torch.Generator().manual_seed(12))
    cur = emulate.split_blocks(x, pdims)
    spec = _xspec(pdims, names)
    used = 0
    kinds = [("x_y", (2, 0, 1)), ("y_z", (1, 2, 0)), ("z_y", (2, 0, 1)), ("y_x", (0, 1, 2))]
    if pdims[0] > 1 and pdims[1] > 1:
        kinds += [("x_z", (1, 2, 0)), ("z_x", (0, 1, 2))]
    for kind, perm in kinds:
        steps = plan.transpose_steps(kind, True)
        lshape = cur[0].shape
        stats = {}
        cur = emulate.emulate_steps(cur, steps, pdims, copy_twin=True, stats=stats)
        used += stats["twin_passes"]
        _, spec = plan.propagate(steps, lshape, spec, pdims, names)
        full = _assemble(cur, pdims, spec, names, tuple(x.permute(perm).shape))
        assert torch.equal(full, x.permute(perm)), kind
    # every pass of every rank went through the tile kernels' restatement
    assert used == len(kinds) * pdims[0] * pdims[1]


def test_rotating_copy_kernels_are_not_chosen_for_other_shapes():
    nat = native.require()
    for lshape, eb, want in (((64, 64, 128), 8, True), ((64, 64, 128), 4, False), ((60, 64, 128), 8, True), ((64, 60, 128), 8, False),
                             ((32, 32, 32), 16, True), ((32, 32, 32), 8, False)):
        specs, _ = passes.compile_passes(plan.transpose_steps("x_y", True), lshape, (1, 1), (0, 0))
        d = passes.fill_desc(nat, specs[0], eb, False, 1.0, 1, remote=False, device_tables=False)
        buf = torch.zeros(specs[0].numel * eb + 64, dtype=torch.uint8)
        d.in_ptr = buf.data_ptr()
        d.set_out(0, buf.data_ptr())
        assert nat.copy_fast_eligible(d) == want, (lshape, eb)
        d.in_ptr = buf.data_ptr() + 8            # an operand that is not 16-byte aligned
        assert nat.copy_fast_eligible(d) == (want and eb == 16), (lshape, eb)
    # the non-contiguous layout mode moves no axes: not a rotating pass
    specs, _ = passes.compile_passes(plan.transpose_steps("x_y", False), (64, 64, 128), (1, 2), (0, 0))
    d = passes.fill_desc(nat, specs[0], 8, False, 1.0, 1, remote=True, device_tables=False)
    assert not nat.copy_fast_eligible(d)


def test_batched_blocks():
    pdims = (2, 2)
    names = ("a0", "a1")
    x = torch.randn((3, 8, 8, 16), dtype=torch.complex64, generator=torch.Generator().manual_seed(3))
    steps = plan.fft_steps(pencil_type_from_pdims(pdims), False, True, native=True)
    outs = emulate.emulate_steps(emulate.split_blocks(x, pdims), steps, pdims)
    ref = torch.fft.fftn(x, dim=(1, 2, 3)).permute(0, 2, 3, 1)
    for b in range(3):
        full = _assemble([o[b] for o in outs], pdims, ("a0", "a1", None), names, tuple(ref.shape[1:]))
        assert (full - ref[b]).abs().max() < 1e-5 * ref.abs().max()


def test_invalid_descriptor_is_rejected():
    nat = native.require()
    d = nat.PassDesc()
    assert nat.validate_pass(d) != 0
    with pytest.raises(ValueError):
        nat.run_pass_host(d)


@pytest.mark.parametrize("n", [64, 128, 256, 512, 1024, 2048, 4096, 100, 384,
                               2, 4, 6, 12, 30, 77, 143, 768, 1000, 1365, 1536, 2310, 34, 97,
                               96, 160, 240, 288, 480])
@pytest.mark.parametrize("dtype", [torch.complex64, torch.complex128])
def test_row_transforms_all_stage_structures(n, dtype):
    """Every radix structure (8.8.2, 8.8.4, 8.8.8, ...) with intra-row padding, mixed-radix lengths
    covering the radices 2..16 and the primes up to 13, and Bluestein lengths (34, 97);
    contiguous and strided, forward and inverse."""
    x = torch.randn((3, 4, n), dtype=dtype, generator=torch.Generator().manual_seed(n))
    tol = 3e-6 if dtype == torch.complex64 else 1e-13
    out = emulate.emulate_steps([x], [plan.Fft(2)], (1, 1))[0]
    ref = torch.fft.fft(x, dim=2)
    assert (out - ref).abs().max() <= tol * ref.abs().max()
    out = emulate.emulate_steps([x], [plan.Fft(2), plan.Perm((2, 0, 1))], (1, 1), inverse=True)[0]
    ref = torch.fft.ifft(x, dim=2, norm="forward").permute(2, 0, 1)
    assert (out - ref).abs().max() <= tol * ref.abs().max()
    y = x.permute(2, 0, 1).contiguous()  # transform along the slowest axis
    out = emulate.emulate_steps([y], [plan.Fft(0)], (1, 1))[0]
    ref = torch.fft.fft(y, dim=0)
    assert (out - ref).abs().max() <= tol * ref.abs().max()


def test_mixed_radix_selection():
    """Lengths with prime factors up to 13 take the mixed-radix mode, others Bluestein, powers of two >= 8 their own."""
    from jaxdecomp_b200.ops import passes

    def mode(n):
        specs, _ = passes.compile_passes([plan.Fft(2)], (2, 16, n), (1, 1), (0, 0))
        return passes.choose_tiling(specs[0], 8, False)

    assert mode(768)["fft_mode"] == 3 and mode(768)["M"] == 768
    assert mode(1000)["fft_mode"] == 3
    assert mode(4)["fft_mode"] == 3
    assert mode(1024)["fft_mode"] == 1
    assert mode(34)["fft_mode"] == 2 and mode(34)["M"] == 128
    t = mode(768)
    assert t["intra_pad"] == 1 and t["pitch"] % 16 == 2 and t["pitch"] >= 768 + 2 * 48
    assert 2 * t["T"] * t["pitch"] * 8 <= 226 * 1024
    specs, _ = passes.compile_passes([plan.Fft(2)], (2, 4, 768), (1, 1), (0, 0))
    t4 = passes.choose_tiling(specs[0], 8, False)   # four rows per tile: pitch == 4 (mod 16)
    assert t4["T"] == 4 and t4["pitch"] % 16 == 4
    assert not passes.mixed_radix_ok(2 * 17, 8)


_MIXED_MENU = [96, 192, 384, 768, 1536, 3072, 288, 576, 1152, 2304, 160, 320, 640, 1280, 2560, 200, 400, 800, 1600,
               250, 500, 1000, 2000, 240, 480, 960, 1920, 448, 896, 1792]


@pytest.mark.parametrize("elem_bytes", [8, 16])
def test_specialised_mixed_kernels_see_the_tiling_they_expect(elem_bytes):
    """The length-specialised kernels are only used when the planner's tile height and pitch equal the
    compile-time geometry: both sides must apply the same rules, for plain and for rotating passes."""
    from jaxdecomp_b200.ops import passes

    nat = native.require()
    for n in _MIXED_MENU:
        for steps, store_t in (([plan.Fft(2)], False), ([plan.Fft(2), plan.Perm(plan.ROT_FWD)], True)):
            specs, _ = passes.compile_passes(steps, (64, 64, n), (1, 1), (0, 0))
            t = passes.choose_tiling(specs[0], elem_bytes, False)
            g = nat.mixed_static_geometry(n, elem_bytes, store_t)
            assert t["fft_mode"] == 3 and (t["T"], t["pitch"]) == (g["T"], g["pitch"]), (n, store_t, t, g)
            assert g["tpr"] >= 1 and g["T"] * g["tpr"] <= (512 if elem_bytes == 8 else 256)
            prod = 1
            for r in g["radices"]:
                prod *= r
            assert prod == n and len(g["radices"]) >= 2
            # two buffers of T rows fit the shared memory of one block
            assert 2 * g["T"] * g["pitch"] * elem_bytes <= 226 * 1024


def test_last_stage_thread_maps_are_bijections():
    """Rotating passes re-assign threads across rows for the last stage: every (row, butterfly index) pair
    must be served by exactly one thread, and consecutive threads must hold consecutive rows."""
    nat = native.require()
    for T in (2, 4, 8, 16, 32):
        for upr in (8, 16, 32, 64, 128, 256):
            nt = T * upr
            if nt > 1024:
                continue
            seen = {nat.fast_last_stage_map(T, tid) for tid in range(nt)}
            assert seen == {(r, j) for r in range(T) for j in range(upr)}, (T, upr)
            assert [nat.fast_last_stage_map(T, tid)[0] for tid in range(min(T, 8))] == list(range(min(T, 8)))
    # the specialised mixed-radix kernels, with the geometry they are compiled for
    for eb in (8, 16):
        for n in _MIXED_MENU:
            g = nat.mixed_static_geometry(n, eb, True)
            T, tpr = g["T"], g["tpr"]
            nt = (T * tpr + 31) // 32 * 32
            got = [nat.mixed_last_stage_map(T, eb, tid) for tid in range(nt)]
            active = [(r, j) for r, j in got if j < tpr]
            assert all(0 <= r < T for r, _ in got)
            assert len(set(active)) == len(active), (eb, n)
            assert set(active) == {(r, j) for r in range(T) for j in range(tpr)}, (eb, n, T, tpr)


def _host_table(ptr, count, dtype):
    import ctypes

    import numpy as np

    nbytes = count * np.dtype(dtype).itemsize
    buf = (ctypes.c_char * nbytes).from_address(ptr)
    return np.frombuffer(buf, dtype=dtype, count=count).copy()


@pytest.mark.parametrize("elem_bytes", [8, 16])
def test_stage_twiddle_records_of_the_power_of_two_kernel(elem_bytes):
    """The specialised power-of-two kernel has no CPU path, so its per-stage twiddle records are checked
    here: record kk of stage s holds w, w^2, w^4, w^8 with w = exp(-2 pi i kk / (Ls * radix))."""
    import numpy as np

    nat = native.require()
    radix_log = {7: [4, 3], 8: [4, 4], 9: [3, 3, 3], 10: [4, 3, 3], 11: [4, 4, 3], 12: [4, 4, 4]}
    cdt = np.complex64 if elem_bytes == 8 else np.complex128
    for logm, plan_ in radix_log.items():
        m = 1 << logm
        tw, _, _, tws = nat.get_fft_tables(m, m, elem_bytes, False)
        assert tw and tws
        roots = _host_table(tw, m, cdt)
        np.testing.assert_allclose(roots, np.exp(-2j * np.pi * np.arange(m) / m), atol=1e-7 if elem_bytes == 8 else 1e-15)
        ls, rec0 = 1, 0
        nrec = sum((1 << sum(plan_[:s])) for s in range(1, len(plan_)))
        recs = _host_table(tws, nrec * 4, cdt).reshape(nrec, 4)
        for s, rl in enumerate(plan_):
            if s > 0:
                span = ls << rl
                kk = np.arange(ls)[:, None]
                want = np.exp(-2j * np.pi * (kk << np.arange(4)[None, :]) / span)
                np.testing.assert_allclose(recs[rec0:rec0 + ls], want, atol=1e-7 if elem_bytes == 8 else 1e-15)
                rec0 += ls
            ls <<= rl


def test_stage_twiddle_records_of_the_mixed_radix_kernels():
    import numpy as np

    nat = native.require()
    for n in (768, 1000, 96, 2310):
        g = nat.mixed_static_geometry(n, 16, False)
        tw, _, _, tws = nat.get_fft_tables(n, n, 16, False)
        assert tw and tws
        ls, rec0 = 1, 0
        radices = list(g["radices"])
        nrec = 0
        acc = 1
        for s, r in enumerate(radices):
            if s > 0:
                nrec += acc
            acc *= r
        recs = _host_table(tws, nrec * 4, np.complex128).reshape(nrec, 4)
        for s, r in enumerate(radices):
            if s > 0:
                tw_mul = n // (ls * r)
                kk = np.arange(ls)[:, None]
                want = np.exp(-2j * np.pi * ((kk * tw_mul * (1 << np.arange(4))[None, :]) % n) / n)
                np.testing.assert_allclose(recs[rec0:rec0 + ls], want, atol=1e-15)
                rec0 += ls
            ls *= r
