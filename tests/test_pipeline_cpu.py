"""Pipelined transports on the CPU: how an exchange pass and the local pass after it are cut into
matching chunks, that running the chunks in pipeline order gives bit-identical results, the checked
stores of the emulation, and the per-chunk barrier protocol with a withheld signal."""
import pytest
import torch

from jaxdecomp_b200 import native
from jaxdecomp_b200.ops import emulate, passes, plan
from jaxdecomp_b200.parallel.mesh import pencil_type_from_pdims
from jaxdecomp_b200.parallel.protocol import OK, TIMEOUT_PEER_SIGNAL, FlagBoard, PipelineModel

pytestmark = pytest.mark.skipif(not native.available(), reason="native core could not be built (no nvcc)")


def _specs(pdims, inverse, contig, lshape):
    pt = pencil_type_from_pdims(pdims)
    steps = plan.fft_steps(pt, inverse, contig, native=True)
    specs, _ = passes.compile_passes(steps, lshape, pdims, (0, 0))
    return steps, specs


@pytest.mark.parametrize("pdims,inverse,expect", [
    # slab 1xP forward: exchange (FFT z) then local FFT y then local FFT x: pair (0, 1)
    ((1, 8), False, {0}),
    # slab inverse: local, exchange, local: the exchange pairs with the pass after it
    ((1, 8), True, {1}),
    # pencils: the second exchange is followed by the last, local pass
    ((2, 4), False, {1}),
    ((2, 4), True, {1}),
    # slab Px1 forward splits along the o axis of its exchange pass: no admissible cut
    ((8, 1), False, set()),
    ((8, 1), True, {0}),
    ((1, 1), False, set()),
])
def test_pipeline_cut_finds_the_exchange_local_pairs(pdims, inverse, expect):
    n = 256
    lshape = (n // pdims[0], n // pdims[1], n)
    if inverse:  # the inverse starts from the block the forward transform produces
        fwd = plan.fft_steps(pencil_type_from_pdims(pdims), False, True, native=True)
        lshape, _ = plan.propagate(fwd, lshape, ("a0" if pdims[0] > 1 else None, "a1" if pdims[1] > 1 else None, None),
                                   pdims, ("a0", "a1"))
    _, specs = _specs(pdims, inverse, True, lshape)
    found = set()
    for i in range(len(specs) - 1):
        cut = passes.pipeline_cut(specs[i], specs[i + 1], 4)
        if cut is not None:
            found.add(i)
            pr, cr, k = cut
            assert pr in (2, 3) and cr in (2, 3) and k in (2, 4)
            # the cut never runs along the axis that selects the destination peer
            assert specs[i].chunks[pr - 1] == specs[i].ext[pr - 1]
            assert specs[i].ext[pr - 1] == specs[i + 1].ext[cr - 1]
    assert found == expect


def test_pipeline_cut_respects_tile_granularity():
    # a t-axis cut must keep whole 32-row tiles: 64 rows allow 2 chunks, not 4
    _, specs = _specs((1, 2), False, True, (64, 32, 64))
    cut = passes.pipeline_cut(specs[0], specs[1], 8)
    assert cut is not None
    pr, cr, k = cut
    ext = specs[0].ext[pr - 1]
    if pr == 2 or cr == 2:
        assert (ext // k) % 32 == 0
    assert ext % k == 0


@pytest.mark.parametrize("pdims", [(1, 4), (4, 1), (2, 2), (2, 4)])
@pytest.mark.parametrize("contig", [True, False])
@pytest.mark.parametrize("dtype", [torch.complex64, torch.complex128])
def test_pipelined_order_is_bit_identical(pdims, contig, dtype):
    shape = (64, 64, 128)
    x = torch.randn(shape, dtype=dtype, generator=torch.Generator().manual_seed(3))
    pt = pencil_type_from_pdims(pdims)
    for inverse in (False, True):
        steps = plan.fft_steps(pt, inverse, contig, native=True)
        blocks = emulate.split_blocks(x, pdims) if not inverse else None
        if inverse:
            fwd = plan.fft_steps(pt, False, contig, native=True)
            blocks = emulate.emulate_steps(emulate.split_blocks(x, pdims), fwd, pdims)
        plain = emulate.emulate_steps(blocks, steps, pdims, inverse, 0.5)
        piped = emulate.emulate_steps(blocks, steps, pdims, inverse, 0.5, pipeline_chunks=4)
        for a, b in zip(plain, piped):
            assert torch.equal(a, b)


def test_restricted_pass_covers_exactly_its_rows():
    nat = native.require()
    _, specs = _specs((1, 2), False, True, (64, 32, 64))
    sp = specs[1]  # local rotating pass
    d = passes.fill_desc(nat, sp, 8, False, 1.0, 1, remote=False, device_tables=False)
    d.use_bulk = 0
    x = torch.randn(sp.in_shape, dtype=torch.complex64)
    full = torch.zeros(sp.out_shape, dtype=torch.complex64)
    d.in_ptr = x.data_ptr()
    d.set_out(0, full.data_ptr())
    nat.run_pass_host(d)
    parts = torch.zeros_like(full)
    d.set_out(0, parts.data_ptr())
    for role in (2, 3):
        parts.zero_()
        ext = sp.ext[role - 1]
        if role == 2 and ext % 64:
            continue
        half = ext // 2
        nat.run_pass_host(d.restricted(role, 0, half))
        assert not torch.equal(parts, full)
        nat.run_pass_host(d.restricted(role, half, half))
        assert torch.equal(parts, full)
    # a range along the axis that selects the peer, or off a tile boundary, is refused
    with pytest.raises(ValueError):
        d.restricted(1, 0, 8)
    with pytest.raises(ValueError):
        d.restricted(2, 8, 24)


def test_emulation_reports_a_store_outside_the_destination():
    nat = native.require()
    _, specs = _specs((1, 1), False, True, (8, 16, 32))
    sp = specs[0]
    d = passes.fill_desc(nat, sp, 8, False, 1.0, 1, remote=False, device_tables=False)
    d.use_bulk = 0
    x = torch.randn(sp.in_shape, dtype=torch.complex64)
    out = torch.zeros(sp.out_shape, dtype=torch.complex64)
    d.in_ptr = x.data_ptr()
    d.set_out(0, out.data_ptr())
    assert d.out_limit == x.numel()
    nat.run_pass_host(d)  # the correct descriptor passes the check
    d.out_limit = x.numel() // 2  # claim a smaller buffer: every store past it must be skipped and reported
    out.zero_()
    with pytest.raises(RuntimeError, match="BOUNDS"):
        nat.run_pass_host(d)
    flat = out.reshape(-1)
    assert flat[: x.numel() // 2].abs().sum() > 0 and flat[x.numel() // 2:].abs().sum() == 0


def test_pipeline_protocol_chunks_arrive_in_order():
    m = PipelineModel(FlagBoard(4), chunks=4)
    log = m.run()
    assert all(code == OK for (_, _, code) in log)
    # every rank consumed chunk k only after every rank had produced chunk k
    for r in range(4):
        assert [k for (rr, k, _) in log if rr == r] == [0, 1, 2, 3]
    assert m.consumed_before_produced == 0


def test_pipeline_protocol_withheld_chunk_signal_times_out_and_aborts_all():
    # rank 2 never signals chunk 1 (the section's second barrier, epoch 2) to rank 0
    board = FlagBoard(4, drop=lambda src, dst, epoch: src == 2 and dst == 0 and epoch == 2)
    m = PipelineModel(board, chunks=4)
    log = m.run()
    codes = {(r, k): code for (r, k, code) in log}
    assert codes[(0, 0)] == OK and codes[(0, 1)] == TIMEOUT_PEER_SIGNAL
    # after the time-out rank 0 marks every rank as aborted: nobody consumes a later chunk
    assert all(k <= 1 for (r, k, code) in log if code == OK)
    assert board.aborted == [1, 1, 1, 1]
    assert m.consumed_before_produced == 0


@pytest.mark.parametrize("pdims", [(1, 1), (2, 2), (1, 4)])
def test_fused_displacement_multiplier_in_the_first_inverse_pass(pdims):
    """Entry b of the batched inverse plan reads delta_k * i k_b / k^2 (multiplier applied inside the first
    pass): against the explicit potentials transformed with torch."""
    import math

    n = (16, 8, 32)
    box = (10.0, 20.0, 30.0)
    names = ("a0", "a1")
    x = torch.randn(n, dtype=torch.complex128, generator=torch.Generator().manual_seed(9))
    pt = pencil_type_from_pdims(pdims)
    fwd = plan.fft_steps(pt, False, True, native=True)
    kblocks = emulate.emulate_steps(emulate.split_blocks(x, pdims), fwd, pdims)
    xspec = (names[0] if pdims[0] > 1 else None, names[1] if pdims[1] > 1 else None, None)
    _, kspec = plan.propagate(fwd, kblocks[0].shape, xspec, pdims, names)
    p0, p1 = pdims
    offs = []
    for r in range(p0 * p1):
        c = (r // p1, r % p1)
        offs.append([0 if s is None else c[names.index(s)] * kblocks[r].shape[ax] for ax, s in enumerate(kspec)])
    inv = plan.fft_steps(pt, True, True, native=True)
    outs = emulate.emulate_steps(kblocks, inv, pdims, True, 1.0 / x.numel(), fused_mul=(n, offs, box))
    # oracle on the gathered spectrum
    kf = [2 * math.pi / box[a] * torch.fft.fftfreq(n[a], d=1.0 / n[a], dtype=torch.float64) for a in range(3)]
    k0, k1, k2 = kf[0].view(-1, 1, 1), kf[1].view(1, -1, 1), kf[2].view(1, 1, -1)
    kk = k0 ** 2 + k1 ** 2 + k2 ** 2
    invk = torch.where(kk > 0, 1.0 / kk.clamp_min(1e-30), torch.zeros_like(kk))
    xk = torch.fft.fftn(x)
    for b, kb in enumerate((k0, k1, k2)):
        want = torch.fft.ifftn(xk * (1j * kb * invk))
        got = torch.zeros(n, dtype=torch.complex128)
        for r, o in enumerate(outs):
            c = (r // p1, r % p1)
            l0, l1 = n[0] // p0, n[1] // p1
            got[c[0] * l0:(c[0] + 1) * l0, c[1] * l1:(c[1] + 1) * l1, :] = o[b]
        torch.testing.assert_close(got, want, rtol=1e-10, atol=1e-12)
