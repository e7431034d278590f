"""Host side of the native core under AddressSanitizer + UndefinedBehaviorSanitizer.

``native.build_host_selftest()`` compiles the CPU emulation of the tile pass and the table construction
with ``g++ -fsanitize=address,undefined`` into a stand-alone program.  The planner's descriptors for a
spread of passes (power-of-two, mixed-radix and Bluestein transforms, copy passes, exchanges over
several peers, batches, both element widths, the inverse direction, a pipelined chunk) are written to a
file together with their operands; the program runs each pass on heap blocks of exactly the claimed
sizes -- a stray index or undefined arithmetic aborts it -- and its results must equal those of the
regular build bit for bit.
"""
import struct
import subprocess

import pytest
import torch

from jaxdecomp_b200 import native
from jaxdecomp_b200.ops import passes, plan
from jaxdecomp_b200.parallel.mesh import pencil_type_from_pdims

pytestmark = pytest.mark.skipif(not native.available() or native.sanitizer_compiler() is None,
                                reason="needs the native core and a C++ compiler with the sanitizer run-times")

MAGIC = 0x32464C455342444A


def _cases(nat):
    """(descriptor, operand, destination sizes in elements) for every pass of a few plans, as rank (0, 0)."""
    out = []
    todo = [
        ((1, 1), (8, 16, 32), torch.complex64, False, True, 1),       # power of two, rotating + plain passes
        ((1, 1), (6, 10, 12), torch.complex128, True, True, 2),       # mixed radix, inverse, batch of two
        ((1, 1), (4, 6, 29), torch.complex64, False, True, 1),        # a prime length: Bluestein
        ((2, 2), (8, 8, 32), torch.complex64, False, True, 1),        # pencils: exchanges over two peers
        ((1, 4), (16, 8, 64), torch.complex128, True, False, 1),      # slab, non-contiguous layout mode
    ]
    for pdims, lshape, dtype, inverse, contig, batch in todo:
        steps = plan.fft_steps(pencil_type_from_pdims(pdims), inverse, contig, native=True)
        specs, _ = passes.compile_passes(steps, lshape, pdims, (0, 0))
        eb = torch.empty((), dtype=dtype).element_size()
        for sp in specs:
            d = passes.fill_desc(nat, sp, eb, inverse, 0.5, batch, remote=sp.npeers > 1, device_tables=False)
            d.use_bulk = 0
            x = torch.randn((batch,) + tuple(sp.in_shape), dtype=dtype, generator=torch.Generator().manual_seed(len(out)))
            out.append((d, x.contiguous(), [sp.numel * batch] * sp.npeers, 0))
    # the six transposes as copy passes on float32 (4-byte elements)
    for kind in plan.TRANSPOSE_KINDS:
        specs, _ = passes.compile_passes(plan.transpose_steps(kind, True), (8, 12, 16), (2, 2), (0, 0))
        for sp in specs:
            d = passes.fill_desc(nat, sp, 4, False, 1.0, 1, remote=sp.npeers > 1, device_tables=False)
            d.use_bulk = 0
            x = torch.randn(tuple(sp.in_shape), dtype=torch.float32, generator=torch.Generator().manual_seed(99))
            out.append((d, x.contiguous(), [sp.numel] * sp.npeers, 0))
    # rotating copy passes in the host restatement of the 64 x 64-tile kernels, local and over two peers
    for pdims, lshape, eb, dtype in (((1, 1), (64, 128, 64), 8, torch.complex64), ((1, 2), (64, 64, 128), 8, torch.float64),
                                     ((2, 2), (32, 32, 64), 16, torch.complex128)):
        for kind in ("x_y", "y_x"):
            specs, _ = passes.compile_passes(plan.transpose_steps(kind, True), lshape, pdims, (0, 0))
            sp = specs[0]
            d = passes.fill_desc(nat, sp, eb, False, 1.0, 1, remote=sp.npeers > 1, device_tables=False)
            d.use_bulk = 0
            x = torch.randn(tuple(sp.in_shape), dtype=dtype, generator=torch.Generator().manual_seed(7))
            out.append((d, x.contiguous(), [sp.numel] * sp.npeers, 1))
    # one chunk of a pipelined local pass
    specs, _ = passes.compile_passes(plan.fft_steps(pencil_type_from_pdims((1, 2)), False, True, native=True),
                                     (64, 32, 64), (1, 2), (0, 0))
    sp = specs[1]
    d = passes.fill_desc(nat, sp, 8, False, 1.0, 1, remote=False, device_tables=False)
    d.use_bulk = 0
    half = sp.ext[2] // 2
    x = torch.randn(tuple(sp.in_shape), dtype=torch.complex64, generator=torch.Generator().manual_seed(5))
    out.append((d.restricted(3, half, half), x.contiguous(), [sp.numel], 0))
    return out


def test_host_passes_are_clean_under_asan_and_ubsan(tmp_path):
    nat = native.require()
    exe = native.build_host_selftest()
    cases = _cases(nat)
    want = []
    blob = [struct.pack("<QQQ", MAGIC, len(cases[0][0].raw_bytes()), len(cases))]
    for d, x, out_elems, mode in cases:
        eb = d.elem_bytes
        raw = bytes(x.view(torch.uint8).reshape(-1).numpy()) if x.numel() else b""
        blob += [d.raw_bytes(), struct.pack("<Q", mode), struct.pack("<Q", len(raw)), raw, struct.pack("<Q", len(out_elems))]
        blob += [struct.pack("<Q", n * eb) for n in out_elems]
        # the regular build on the same descriptor
        outs = [torch.zeros(n * eb, dtype=torch.uint8) for n in out_elems]
        d.in_ptr = x.data_ptr()
        for p, o in enumerate(outs):
            d.set_out(p, o.data_ptr())
        if mode == 1:
            assert nat.copy_fast_eligible(d)
        nat.run_pass_host(d)          # the general pass is the oracle for the restated kernels too
        want += outs
    (tmp_path / "cases.bin").write_bytes(b"".join(blob))
    r = subprocess.run([str(exe), str(tmp_path / "cases.bin"), str(tmp_path / "results.bin")], capture_output=True,
                       text=True, timeout=600,
                       env={"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0", "UBSAN_OPTIONS": "print_stacktrace=1",
                            "PATH": "/usr/bin:/bin"})
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ERROR: AddressSanitizer" not in r.stderr and "runtime error" not in r.stderr, r.stderr
    assert f"{len(cases)} cases ok" in r.stdout
    got = (tmp_path / "results.bin").read_bytes()
    assert len(got) == sum(o.numel() for o in want)
    pos = 0
    for i, o in enumerate(want):
        assert got[pos:pos + o.numel()] == bytes(o.numpy()), f"destination {i} differs from the regular build"
        pos += o.numel()


def test_sanitizer_build_catches_a_descriptor_that_overruns_its_destination(tmp_path):
    """The self-test's heap blocks have the claimed sizes: a descriptor whose destination is claimed too
    small (and whose own store check is told otherwise) must be stopped by AddressSanitizer."""
    nat = native.require()
    exe = native.build_host_selftest()
    specs, _ = passes.compile_passes(plan.fft_steps(pencil_type_from_pdims((1, 1)), False, True, native=True),
                                     (8, 16, 32), (1, 1), (0, 0))
    sp = specs[0]
    d = passes.fill_desc(nat, sp, 8, False, 1.0, 1, remote=False, device_tables=False)
    d.use_bulk = 0
    x = torch.randn(tuple(sp.in_shape), dtype=torch.complex64, generator=torch.Generator().manual_seed(1))
    raw = bytes(x.view(torch.uint8).reshape(-1).numpy())
    short = sp.numel * 8 // 2                       # half of what the pass writes; out_limit still says "all"
    blob = [struct.pack("<QQQ", MAGIC, len(d.raw_bytes()), 1), d.raw_bytes(), struct.pack("<Q", 0), struct.pack("<Q", len(raw)), raw,
            struct.pack("<Q", 1), struct.pack("<Q", short)]
    (tmp_path / "bad.bin").write_bytes(b"".join(blob))
    r = subprocess.run([str(exe), str(tmp_path / "bad.bin"), str(tmp_path / "out.bin")], capture_output=True, text=True,
                       timeout=600, env={"ASAN_OPTIONS": "detect_leaks=0:abort_on_error=0", "PATH": "/usr/bin:/bin"})
    assert r.returncode != 0
    assert "AddressSanitizer: heap-buffer-overflow" in r.stderr
