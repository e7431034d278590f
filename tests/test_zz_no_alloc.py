"""The allocation-free local FFT entry point (``jdb_fft3d_c64_static``).

Some callers of this library cannot allocate device memory at the moment they
call it -- code inside a stream capture, a real-time loop that must not block
on the allocator, a C or Fortran host with no tensor framework to own
temporaries.  For them the library exports one C entry point whose scratch
memory is a fixed device array.  This test calls it through the exported C
symbol, twice in a row (the scratch is shared between calls), and checks the
results against the regular entry point.  It is collected last so that a run
that stops at the first failure has already executed every other test.
"""
import ctypes

import pytest
import torch

import jaxdecomp_b200 as jd
from jaxdecomp_b200 import native

pytestmark = pytest.mark.gpu


def _lib():
    native.require()
    lib = ctypes.CDLL(str(native.so_path()))
    lib.jdb_fft3d_c64_static.restype = ctypes.c_int
    lib.jdb_fft3d_c64_static.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                         ctypes.c_int, ctypes.c_void_p]
    lib.jdb_fft3d_c64_static_error.restype = ctypes.c_char_p
    return lib


def _rel(a, b):
    return ((a - b).abs().max() / b.abs().max()).item()


def test_static_scratch_fft_matches_regular_entry_point_twice():
    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    n0, n1, n2 = 32, 64, 128  # exactly the documented maximum of 262144 elements
    x = torch.randn((n0, n1, n2), device=dev, dtype=torch.complex64)
    k = torch.empty((n1, n2, n0), device=dev, dtype=torch.complex64)
    # first call: forward transform
    rc = lib.jdb_fft3d_c64_static(x.data_ptr(), k.data_ptr(), n0, n1, n2, 0, stream)
    assert rc == 0, lib.jdb_fft3d_c64_static_error()
    torch.cuda.synchronize()
    want = jd.pfft3d(x, backend="b200")
    assert _rel(k, want) < 3e-6
    assert _rel(k, torch.fft.fftn(x).permute(1, 2, 0)) < 3e-6
    # second call right after, on other data and in the other direction: the shared scratch is reused
    back = torch.empty_like(x)
    rc = lib.jdb_fft3d_c64_static(k.data_ptr(), back.data_ptr(), n0, n1, n2, 1, stream)
    assert rc == 0, lib.jdb_fft3d_c64_static_error()
    torch.cuda.synchronize()
    assert _rel(back, jd.pifft3d(want, backend="b200")) < 3e-5
    assert _rel(back, x) < 3e-5
    # a smaller problem after a larger one must not see stale scratch contents
    y = torch.randn((8, 16, 32), device=dev, dtype=torch.complex64)
    ky = torch.empty((16, 32, 8), device=dev, dtype=torch.complex64)
    assert lib.jdb_fft3d_c64_static(y.data_ptr(), ky.data_ptr(), 8, 16, 32, 0, stream) == 0
    torch.cuda.synchronize()
    assert _rel(ky, jd.pfft3d(y, backend="b200")) < 3e-6


def test_static_scratch_fft_rejects_what_does_not_fit():
    lib = _lib()
    dev = torch.device("cuda", 0)
    a = torch.zeros(16, device=dev, dtype=torch.complex64)
    b = torch.zeros(16, device=dev, dtype=torch.complex64)
    assert lib.jdb_fft3d_c64_static(a.data_ptr(), b.data_ptr(), 64, 64, 128, 0, None) != 0
    assert b"exceeds" in lib.jdb_fft3d_c64_static_error()
    assert lib.jdb_fft3d_c64_static(a.data_ptr(), b.data_ptr(), 8, 12, 8, 0, None) != 0
    assert b"power of two" in lib.jdb_fft3d_c64_static_error()
    assert lib.jdb_fft3d_c64_static(a.data_ptr(), a.data_ptr(), 8, 8, 8, 0, None) != 0
    assert b"alias" in lib.jdb_fft3d_c64_static_error()
    buf = torch.zeros(1024, device=dev, dtype=torch.complex64)
    assert lib.jdb_fft3d_c64_static(buf.data_ptr(), buf[256:].data_ptr(), 8, 8, 8, 0, None) != 0   # half-overlapping ranges
    assert b"overlap" in lib.jdb_fft3d_c64_static_error()
    assert lib.jdb_fft3d_c64_static(buf.data_ptr(), buf[512:].data_ptr(), 8, 8, 8, 0, None) == 0   # adjacent ranges are fine
    torch.cuda.synchronize()
