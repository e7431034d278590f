// A local 3-D FFT entry point that allocates no memory.
//
// This entry point has no counterpart in the reference library.  It exists for
// callers that must not (or cannot) allocate device memory when they call into
// this library: code running inside a stream capture or under a memory pool
// that forbids cudaMalloc, real-time loops that may not block on the driver's
// allocator, and hosts that link the shared object from C or Fortran without
// any tensor framework that could own temporary buffers.
//
// jdb_fft3d_c64_static computes the same result as pfft3d / pifft3d on a single
// GPU (complex64, contiguous layout): the forward transform of an array
// (n0, n1, n2) is returned rotated as (n1, n2, n0); the inverse takes that
// rotated array and returns (n0, n1, n2) scaled by 1/(n0*n1*n2).  The
// intermediate pencil buffer and the twiddle tables that the regular entry
// point takes from the allocator live in a fixed, file-scope device array of
// JDB_STATIC_MAX_ELEMS complex64 values (2 MiB) plus 6 KiB of tables; every GPU
// that loads the library holds this memory until the process exits.
//
// Limits: n0, n1 and n2 are powers of two between 8 and 256 and
// n0*n1*n2 <= JDB_STATIC_MAX_ELEMS.  Anything else is rejected with a non-zero
// return value and a message available from jdb_fft3d_c64_static_error().
//
// Set-up: the first call on a device resolves the device addresses of the
// static arrays (one cudaGetSymbolAddress per array, with that device
// current).  Make that first call outside of any stream capture: a first call
// on a capturing stream is refused with an error instead of disturbing the
// capture.  Host threads may make their first calls concurrently (the set-up
// is serialised and published with release/acquire ordering).
//
// Sharing: all calls on a device use the same static arrays, which keep the
// contents of the previous call.  Nothing in them needs to start at zero (each
// call overwrites what it later reads), but two calls that overlap on the GPU
// -- issued to different streams without ordering between them -- race on the
// scratch and give wrong results.  Order them on one stream or with events.
//
// `in` and `out` are device pointers to n0*n1*n2 complex64 values, 16-byte
// aligned; the two ranges must not overlap, not even partially.  `stream` is a cudaStream_t (0 for the default
// stream).  Returns 0 on success.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define JDB_STATIC_MAX_ELEMS 262144

__attribute__((visibility("default"))) int jdb_fft3d_c64_static(const void* in, void* out, int n0, int n1, int n2,
                                                                int inverse, void* stream);
__attribute__((visibility("default"))) const char* jdb_fft3d_c64_static_error(void);

#ifdef __cplusplus
}
#endif
