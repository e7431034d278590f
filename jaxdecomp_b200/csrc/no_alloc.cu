// Allocation-free local 3-D FFT (see no_alloc.h for the contract and for who needs it).
//
// The three passes are the same tile passes that pfft3d runs on one GPU
// (transform along the last axis + rotated store, twice, then a plain
// transform in place); only the provenance of the temporary memory differs: a
// file-scope __device__ array instead of the arena, and twiddle tables that a
// small kernel writes into file-scope arrays instead of host-built tables.
#include "no_alloc.h"

#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "launch.h"
#include "tile_ops.h"

namespace {

using jdb::PassDesc;

constexpr int kMaxAxis = 256;
constexpr int kMaxDevices = 64;

// Scratch shared by every call on a device.  In host code these names are only
// handles for cudaGetSymbolAddress; kernels receive the resolved addresses.
static __device__ __align__(256) float2 g_static_scratch[JDB_STATIC_MAX_ELEMS];
static __device__ __align__(256) float2 g_static_twiddle[3][kMaxAxis];

struct DeviceSlots {
  std::atomic<bool> ready{false};
  float2* scratch = nullptr;
  float2* twiddle = nullptr;
};
DeviceSlots g_slots[kMaxDevices];
std::mutex g_setup_mutex;
thread_local char g_error[256] = "";

int fail(const char* msg) {
  std::snprintf(g_error, sizeof(g_error), "%s", msg);
  return 1;
}

__global__ void fill_twiddle_kernel(float2* table, int M) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n < M) {
    double s, c;
    sincospi(-2.0 * (double)n / (double)M, &s, &c);
    table[n] = make_float2((float)c, (float)s);
  }
}

bool pow2_in_range(int n) { return n >= 8 && n <= kMaxAxis && (n & (n - 1)) == 0; }

int ilog2(int n) {
  int l = 0;
  while ((1 << l) < n) ++l;
  return l;
}

// One pass over a dense block (A, B, C): transform along C, then either keep
// the layout (rotate == 0), or write (C, A, B) (rotate == +1, forward
// pipeline), or write (B, C, A) (rotate == -1, inverse pipeline).
PassDesc make_pass(int A, int B, int C, int rotate, const float2* tw, int inverse, double scale) {
  PassDesc d;
  std::memset(&d, 0, sizeof(d));
  d.B = 1;
  d.C = C;
  d.is_c = 1;
  d.os_b = d.is_b = (long long)A * B * C;
  if (rotate >= 0) {  // t = b, o = a
    d.Tn = B; d.On = A;
    d.is_t = C; d.is_o = (long long)B * C;
    if (rotate > 0) { d.os_c = (long long)A * B; d.os_o = B; d.os_t = 1; }
    else { d.os_c = 1; d.os_t = C; d.os_o = (long long)B * C; }
  } else {  // t = a, o = b; output (B, C, A)
    d.Tn = A; d.On = B;
    d.is_t = (long long)B * C; d.is_o = C;
    d.os_o = (long long)C * A; d.os_c = A; d.os_t = 1;
  }
  d.Cl = d.C; d.Tl = d.Tn; d.Ol = d.On;
  d.npeers = 1;
  d.split_axis = 0;
  d.fft_mode = jdb::JD_FFT_POW2;
  d.M = C;
  d.logW = ilog2(C);
  d.inverse = inverse;
  d.scale = scale;
  d.elem_bytes = 8;
  d.load_t_contig = 0;
  d.store_t_contig = rotate != 0;
  int T = 4096 / C;  // at most 512 threads, one round per thread
  if (T > 32) T = 32;
  if (T > d.Tn) T = d.Tn;
  if (T < 1) T = 1;
  d.T = T;
  d.logT = ilog2(T);
  d.Cc = C;
  d.pitch = C + 2;
  d.twiddle = tw;
  return d;
}

}  // namespace

extern "C" const char* jdb_fft3d_c64_static_error(void) { return g_error; }

extern "C" int jdb_fft3d_c64_static(const void* in, void* out, int n0, int n1, int n2, int inverse, void* stream_) {
  g_error[0] = 0;
  if (!in || !out) return fail("jdb_fft3d_c64_static: null pointer");
  if (in == out) return fail("jdb_fft3d_c64_static: in and out must not alias");
  if (((uintptr_t)in | (uintptr_t)out) % 16) return fail("jdb_fft3d_c64_static: pointers must be 16-byte aligned");
  if (!pow2_in_range(n0) || !pow2_in_range(n1) || !pow2_in_range(n2))
    return fail("jdb_fft3d_c64_static: every extent must be a power of two between 8 and 256");
  const long long total = (long long)n0 * n1 * n2;
  if (total > JDB_STATIC_MAX_ELEMS)
    return fail("jdb_fft3d_c64_static: n0*n1*n2 exceeds the static scratch (262144 complex64 values)");
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail("jdb_fft3d_c64_static: no current CUDA device");
  {
    // partially overlapping buffers would let pass 2 or 3 overwrite input that pass 1 has not read yet
    const uintptr_t a = (uintptr_t)in, b = (uintptr_t)out, bytes = (uintptr_t)total * sizeof(float2);
    if (a < b + bytes && b < a + bytes) return fail("jdb_fft3d_c64_static: in and out must not overlap");
  }
  cudaStream_t stream = (cudaStream_t)stream_;
  DeviceSlots& sl = g_slots[dev];
  // Set-up, once per device and with that device current: turn the symbols into device addresses.  The
  // flag is read with acquire and written with release ordering, and the set-up itself runs under a
  // mutex, so two host threads that make their first call at the same time both see complete slots.
  if (!sl.ready.load(std::memory_order_acquire)) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) {
      cudaGetLastError();
      return fail("jdb_fft3d_c64_static: cannot query the stream");
    }
    if (cap != cudaStreamCaptureStatusNone)
      return fail("jdb_fft3d_c64_static: the first call on a device resolves symbol addresses and must be made "
                  "outside of a stream capture");
    std::lock_guard<std::mutex> lk(g_setup_mutex);
    if (!sl.ready.load(std::memory_order_relaxed)) {
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess) return fail(cudaGetErrorString(e));
      sl.scratch = static_cast<float2*>(p);
      e = cudaGetSymbolAddress(&p, g_static_twiddle);
      if (e != cudaSuccess) return fail(cudaGetErrorString(e));
      sl.twiddle = static_cast<float2*>(p);
      sl.ready.store(true, std::memory_order_release);
    }
  }
  // lengths in the order the passes use them
  const int len[3] = {inverse ? n0 : n2, n1, inverse ? n2 : n0};
  for (int i = 0; i < 3; ++i) {
    fill_twiddle_kernel<<<(len[i] + 127) / 128, 128, 0, stream>>>(sl.twiddle + i * kMaxAxis, len[i]);
    if (cudaGetLastError() != cudaSuccess) return fail("jdb_fft3d_c64_static: table kernel launch failed");
  }
  PassDesc p[3];
  if (!inverse) {
    // (n0,n1,n2) -> scratch (n2,n0,n1) -> out (n1,n2,n0) -> in place along n0
    p[0] = make_pass(n0, n1, n2, +1, sl.twiddle + 0 * kMaxAxis, 0, 1.0);
    p[1] = make_pass(n2, n0, n1, +1, sl.twiddle + 1 * kMaxAxis, 0, 1.0);
    p[2] = make_pass(n1, n2, n0, 0, sl.twiddle + 2 * kMaxAxis, 0, 1.0);
  } else {
    // (n1,n2,n0) -> scratch (n2,n0,n1) -> out (n0,n1,n2) -> in place along n2, scaled
    p[0] = make_pass(n1, n2, n0, -1, sl.twiddle + 0 * kMaxAxis, 1, 1.0);
    p[1] = make_pass(n2, n0, n1, -1, sl.twiddle + 1 * kMaxAxis, 1, 1.0);
    p[2] = make_pass(n0, n1, n2, 0, sl.twiddle + 2 * kMaxAxis, 1, 1.0 / (double)total);
  }
  p[0].in = in;          p[0].out[0] = sl.scratch;
  p[1].in = sl.scratch;  p[1].out[0] = out;
  p[2].in = out;         p[2].out[0] = out;
  for (int i = 0; i < 3; ++i) {
    const int rc = jdb::launch_pass(p[i], stream, nullptr);
    if (rc != jdb::JD_OK) {
      std::snprintf(g_error, sizeof(g_error), "jdb_fft3d_c64_static: pass %d failed: %s (%s)", i, jdb::status_name(rc),
                    jdb::last_error_message());
      return 2;
    }
  }
  return 0;
}
