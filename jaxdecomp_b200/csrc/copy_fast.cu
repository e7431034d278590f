// Rotating copy pass (a pencil transpose without a transform) for 8- and 16-byte elements.
//
// The general tile pass (fft_pass.cu) moves a copy tile with per-element index arithmetic and is bound by
// its instruction count (3.4 TB/s read + write on a 1024^3 complex64 rotation).  This kernel covers the
// common case -- rows contiguous along c on the way in, runs contiguous along t on the way out, extents
// that are multiples of the tile -- with 16-byte accesses on both sides of a shared-memory tile and no
// bank conflicts:
//
//   8-byte elements  : a 64 (c) x 64 (t) tile.  A thread loads the 2 x 2 block (t, t+1) x (c, c+1) as two
//                      16-byte vectors, re-pairs it in registers into (t, t+1) for column c and for column
//                      c+1, and writes those as 16-byte units of a [c][t/2] array whose unit index is
//                      XOR-swizzled with (c/2) mod 8.  A warp then reads one column -- 32 consecutive
//                      units -- and stores a 512-byte run.
//   16-byte elements : a 32 (c) x 32 (t) tile of a [t][c] array with an odd pitch (33 units).
//
// Destination addressing (peer of a column or of the tile's rows, offsets inside the peer's buffer) is
// that of tile_store in tile_ops.h; the stores go through store_pair / store_elem, so the checked build
// covers them, and the same bits arrive as with the general kernel.  Stores may cross NVLink (plain peer
// stores); loads never do.
#include <cuda_runtime.h>

#include "launch.h"
#include "tile_ops.h"

namespace jdb {

namespace {

constexpr int kThreads = 256;

struct TileCoord {
  int c0, t0, o, b;
};

template <int TC, int TT>
__device__ __forceinline__ TileCoord tile_of_block(const PassDesc& d) {
  const int tiles_c = d.C / TC, tiles_t = d.Tn / TT;
  long long bid = blockIdx.x;
  TileCoord tc;
  tc.c0 = (int)(bid % tiles_c) * TC;
  bid /= tiles_c;
  tc.t0 = (int)(bid % tiles_t) * TT;
  tc.o = (int)(bid / tiles_t);
  tc.b = blockIdx.y;
  return tc;
}

__global__ void __launch_bounds__(kThreads, 4) copy_rotate8_kernel(const __grid_constant__ PassDesc d) {
  using E = cx<float>;  // stands for any 8-byte element: the bits are only moved
  constexpr int TC = 64, TT = 64, UNITS = TT / 2;
  __shared__ __align__(16) float4 sm[TC * UNITS];
  if (pass_aborted(d)) return;
  const TileCoord tc = tile_of_block<TC, TT>(d);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  const E* in = (const E*)d.in + ((long long)tc.o * d.is_o + (long long)tc.b * d.is_b + (long long)tc.t0 * d.is_t +
                                  tc.c0 + 2 * lane);
  float4 r[4][2];
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const E* p = in + (long long)(2 * (it * 8 + warp)) * d.is_t;
    r[it][0] = *reinterpret_cast<const float4*>(p);           // (t, c), (t, c + 1)
    r[it][1] = *reinterpret_cast<const float4*>(p + d.is_t);  // (t + 1, c), (t + 1, c + 1)
  }
  const int sw_w = lane & 7;  // ((2 * lane) / 2) mod 8, the same for columns 2 * lane and 2 * lane + 1
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int tp = it * 8 + warp;
    sm[(2 * lane) * UNITS + (tp ^ sw_w)] = make_float4(r[it][0].x, r[it][0].y, r[it][1].x, r[it][1].y);
    sm[(2 * lane + 1) * UNITS + (tp ^ sw_w)] = make_float4(r[it][0].z, r[it][0].w, r[it][1].z, r[it][1].w);
  }
  __syncthreads();

  const OutBase ob = out_base_for(d, tc.o, tc.b);
  const int pt = d.split_axis == 2 ? tc.t0 / d.Tl : 0;  // Tl is a multiple of the tile: one peer per tile
  const long long toff = ob.off + (long long)(tc.t0 - pt * d.Tl + 2 * lane);  // os_t == 1
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int c = it * 8 + warp;
    const float4 v = sm[c * UNITS + (lane ^ ((c >> 1) & 7))];
    const int gc = tc.c0 + c;
    const int pc = d.split_axis == 1 ? gc / d.Cl : 0;
    pair_of<E> p;
    p.a = E{v.x, v.y};
    p.b = E{v.z, v.w};
    store_pair<E>(d, ob.peer + pc + pt, toff + (long long)(gc - pc * d.Cl) * d.os_c, p);
  }
}

__global__ void __launch_bounds__(kThreads, 4) copy_rotate16_kernel(const __grid_constant__ PassDesc d) {
  using E = cx<double>;  // any 16-byte element
  constexpr int TC = 32, TT = 32, PITCH = TC + 1;
  __shared__ __align__(16) double2 sm[TT * PITCH];
  if (pass_aborted(d)) return;
  const TileCoord tc = tile_of_block<TC, TT>(d);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  const E* in = (const E*)d.in + ((long long)tc.o * d.is_o + (long long)tc.b * d.is_b + (long long)tc.t0 * d.is_t +
                                  tc.c0 + lane);
  double2 r[4];
#pragma unroll
  for (int it = 0; it < 4; ++it) r[it] = *reinterpret_cast<const double2*>(in + (long long)(it * 8 + warp) * d.is_t);
#pragma unroll
  for (int it = 0; it < 4; ++it) sm[(it * 8 + warp) * PITCH + lane] = r[it];
  __syncthreads();

  const OutBase ob = out_base_for(d, tc.o, tc.b);
  const int pt = d.split_axis == 2 ? tc.t0 / d.Tl : 0;
  const long long toff = ob.off + (long long)(tc.t0 - pt * d.Tl + lane);
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int c = it * 8 + warp;
    const double2 v = sm[lane * PITCH + c];
    const int gc = tc.c0 + c;
    const int pc = d.split_axis == 1 ? gc / d.Cl : 0;
    store_elem<E>(d, ob.peer + pc + pt, toff + (long long)(gc - pc * d.Cl) * d.os_c, E{v.x, v.y});
  }
}

bool even(long long v) { return (v & 1) == 0; }

}  // namespace

bool copy_fast_eligible(const PassDesc& d) {
  if (d.fft_mode != JD_COPY || d.mul_mode != JD_MUL_NONE) return false;
  if (d.elem_bytes != 8 && d.elem_bytes != 16) return false;
  if (d.is_c != 1 || d.os_t != 1 || !d.store_t_contig || d.load_t_contig) return false;
  if (d.grid_limit > 0) return false;  // no looping variant: copy passes are not pipelined
  const int tc = d.elem_bytes == 8 ? 64 : 32, tt = tc;
  if (d.C % tc || d.Tn % tt) return false;
  if (d.split_axis == 2 && d.Tl % tt) return false;
  if (d.split_axis == 1 && (d.Cl < 1 || d.C % d.Cl)) return false;
  if (d.elem_bytes == 8) {
    // 16-byte accesses: every row start and every stored run must sit on a 16-byte boundary
    if (!even(d.is_t) || !even(d.is_o) || !even(d.is_b)) return false;
    if (!even(d.os_c) || !even(d.os_o) || !even(d.os_b) || !even(d.out_base)) return false;
    if (((uintptr_t)d.in) % 16) return false;
    for (int p = 0; p < d.npeers; ++p)
      if (((uintptr_t)d.out[p]) % 16) return false;
  }
  return true;
}

int launch_copy_fast(const PassDesc& d, void* stream) {
  const int tc = d.elem_bytes == 8 ? 64 : 32;
  const long long nblocks = (long long)(d.C / tc) * (d.Tn / tc) * d.On;
  if (nblocks > 2147483647LL || d.B > 65535) {
    set_last_error("copy pass: grid too large");
    return JD_ERR_INVALID_ARG;
  }
  const dim3 grid((unsigned)nblocks, (unsigned)d.B, 1);
  if (d.elem_bytes == 8)
    copy_rotate8_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(d);
  else
    copy_rotate16_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(d);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return JD_ERR_CUDA;
  }
  return JD_OK;
}

}  // namespace jdb
