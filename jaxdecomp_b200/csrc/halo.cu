// Halo exchange kernels: one launch pushes all (up to eight) face and corner
// slabs of a padded block to the ranks that need them, with plain peer stores
// over NVLink, reading the slabs in place (no local pack buffer).  Corners go
// straight to the diagonal neighbour -- every peer is one NVSwitch hop away --
// instead of the two chained permutes of the reference
// (src/jaxdecomp/_src/jax/halo.py:160-184); the reference's native backend does
// three sequential cudecompUpdateHalosX calls (src/csrc/halo.cu:45-73).
//
// pack   : src[region r]  ->  stage[peer_r] + off_r      (peer stores)
// unpack : dst[region r]  =   stage[me] + off_r          (local loads; or zero fill)
//          dst[region r] +=   stage[me] + off_r          (accumulate variant, one
//                                                         region per launch in a fixed
//                                                         order: deterministic sums)
// A region is [lo0,hi0) x [lo1,hi1) x [0,S2) of every batch entry; its slab in
// the staging buffer is dense in (batch, rows, cols, S2) order.  The eight
// receive regions are disjoint, so one launch can fill them all.
#include <cuda_runtime.h>

#include "launch.h"

namespace jdb {

struct RegionIndex {
  long long start[9];  // prefix sums of the per-region vector counts
};

template <typename V>
__global__ void halo_pack_kernel(HaloDesc d, RegionIndex ri, int vec_per_row) {
  const long long total = ri.start[d.nregions];
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int r = 0;
    while (i >= ri.start[r + 1]) ++r;
    const HaloRegion& g = d.reg[r];
    if (g.peer < 0) continue;
    long long k = i - ri.start[r];
    const int n0 = g.hi0 - g.lo0, n1 = g.hi1 - g.lo1;
    const int v = (int)(k % vec_per_row);
    k /= vec_per_row;
    const int j = (int)(k % n1);
    k /= n1;
    const int a = (int)(k % n0);
    const int b = (int)(k / n0);
    const long long src_idx = (((long long)b * d.S0 + (g.lo0 + a)) * d.S1 + (g.lo1 + j)) * vec_per_row + v;
    const V* src = (const V*)d.src;
    if (d.direct) {
      // final position in the neighbour's block: no staging slab, no unpack
      const long long dst_idx = (((long long)b * d.S0 + (g.dlo0 + a)) * d.S1 + (g.dlo1 + j)) * vec_per_row + v;
      ((V*)d.stage[g.peer])[dst_idx] = src[src_idx];
    } else {
      V* dst = (V*)d.stage[g.peer] + g.stage_off;
      dst[i - ri.start[r]] = src[src_idx];
    }
  }
}

__device__ __forceinline__ float4 vadd(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float vadd(float a, float b) { return a + b; }
__device__ __forceinline__ double vadd(double a, double b) { return a + b; }
__device__ __forceinline__ double2 vadd(double2 a, double2 b) { return make_double2(a.x + b.x, a.y + b.y); }

// mode 0: overwrite from staging (peer >= 0) or zero (peer < 0); mode 1: add from staging
template <typename V>
__global__ void halo_unpack_kernel(HaloDesc d, RegionIndex ri, int vec_per_row, int first, int count) {
  const long long base = ri.start[first];
  const long long total = ri.start[first + count] - base;
  for (long long ii = blockIdx.x * (long long)blockDim.x + threadIdx.x; ii < total;
       ii += (long long)gridDim.x * blockDim.x) {
    const long long i = ii + base;
    int r = first;
    while (i >= ri.start[r + 1]) ++r;
    const HaloRegion& g = d.reg[r];
    long long k = i - ri.start[r];
    const int n0 = g.hi0 - g.lo0, n1 = g.hi1 - g.lo1;
    const int v = (int)(k % vec_per_row);
    k /= vec_per_row;
    const int j = (int)(k % n1);
    k /= n1;
    const int a = (int)(k % n0);
    const int b = (int)(k / n0);
    const long long dst_idx = (((long long)b * d.S0 + (g.lo0 + a)) * d.S1 + (g.lo1 + j)) * vec_per_row + v;
    V* dst = (V*)d.dst;
    if (d.accumulate) {
      if (g.peer < 0) continue;
      const V* st = (const V*)d.stage[g.peer] + g.stage_off;
      dst[dst_idx] = vadd(dst[dst_idx], st[i - ri.start[r]]);
    } else if (g.peer < 0) {
      V z;
      memset(&z, 0, sizeof(V));
      dst[dst_idx] = z;
    } else {
      const V* st = (const V*)d.stage[g.peer] + g.stage_off;
      dst[dst_idx] = st[i - ri.start[r]];
    }
  }
}

static int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return JD_ERR_CUDA;
  }
  return JD_OK;
}

// Data is moved in "units": 16-byte vectors when the row length and every
// address allow it, else 4-byte words (8-byte for float64 arithmetic).
static bool wide_ok(const HaloDesc& d) {
  const long long row_bytes = (long long)d.S2 * d.elem_bytes;
  if (row_bytes % 16) return false;
  if (((uintptr_t)d.src | (uintptr_t)d.dst) % 16) return false;
  for (int r = 0; r < d.nregions; ++r) {
    if (((long long)d.reg[r].stage_off * d.elem_bytes) % 16) return false;
    if (d.reg[r].peer >= 0 && ((uintptr_t)d.stage[d.reg[r].peer]) % 16) return false;
  }
  return true;
}

static RegionIndex make_index(const HaloDesc& d, int units_per_row) {
  RegionIndex ri;
  ri.start[0] = 0;
  for (int r = 0; r < 8; ++r) {
    long long n = 0;
    if (r < d.nregions)
      n = (long long)d.B * (d.reg[r].hi0 - d.reg[r].lo0) * (d.reg[r].hi1 - d.reg[r].lo1) * units_per_row;
    ri.start[r + 1] = ri.start[r] + n;
  }
  return ri;
}

static int grid_for(long long total) {
  long long g = (total + 255) / 256;
  if (g < 1) g = 1;
  if (g > 148 * 16) g = 148 * 16;
  return (int)g;
}

// Rescale the element offsets of the staging slabs to units of `unit` bytes.
static int to_units(HaloDesc& d, int unit) {
  for (int r = 0; r < d.nregions; ++r) d.reg[r].stage_off = d.reg[r].stage_off * d.elem_bytes / unit;
  return (int)((long long)d.S2 * d.elem_bytes / unit);
}

static bool valid(const HaloDesc& d) {
  if (d.nregions < 0 || d.nregions > 8) return false;
  if (d.elem_bytes != 4 && d.elem_bytes != 8 && d.elem_bytes != 16) return false;
  for (int r = 0; r < d.nregions; ++r) {
    const HaloRegion& g = d.reg[r];
    if (g.lo0 < 0 || g.hi0 > d.S0 || g.lo1 < 0 || g.hi1 > d.S1 || g.lo0 > g.hi0 || g.lo1 > g.hi1) return false;
    if (g.peer >= JD_MAX_PEERS) return false;
    if (d.direct && (g.dlo0 < 0 || g.dlo0 + (g.hi0 - g.lo0) > d.S0 || g.dlo1 < 0 || g.dlo1 + (g.hi1 - g.lo1) > d.S1))
      return false;
  }
  return true;
}

int launch_halo_pack(const HaloDesc& d0, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  HaloDesc d = d0;
  if (!valid(d)) return JD_ERR_INVALID_ARG;
  if (d.nregions == 0) return JD_OK;
  if (wide_ok(d)) {
    const int upr = to_units(d, 16);
    RegionIndex ri = make_index(d, upr);
    if (ri.start[d.nregions] == 0) return JD_OK;
    halo_pack_kernel<float4><<<grid_for(ri.start[d.nregions]), 256, 0, stream>>>(d, ri, upr);
  } else {
    const int upr = to_units(d, 4);
    RegionIndex ri = make_index(d, upr);
    if (ri.start[d.nregions] == 0) return JD_OK;
    halo_pack_kernel<float><<<grid_for(ri.start[d.nregions]), 256, 0, stream>>>(d, ri, upr);
  }
  return check_launch();
}

template <typename V>
static int unpack_t(const HaloDesc& d, const RegionIndex& ri, int upr, cudaStream_t stream) {
  if (!d.accumulate) {
    const long long total = ri.start[d.nregions];
    if (total == 0) return JD_OK;
    halo_unpack_kernel<V><<<grid_for(total), 256, 0, stream>>>(d, ri, upr, 0, d.nregions);
    return check_launch();
  }
  for (int r = 0; r < d.nregions; ++r) {  // targets may overlap: one region at a time, fixed order
    const long long total = ri.start[r + 1] - ri.start[r];
    if (total == 0 || d.reg[r].peer < 0) continue;
    halo_unpack_kernel<V><<<grid_for(total), 256, 0, stream>>>(d, ri, upr, r, 1);
    int rc = check_launch();
    if (rc != JD_OK) return rc;
  }
  return JD_OK;
}

int launch_halo_unpack(const HaloDesc& d0, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  HaloDesc d = d0;
  if (!valid(d)) return JD_ERR_INVALID_ARG;
  if (d.nregions == 0) return JD_OK;
  const bool wide = wide_ok(d);
  if (d.accumulate && d.is_f64) {
    if (wide) {
      const int upr = to_units(d, 16);
      return unpack_t<double2>(d, make_index(d, upr), upr, stream);
    }
    const int upr = to_units(d, 8);
    return unpack_t<double>(d, make_index(d, upr), upr, stream);
  }
  if (wide) {
    const int upr = to_units(d, 16);
    return unpack_t<float4>(d, make_index(d, upr), upr, stream);
  }
  const int upr = to_units(d, 4);
  return unpack_t<float>(d, make_index(d, upr), upr, stream);
}

}  // namespace jdb
