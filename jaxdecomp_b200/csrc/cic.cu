// Cloud-in-cell particle-mesh kernels: paint (scatter-add with trilinear
// weights), read-out (the adjoint gather) and the gradient of paint with
// respect to the particle positions.  They replace the XLA scatter of the
// reference's example (examples/scatter.py:59-153: `enmesh` builds the eight
// neighbour indices and weights, `_scatter_chunk` does mesh.at[ind].add).
//
// Positions are given in cell units relative to the origin of the local
// (padded) mesh block of shape (S0, S1, S2).  Along an axis with wrap == 1 the
// neighbour index is taken modulo the extent (periodic local axis, e.g. the
// unsharded third axis); with wrap == 0 contributions that fall outside the
// block are dropped.  In "grid mode" (g0 > 0) particle i starts at lattice site
// (i / (g1*g2) + o0, (i / g2) % g1 + o1, i % g2 + o2) and `pos` holds its
// displacement, which avoids materialising the lattice.
#include <cuda_runtime.h>

#include <cstdlib>

#include "launch.h"

namespace jdb {

struct CicGeom {
  int S0, S1, S2;
  int wrap0, wrap1, wrap2;
  int g0, g1, g2;      // lattice of initial positions (grid mode) or 0
  float o0, o1, o2;    // offset of the lattice inside the block
  long long pi, pd;    // element strides of `pos` between particles and between the three components:
                       // (3, 1) for an [n, 3] array, (1, n) for three planes [3, n]
};

__device__ __forceinline__ void particle_pos(const CicGeom& g, const float* __restrict__ pos, long long i, float& x, float& y,
                                             float& z) {
  x = pos[g.pi * i];
  y = pos[g.pi * i + g.pd];
  z = pos[g.pi * i + 2 * g.pd];
  if (g.g0 > 0) {
    const long long plane = (long long)g.g1 * g.g2;
    const int a = (int)(i / plane);
    const long long r = i - a * plane;
    const int b = (int)(r / g.g2);
    const int c = (int)(r - (long long)b * g.g2);
    x += (float)a + g.o0;
    y += (float)b + g.o1;
    z += (float)c + g.o2;
  }
}

__device__ __forceinline__ bool cell_index(int i, int S, int wrap, int& out) {
  if (wrap) {
    i %= S;
    if (i < 0) i += S;
    out = i;
    return true;
  }
  out = i;
  return i >= 0 && i < S;
}

__global__ void cic_paint_kernel(CicGeom g, const float* __restrict__ pos, const float* __restrict__ weight, float wscalar,
                                 long long n, float* __restrict__ mesh) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float x, y, z;
    particle_pos(g, pos, i, x, y, z);
    const float w = weight ? weight[i] : wscalar;
    const float fx = floorf(x), fy = floorf(y), fz = floorf(z);
    const int ix = (int)fx, iy = (int)fy, iz = (int)fz;
    const float dx = x - fx, dy = y - fy, dz = z - fz;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int bx = c & 1, by = (c >> 1) & 1, bz = (c >> 2) & 1;
      int jx, jy, jz;
      if (!cell_index(ix + bx, g.S0, g.wrap0, jx)) continue;
      if (!cell_index(iy + by, g.S1, g.wrap1, jy)) continue;
      if (!cell_index(iz + bz, g.S2, g.wrap2, jz)) continue;
      const float f = (bx ? dx : 1.f - dx) * (by ? dy : 1.f - dy) * (bz ? dz : 1.f - dz);
      atomicAdd(mesh + ((long long)jx * g.S1 + jy) * g.S2 + jz, w * f);
    }
  }
}

// Tiled paint for particles that start on a lattice (grid mode).  A block owns a BX x BY x BZ brick of
// lattice sites and accumulates their contributions in a shared-memory copy of the mesh cells around
// that brick (the brick plus an apron of A cells below and A + 1 above on every axis); the few
// contributions that a large displacement carries beyond the apron go to global memory directly.  At
// the end the block adds every non-zero cell of its copy to the mesh with one reduction per cell.
// Particles of neighbouring sites mostly hit the same cells, so most of the eight adds per particle
// stay on chip, and what reaches L2 is one pass over the block's cells in rows along the last axis.
template <int BX, int BY, int BZ, int A>
struct CicTile {
  static constexpr int SX = BX + 2 * A + 1, SY = BY + 2 * A + 1, SZ = BZ + 2 * A + 1;
  static constexpr int CELLS = SX * SY * SZ;
  static constexpr int SITES = BX * BY * BZ;
};

template <int BX, int BY, int BZ, int A>
__global__ void __launch_bounds__(256) cic_paint_tiled_kernel(CicGeom g, const float* __restrict__ pos,
                                                              const float* __restrict__ weight, float wscalar,
                                                              float* __restrict__ mesh) {
  using T = CicTile<BX, BY, BZ, A>;
  extern __shared__ float cic_tile[];
  for (int e = threadIdx.x; e < T::CELLS; e += blockDim.x) cic_tile[e] = 0.f;
  const int tz = g.g2 / BZ, ty = g.g1 / BY;
  const int bz = blockIdx.x % tz, by = (blockIdx.x / tz) % ty, bx = blockIdx.x / (tz * ty);
  const int a0 = bx * BX, b0 = by * BY, c0 = bz * BZ;
  // mesh cell of the tile's first shared cell
  const int ox = a0 + (int)floorf(g.o0) - A, oy = b0 + (int)floorf(g.o1) - A, oz = c0 + (int)floorf(g.o2) - A;
  __syncthreads();
  for (int p = threadIdx.x; p < T::SITES; p += blockDim.x) {
    const int c = p % BZ, b = (p / BZ) % BY, a = p / (BZ * BY);
    const long long i = ((long long)(a0 + a) * g.g1 + (b0 + b)) * g.g2 + (c0 + c);
    const float x = pos[g.pi * i] + (float)(a0 + a) + g.o0;
    const float y = pos[g.pi * i + g.pd] + (float)(b0 + b) + g.o1;
    const float z = pos[g.pi * i + 2 * g.pd] + (float)(c0 + c) + g.o2;
    const float w = weight ? weight[i] : wscalar;
    const float fx = floorf(x), fy = floorf(y), fz = floorf(z);
    const int ix = (int)fx, iy = (int)fy, iz = (int)fz;
    const float dx = x - fx, dy = y - fy, dz = z - fz;
    const int lx = ix - ox, ly = iy - oy, lz = iz - oz;
    const bool inside = lx >= 0 && lx + 1 < T::SX && ly >= 0 && ly + 1 < T::SY && lz >= 0 && lz + 1 < T::SZ;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int kx = k & 1, ky = (k >> 1) & 1, kz = (k >> 2) & 1;
      const float f = w * (kx ? dx : 1.f - dx) * (ky ? dy : 1.f - dy) * (kz ? dz : 1.f - dz);
      if (inside) {
        atomicAdd(cic_tile + ((lx + kx) * T::SY + (ly + ky)) * T::SZ + (lz + kz), f);
      } else {
        int jx, jy, jz;
        if (!cell_index(ix + kx, g.S0, g.wrap0, jx)) continue;
        if (!cell_index(iy + ky, g.S1, g.wrap1, jy)) continue;
        if (!cell_index(iz + kz, g.S2, g.wrap2, jz)) continue;
        atomicAdd(mesh + ((long long)jx * g.S1 + jy) * g.S2 + jz, f);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < T::CELLS; e += blockDim.x) {
    const float v = cic_tile[e];
    if (v == 0.f) continue;
    const int lz = e % T::SZ, ly = (e / T::SZ) % T::SY, lx = e / (T::SZ * T::SY);
    int jx, jy, jz;
    if (!cell_index(ox + lx, g.S0, g.wrap0, jx)) continue;
    if (!cell_index(oy + ly, g.S1, g.wrap1, jy)) continue;
    if (!cell_index(oz + lz, g.S2, g.wrap2, jz)) continue;
    atomicAdd(mesh + ((long long)jx * g.S1 + jy) * g.S2 + jz, v);
  }
}

__global__ void cic_readout_kernel(CicGeom g, const float* __restrict__ pos, long long n, const float* __restrict__ mesh,
                                   float* __restrict__ out) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float x, y, z;
    particle_pos(g, pos, i, x, y, z);
    const float fx = floorf(x), fy = floorf(y), fz = floorf(z);
    const int ix = (int)fx, iy = (int)fy, iz = (int)fz;
    const float dx = x - fx, dy = y - fy, dz = z - fz;
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int bx = c & 1, by = (c >> 1) & 1, bz = (c >> 2) & 1;
      int jx, jy, jz;
      if (!cell_index(ix + bx, g.S0, g.wrap0, jx)) continue;
      if (!cell_index(iy + by, g.S1, g.wrap1, jy)) continue;
      if (!cell_index(iz + bz, g.S2, g.wrap2, jz)) continue;
      const float f = (bx ? dx : 1.f - dx) * (by ? dy : 1.f - dy) * (bz ? dz : 1.f - dz);
      acc += f * mesh[((long long)jx * g.S1 + jy) * g.S2 + jz];
    }
    out[i] = acc;
  }
}

// d/dpos of sum_cells gmesh[cell] * w * f(cell; pos): per axis the derivative of
// the hat function is +-1 times the weights of the other two axes.
__global__ void cic_paint_grad_pos_kernel(CicGeom g, const float* __restrict__ pos, const float* __restrict__ weight,
                                          float wscalar, long long n, const float* __restrict__ gmesh,
                                          float* __restrict__ gpos) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float x, y, z;
    particle_pos(g, pos, i, x, y, z);
    const float w = weight ? weight[i] : wscalar;
    const float fx = floorf(x), fy = floorf(y), fz = floorf(z);
    const int ix = (int)fx, iy = (int)fy, iz = (int)fz;
    const float dx = x - fx, dy = y - fy, dz = z - fz;
    float gx = 0.f, gy = 0.f, gz = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int bx = c & 1, by = (c >> 1) & 1, bz = (c >> 2) & 1;
      int jx, jy, jz;
      if (!cell_index(ix + bx, g.S0, g.wrap0, jx)) continue;
      if (!cell_index(iy + by, g.S1, g.wrap1, jy)) continue;
      if (!cell_index(iz + bz, g.S2, g.wrap2, jz)) continue;
      const float v = gmesh[((long long)jx * g.S1 + jy) * g.S2 + jz] * w;
      const float wx = bx ? dx : 1.f - dx, wy = by ? dy : 1.f - dy, wz = bz ? dz : 1.f - dz;
      gx += v * (bx ? 1.f : -1.f) * wy * wz;
      gy += v * wx * (by ? 1.f : -1.f) * wz;
      gz += v * wx * wy * (bz ? 1.f : -1.f);
    }
    gpos[g.pi * i] = gx;
    gpos[g.pi * i + g.pd] = gy;
    gpos[g.pi * i + 2 * g.pd] = gz;
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

static int grid_for(long long n) {
  long long g = (n + 255) / 256;
  if (g < 1) g = 1;
  if (g > 148LL * 32) g = 148LL * 32;
  return (int)g;
}

static CicGeom geom(const CicArgs& a) {
  CicGeom g;
  g.S0 = a.S0; g.S1 = a.S1; g.S2 = a.S2;
  g.wrap0 = a.wrap0; g.wrap1 = a.wrap1; g.wrap2 = a.wrap2;
  g.g0 = a.g0; g.g1 = a.g1; g.g2 = a.g2;
  g.o0 = a.o0; g.o1 = a.o1; g.o2 = a.o2;
  g.pi = a.planar ? 1 : 3;
  g.pd = a.planar ? a.n : 1;
  return g;
}

static bool valid(const CicArgs& a) {
  if (a.S0 < 1 || a.S1 < 1 || a.S2 < 1 || a.n < 0) return false;
  if (a.g0 > 0 && (long long)a.g0 * a.g1 * a.g2 != a.n) return false;
  return true;
}

// Which paint kernel: the tiled one needs lattice mode and a lattice that splits into whole bricks.
// JD_B200_CIC_TILED=0/1 forces the choice (default: tiled whenever it applies).
static bool use_tiled_paint(const CicArgs& a, int bx, int by, int bz) {
  if (a.g0 <= 0 || a.g0 % bx || a.g1 % by || a.g2 % bz) return false;
  if ((long long)(a.g0 / bx) * (a.g1 / by) * (a.g2 / bz) > 2147483647LL) return false;
  const char* env = std::getenv("JD_B200_CIC_TILED");
  if (env && *env) return env[0] != '0';
  return true;
}

int launch_cic_paint(const CicArgs& a, const float* pos, const float* weight, float* mesh, void* stream) {
  if (!valid(a) || !pos || !mesh) return JD_ERR_INVALID_ARG;
  if (a.n == 0) return JD_OK;
  constexpr int BX = 8, BY = 8, BZ = 32, AP = 3;
  if (use_tiled_paint(a, BX, BY, BZ)) {
    using T = CicTile<BX, BY, BZ, AP>;
    auto kern = cic_paint_tiled_kernel<BX, BY, BZ, AP>;
    const int smem = T::CELLS * (int)sizeof(float);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) {
        set_last_error(cudaGetErrorString(e));
        return JD_ERR_CUDA;
      }
      configured = true;
    }
    const unsigned blocks = (unsigned)((a.g0 / BX) * (a.g1 / BY) * (a.g2 / BZ));
    kern<<<blocks, 256, smem, (cudaStream_t)stream>>>(geom(a), pos, weight, a.wscalar, mesh);
    return check_launch();
  }
  cic_paint_kernel<<<grid_for(a.n), 256, 0, (cudaStream_t)stream>>>(geom(a), pos, weight, a.wscalar, a.n, mesh);
  return check_launch();
}

int launch_cic_readout(const CicArgs& a, const float* pos, const float* mesh, float* out, void* stream) {
  if (!valid(a) || !pos || !mesh || !out) return JD_ERR_INVALID_ARG;
  if (a.n == 0) return JD_OK;
  cic_readout_kernel<<<grid_for(a.n), 256, 0, (cudaStream_t)stream>>>(geom(a), pos, a.n, mesh, out);
  return check_launch();
}

int launch_cic_paint_grad_pos(const CicArgs& a, const float* pos, const float* weight, const float* gmesh, float* gpos,
                              void* stream) {
  if (!valid(a) || !pos || !gmesh || !gpos) return JD_ERR_INVALID_ARG;
  if (a.n == 0) return JD_OK;
  cic_paint_grad_pos_kernel<<<grid_for(a.n), 256, 0, (cudaStream_t)stream>>>(geom(a), pos, weight, a.wscalar, a.n, gmesh,
                                                                              gpos);
  return check_launch();
}

}  // namespace jdb
