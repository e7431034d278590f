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

#include "launch.h"

namespace jdb {

struct CicGeom {
  int S0, S1, S2;
  int wrap0, wrap1, wrap2;
  int g0, g1, g2;      // lattice of initial positions (grid mode) or 0
  float o0, o1, o2;    // offset of the lattice inside the block
};

__device__ __forceinline__ void particle_pos(const CicGeom& g, const float* __restrict__ pos, long long i, float& x, float& y,
                                             float& z) {
  x = pos[3 * i];
  y = pos[3 * i + 1];
  z = pos[3 * i + 2];
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
    gpos[3 * i] = gx;
    gpos[3 * i + 1] = gy;
    gpos[3 * i + 2] = gz;
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
  return g;
}

static bool valid(const CicArgs& a) {
  if (a.S0 < 1 || a.S1 < 1 || a.S2 < 1 || a.n < 0) return false;
  if (a.g0 > 0 && (long long)a.g0 * a.g1 * a.g2 != a.n) return false;
  return true;
}

int launch_cic_paint(const CicArgs& a, const float* pos, const float* weight, float* mesh, void* stream) {
  if (!valid(a) || !pos || !mesh) return JD_ERR_INVALID_ARG;
  if (a.n == 0) return JD_OK;
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
