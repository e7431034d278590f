// Pointwise Fourier-space kernels on the rotated output layout of pfft3d.
// They replace the XLA-fused expressions of the reference's LPT example
// (examples/lpt_nbody_demo.py:75-133): scaling the modes of a white-noise
// field by sqrt(P(k)) and forming the three displacement fields i k_d / k^2.
//
// The local block has dims (L0, L1, L2) holding the original axes (1, 2, 0);
// off* are the global indices of its first element, N* the global extents of
// the original axes 0, 1, 2, and box* the physical box lengths, so that the
// physical wave number along original axis d is 2*pi*fftfreq(N_d)[idx]*N_d/box_d.
//
// mode 0: out0 = in * sqrt(A * k^n * exp(-(k/kcut)^2) * norm)     (k == 0 -> 0)
// mode 1: out0 = in * sqrt(table(k) * norm), table = P sampled at log-spaced k (linear interpolation in log k)
// mode 2: out_d = in * i * k_d / k^2 for d = 0, 1, 2              (k == 0 -> 0)
// mode 3: out0 = in * (-1 / k^2)                                   (k == 0 -> 0)  inverse Laplacian
// mode 4: out0 = sum_d conj(i k_d / k^2) * in_d, with in_0 = in, in_1 = out1, in_2 = out2 (read-only):
//         the adjoint of mode 2, used by its gradient
#include <cuda_runtime.h>

#include "launch.h"

namespace jdb {

__device__ __forceinline__ float wavenumber(int idx, int N, float box) {
  const int f = idx < (N + 1) / 2 ? idx : idx - N;
  return 6.28318530717958647692f * (float)f / box;
}

__device__ __forceinline__ float table_lookup(const float* __restrict__ tab, int n, float lk0, float dlk, float k) {
  if (k <= 0.f) return 0.f;
  float u = (logf(k) - lk0) / dlk;
  if (u <= 0.f) return tab[0];
  if (u >= (float)(n - 1)) return tab[n - 1];
  const int i = (int)u;
  const float t = u - (float)i;
  return tab[i] * (1.f - t) + tab[i + 1] * t;
}

__global__ void kspace_kernel(KSpaceDesc d, const float2* __restrict__ in, float2* __restrict__ out0, float2* __restrict__ out1,
                              float2* __restrict__ out2, const float* __restrict__ table) {
  const long long total = (long long)d.L0 * d.L1 * d.L2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int i2 = (int)(i % d.L2);
    const long long r = i / d.L2;
    const int i1 = (int)(r % d.L1);
    const int i0 = (int)(r / d.L1);
    // local dims hold original axes (1, 2, 0)
    const float k1 = wavenumber(d.off0 + i0, d.N1, d.box1);
    const float k2 = wavenumber(d.off1 + i1, d.N2, d.box2);
    const float k0 = wavenumber(d.off2 + i2, d.N0, d.box0);
    const float kk = k0 * k0 + k1 * k1 + k2 * k2;
    const float2 v = in[i];
    if (d.mode == 0 || d.mode == 1) {
      float p = 0.f;
      if (kk > 0.f) {
        const float k = sqrtf(kk);
        if (d.mode == 0) {
          const float c = k / d.p2;
          p = d.p0 * powf(k, d.p1) * expf(-c * c);
        } else {
          p = table_lookup(table, d.ntable, d.p0, d.p1, k);
        }
      }
      const float s = sqrtf(fmaxf(p * d.p3, 0.f));
      out0[i] = make_float2(v.x * s, v.y * s);
    } else if (d.mode == 2) {
      const float inv = kk > 0.f ? 1.f / kk : 0.f;
      // i * k_d / k^2 * (x + i y) = (-y + i x) * k_d / k^2
      const float a0 = k0 * inv, a1 = k1 * inv, a2 = k2 * inv;
      out0[i] = make_float2(-v.y * a0, v.x * a0);
      out1[i] = make_float2(-v.y * a1, v.x * a1);
      out2[i] = make_float2(-v.y * a2, v.x * a2);
    } else if (d.mode == 3) {
      const float s = kk > 0.f ? -1.f / kk : 0.f;
      out0[i] = make_float2(v.x * s, v.y * s);
    } else {
      const float inv = kk > 0.f ? 1.f / kk : 0.f;
      const float2 v1 = out1[i], v2 = out2[i];
      // -i * a * (x + i y) = a * (y - i x)
      const float a0 = k0 * inv, a1 = k1 * inv, a2 = k2 * inv;
      out0[i] = make_float2(a0 * v.y + a1 * v1.y + a2 * v2.y, -(a0 * v.x + a1 * v1.x + a2 * v2.x));
    }
  }
}

int launch_kspace(const KSpaceDesc& d, const void* in, void* out0, void* out1, void* out2, const float* table,
                  void* stream) {
  if (d.L0 < 1 || d.L1 < 1 || d.L2 < 1 || d.mode < 0 || d.mode > 4 || !in || !out0) return JD_ERR_INVALID_ARG;
  if ((d.mode == 2 || d.mode == 4) && (!out1 || !out2)) return JD_ERR_INVALID_ARG;
  if (d.mode == 1 && (!table || d.ntable < 2)) return JD_ERR_INVALID_ARG;
  const long long total = (long long)d.L0 * d.L1 * d.L2;
  long long g = (total + 255) / 256;
  if (g > 148LL * 32) g = 148LL * 32;
  kspace_kernel<<<(int)g, 256, 0, (cudaStream_t)stream>>>(d, (const float2*)in, (float2*)out0, (float2*)out1,
                                                           (float2*)out2, table);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return JD_ERR_CUDA;
  }
  return JD_OK;
}

}  // namespace jdb
