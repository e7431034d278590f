// Tile pass for transform lengths that are not powers of two but factor into
// the primes 2, 3, 5, 7, 11, 13 (384, 768, 1000, 1536, ...): a mixed-radix
// Stockham transform on T pencils held in shared memory, with the same
// contract as the other pass kernels (one PassDesc; results scattered with
// plain stores into the buffer of the peer that owns them, all-to-all routing
// and rotation folded into the addresses).
//
//   * the first stage reads its inputs straight from global memory when the
//     transform axis is the contiguous one (coalesced: butterfly bf of a row
//     reads x[bf + q*N/r]), otherwise the tile is staged by tile_load();
//   * stages ping-pong between two shared-memory buffers in the padded row
//     layout of fft_core.h: one block barrier per stage;
//   * a plain pass writes the last stage's outputs straight to global memory
//     (coalesced: y[bf + q*N/r]); a rotating pass leaves them in shared memory
//     and stores them transposed with tile_store() (16-byte pieces along the
//     destination's fastest axis).
//
// Lengths with larger prime factors keep using Bluestein's algorithm in the
// general kernel.  The reference hands all lengths to cuFFT
// (src/csrc/fft.cu:72-121).
#include <cuda_runtime.h>

#include <cstdlib>

#include "fft_mixed.h"
#include "launch.h"
#include "tile_ops.h"

namespace jdb {

template <typename R, bool SG, bool DG>
struct DevStage {
  using E = cx<R>;
  const PassDesc& d;
  const MixedStage& st;
  const E* tw;
  const E* tws;   // per-stage twiddle records (or null)
  const E* src;   // shared-memory row (when !SG)
  E* dst;         // shared-memory row (when !DG)
  const E* gsrc;  // global row (when SG)
  int j, tpr;
  bool inv, do_scale;
  R scale;
  int peer0;       // peer contribution of (o, t)
  long long toff;  // destination offset of column 0 of this row (when DG)

  template <int RADIX>
  __host__ __device__ __forceinline__ void run() const {
    const int nb = st.nb, ls = st.ls;
    for (int bf = j; bf < nb; bf += tpr) {
      E a[RADIX];
      if constexpr (SG) {
#pragma unroll
        for (int q = 0; q < RADIX; ++q) a[q] = gsrc[bf + q * nb];
        if (inv) {
#pragma unroll
          for (int q = 0; q < RADIX; ++q) a[q] = cswap(a[q]);
        }
      } else {
#pragma unroll
        for (int q = 0; q < RADIX; ++q) a[q] = src[padidx(bf + q * nb, 1)];
      }
      const int base = mixed_butterfly<R, RADIX>(st, tw, tws, bf, a);
      if constexpr (DG) {
#pragma unroll
        for (int q = 0; q < RADIX; ++q) {
          const int c = base + q * ls;
          E v = a[q];
          if (inv) v = cswap(v);
          if (do_scale) v = cscale(v, scale);
          const int pc = d.split_axis == 1 ? c / d.Cl : 0;
          store_elem<E>(d, peer0 + pc, toff + (c - pc * d.Cl), v);
        }
      } else {
#pragma unroll
        for (int q = 0; q < RADIX; ++q) dst[padidx(base + q * ls, 1)] = a[q];
      }
    }
  }
};

template <typename R, bool DIN, bool DOUT>
__global__ void __launch_bounds__(sizeof(R) == 4 ? 512 : 256, 2)
    fft_mixed_kernel(const __grid_constant__ PassDesc d, const __grid_constant__ MixedPlan pl, int tpr) {
  using E = cx<R>;
  extern __shared__ __align__(16) unsigned char mixed_smem[];
  E* buf0 = reinterpret_cast<E*>(mixed_smem);
  E* buf1 = buf0 + (size_t)d.T * d.pitch;

  if (pass_aborted(d)) return;
  const int tid = threadIdx.x;
  const int tiles_t = (d.Tn + d.T - 1) / d.T;
  const int tt = blockIdx.x % tiles_t;
  const int o = blockIdx.x / tiles_t;
  const int b = blockIdx.y;
  const int t0 = tt * d.T;
  const int row = tid / tpr;
  const int j = tid - row * tpr;
  const bool active = row < d.T && t0 + row < d.Tn;
  const bool inv = d.inverse != 0;

  if constexpr (!DIN) {
    tile_load<E>(d, buf0, o, t0, 0, b, tid, blockDim.x);
    __syncthreads();
  }
  const E* gsrc = (const E*)d.in + ((long long)o * d.is_o + (long long)b * d.is_b + (long long)(t0 + row) * d.is_t);
  const OutBase ob = out_base_for(d, o, b);
  const int t = t0 + row;
  const int pt = d.split_axis == 2 ? t / d.Tl : 0;
  const long long toff = ob.off + (long long)(t - pt * d.Tl) * d.os_t;
  const E* tw = (const E*)d.twiddle;
  const E* tws = (const E*)d.tw_stage;
  const R scale = (R)d.scale;
  const bool do_scale = d.scale != 1.0;

  int cur = DIN ? -1 : 0;  // buffer that holds the current data (-1: still in global memory)
  for (int s = 0; s < pl.ns; ++s) {
    const bool sg = DIN && s == 0;
    const bool dg = DOUT && s == pl.ns - 1;
    const E* src = (cur == 0 ? buf0 : buf1) + row * d.pitch;
    E* dst = (cur == 0 ? buf1 : buf0) + row * d.pitch;
    if (active) {
      const MixedStage& st = pl.st[s];
      if (sg && dg) {
        if constexpr (DIN && DOUT)
          mixed_dispatch(st.radix, DevStage<R, true, true>{d, st, tw, tws, src, dst, gsrc, j, tpr, inv, do_scale, scale,
                                                           ob.peer + pt, toff});
      } else if (sg) {
        if constexpr (DIN)
          mixed_dispatch(st.radix, DevStage<R, true, false>{d, st, tw, tws, src, dst, gsrc, j, tpr, inv, do_scale, scale,
                                                            ob.peer + pt, toff});
      } else if (dg) {
        if constexpr (DOUT)
          mixed_dispatch(st.radix, DevStage<R, false, true>{d, st, tw, tws, src, dst, gsrc, j, tpr, inv, do_scale, scale,
                                                            ob.peer + pt, toff});
      } else {
        mixed_dispatch(st.radix, DevStage<R, false, false>{d, st, tw, tws, src, dst, gsrc, j, tpr, inv, do_scale, scale,
                                                           ob.peer + pt, toff});
      }
    }
    if (!dg) {
      __syncthreads();
      cur = cur == 0 ? 1 : 0;
    }
  }
  if constexpr (!DOUT) tile_store<E>(d, cur == 0 ? buf0 : buf1, o, t0, 0, b, tid, blockDim.x);
}

// ---- host side --------------------------------------------------------------------------------------------------
static int mixed_threads(const PassDesc& d, const MixedPlan& pl, int* tpr_out) {
  const int tpr = mixed_threads_per_row(pl, d.T, d.elem_bytes);
  if (tpr <= 0) return 0;
  *tpr_out = tpr;
  int nt = d.T * tpr;
  nt = (nt + 31) / 32 * 32;
  return nt < 32 ? 32 : nt;
}

template <typename R, bool DIN, bool DOUT>
static int launch_mixed_t(const PassDesc& d, const MixedPlan& pl, cudaStream_t stream) {
  int tpr = 1;
  const int nt = mixed_threads(d, pl, &tpr);
  if (nt <= 0) {
    set_last_error("mixed-radix pass: tile has more rows than one thread block can serve (reduce T)");
    return JD_ERR_INVALID_ARG;
  }
  const size_t smem = 2 * (size_t)d.T * d.pitch * d.elem_bytes;
  constexpr size_t kMaxDynSmem = 226 * 1024;
  if (smem > kMaxDynSmem) {
    set_last_error("mixed-radix pass: tile exceeds the shared memory of one block");
    return JD_ERR_INVALID_ARG;
  }
  auto kern = fft_mixed_kernel<R, DIN, DOUT>;
  static bool configured = false;  // one flag per template instantiation
  if (smem > 48 * 1024 && !configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxDynSmem);
    if (e != cudaSuccess) {
      set_last_error(cudaGetErrorString(e));
      return JD_ERR_CUDA;
    }
    configured = true;
  }
  const long long nblocks = (long long)((d.Tn + d.T - 1) / d.T) * d.On;
  if (nblocks > 2147483647LL || d.B > 65535) {
    set_last_error("mixed-radix pass: grid too large");
    return JD_ERR_INVALID_ARG;
  }
  kern<<<dim3((unsigned)nblocks, (unsigned)d.B, 1), nt, smem, stream>>>(d, pl, tpr);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return JD_ERR_CUDA;
  }
  return JD_OK;
}

template <typename R>
static int launch_mixed_r(const PassDesc& d, const MixedPlan& pl, cudaStream_t stream) {
  const bool din = !d.load_t_contig && d.is_c == 1;
  const bool dout = !d.store_t_contig && d.os_c == 1;
  if (din && dout) return launch_mixed_t<R, true, true>(d, pl, stream);
  if (din) return launch_mixed_t<R, true, false>(d, pl, stream);
  return launch_mixed_t<R, false, false>(d, pl, stream);
}

int launch_mixed_pass(const PassDesc& d, void* stream) {
  MixedPlan pl;
  if (d.fft_mode != JD_FFT_MIXED || !make_mixed_plan(d.M, &pl)) {
    set_last_error("mixed-radix pass: length has a prime factor above 13");
    return JD_ERR_INVALID_ARG;
  }
  if (d.elem_bytes != 8 && d.elem_bytes != 16) return JD_ERR_INVALID_ARG;
  const char* env = std::getenv("JD_B200_MIXED_STATIC");
  if (!(env && env[0] == '0')) {
    for (auto fn : {launch_mixed_static_a, launch_mixed_static_b, launch_mixed_static_c}) {
      const int rc = fn(d, stream);
      if (rc != JD_ERR_UNSUPPORTED) return rc;
    }
  }
  if (d.elem_bytes == 8) return launch_mixed_r<float>(d, pl, (cudaStream_t)stream);
  if (d.elem_bytes == 16) return launch_mixed_r<double>(d, pl, (cudaStream_t)stream);
  return JD_ERR_INVALID_ARG;
}

}  // namespace jdb
