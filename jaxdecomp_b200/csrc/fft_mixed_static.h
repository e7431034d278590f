// Mixed-radix tile pass specialised on the transform length: same algorithm
// and data path as fft_mixed.cu (first stage from global memory, ping-pong
// stages in shared memory, stores straight from the registers of the last stage), but the stage plan,
// the tile height, the row pitch and the thread layout are compile-time
// constants, so the per-element index arithmetic (the limiter of the generic
// kernel: 146 instructions per element, two thirds of them integer) folds
// into immediates.  Instantiated for the common lengths 2^k * {3, 5, 7, 9, 15,
// 25, 125} in fft_mixed_s*.cu; other lengths use the generic kernel.
#pragma once
#include <cuda_runtime.h>

#include "fft_mixed.h"
#include "launch.h"
#include "tile_ops.h"

namespace jdb {

template <typename R, int N_, int T_, bool DOUT_>
struct MixedCfg {
  static constexpr int N = N_, T = T_;
  static constexpr bool DOUT = DOUT_;
  static constexpr int EB = 2 * (int)sizeof(R);
  static constexpr MixedPlan PL = mixed_plan_of(N);
  static constexpr int NS = PL.ns;
  static constexpr int PITCH = mixed_static_pitch(N, EB, T);
  static constexpr int RH = T < 8 ? T : 8;                 // rows per shared-memory wavefront in the last rotating stage
  static constexpr int CB = (EB == 8 ? 16 : 8) / RH;       // columns per wavefront
  static constexpr int TPR = mixed_threads_per_row(PL, T, EB);
  static constexpr int NT = (T * TPR + 31) / 32 * 32;
  static constexpr size_t SMEM = 2 * (size_t)T * PITCH * EB;
  static constexpr int MINB = SMEM * 2 + 2048 <= 227 * 1024 ? 2 : 1;
  static_assert(NS >= 2 && TPR > 0, "length not supported by the specialised mixed-radix kernel");
  static_assert(SMEM <= 226 * 1024, "tile exceeds shared memory");
  // the row-major layout of the last rotating stage must reach every (row, butterfly index) pair
  static_assert(DOUT || CB * ((NT / (RH * CB)) / (T / RH)) >= TPR, "last-stage thread layout does not cover the tile");
};

// Stage S of the plan on the butterflies of one thread.  SG: inputs come from global memory; DG: outputs go
// to global memory, along the row (ROT false: column c at toff + c) or transposed (ROT true: column c at
// toff + c * os_c, toff being the position of this thread's row on the destination's fastest axis).
template <typename Cfg, typename R, int S, bool SG, bool DG, bool ROT>
__device__ __forceinline__ void static_stage(const PassDesc& d, const cx<R>* __restrict__ tw,
                                             const cx<R>* __restrict__ tws, const cx<R>* src, cx<R>* dst,
                                             const cx<R>* __restrict__ gsrc, int j, bool inv, bool do_scale, R scale,
                                             int peer0, long long toff) {
  using E = cx<R>;
  constexpr int RADIX = Cfg::PL.st[S].radix, NB = Cfg::PL.st[S].nb, LS = Cfg::PL.st[S].ls;
  constexpr int REC0 = Cfg::PL.st[S].rec0;
  constexpr int TPR = Cfg::TPR;
  constexpr int ITERS = (NB + TPR - 1) / TPR;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int bf = j + it * TPR;
    if ((NB % TPR) != 0 && it == ITERS - 1 && bf >= NB) break;
    E a[RADIX];
    if constexpr (SG) {
#pragma unroll
      for (int q = 0; q < RADIX; ++q) a[q] = gsrc[bf + q * NB];
      if (inv) {
#pragma unroll
        for (int q = 0; q < RADIX; ++q) a[q] = cswap(a[q]);
      }
    } else if constexpr (NB % 16 == 0) {
      const E* p = src + padidx(bf, 1);  // the padded distance is linear when NB is a multiple of 16
#pragma unroll
      for (int q = 0; q < RADIX; ++q) a[q] = p[q * (NB + NB / 8)];
    } else {
#pragma unroll
      for (int q = 0; q < RADIX; ++q) a[q] = src[padidx(bf + q * NB, 1)];
    }
    int kk = 0, blk = bf;
    if constexpr (LS > 1) {
      blk = bf / LS;
      kk = bf - blk * LS;
      twiddle_record<R, RADIX>(tws + 4 * (REC0 + kk), a);
    }
    dft_any<R, RADIX>(a);
    const int base = blk * (LS * RADIX) + kk;
    if constexpr (DG) {
      // c / Cl by multiply-high (c, Cl < 2^16; Cl >= 2 whenever the columns are split)
      const uint32_t clm = d.split_axis == 1 ? (uint32_t)(0x100000000ULL / (unsigned)d.Cl) + 1u : 0u;
#pragma unroll
      for (int q = 0; q < RADIX; ++q) {
        const int c = base + q * LS;
        E v = a[q];
        if (inv) v = cswap(v);
        if (do_scale) v = cscale(v, scale);
        const int pc = d.split_axis == 1 ? (int)__umulhi((uint32_t)c, clm) : 0;
        const int cl = c - pc * d.Cl;
        if constexpr (ROT) {
          store_elem<E>(d, peer0 + pc, toff + (long long)cl * d.os_c, v);
        } else {
          store_elem<E>(d, peer0 + pc, toff + cl, v);
        }
      }
    } else if constexpr (LS % 16 == 0) {
      E* p = dst + padidx(base, 1);
#pragma unroll
      for (int q = 0; q < RADIX; ++q) p[q * (LS + LS / 8)] = a[q];
    } else if constexpr (LS == 1 && sizeof(R) == 4 && (RADIX == 16 || RADIX == 8 || RADIX == 4 || RADIX == 2)) {
      // RADIX consecutive columns starting at a multiple of RADIX: inside one padded group of sixteen
      cx2<R>* v = reinterpret_cast<cx2<R>*>(dst + padidx(base, 1));
#pragma unroll
      for (int q = 0; q < RADIX / 2; ++q) v[q] = cx2<R>{a[2 * q], a[2 * q + 1]};
    } else {
#pragma unroll
      for (int q = 0; q < RADIX; ++q) dst[padidx(base + q * LS, 1)] = a[q];
    }
  }
}

// Which row and which butterflies a thread serves, and where that row lands in the destination.
struct MixedThreadMap {
  int row, j;
  bool active;
  int peer0;
  long long toff;
};

template <typename Cfg, typename R, int S>
__device__ __forceinline__ void static_stages(const PassDesc& d, const cx<R>* tw, const cx<R>* tws, cx<R>* buf0,
                                              cx<R>* buf1,
                                              const cx<R>* gsrc, const MixedThreadMap& m, const MixedThreadMap& mlast,
                                              bool inv, bool do_scale, R scale) {
  using E = cx<R>;
  constexpr bool SG = S == 0;
  constexpr bool LAST = S == Cfg::NS - 1;
  constexpr bool ROT = LAST && !Cfg::DOUT;  // last stage of a rotating pass: transposed store from registers
  constexpr bool DG = LAST;
  const MixedThreadMap& mm = ROT ? mlast : m;
  // stage 0 writes buffer 0, stage 1 reads it and writes buffer 1, ...
  const E* src = ((S - 1) % 2 == 0 ? buf0 : buf1) + mm.row * Cfg::PITCH;
  E* dst = (S % 2 == 0 ? buf0 : buf1) + mm.row * Cfg::PITCH;
  if (mm.active)
    static_stage<Cfg, R, S, SG, DG, ROT>(d, tw, tws, src, dst, gsrc, mm.j, inv, do_scale, scale, mm.peer0, mm.toff);
  if constexpr (!LAST) {
    __syncthreads();
    static_stages<Cfg, R, S + 1>(d, tw, tws, buf0, buf1, gsrc, m, mlast, inv, do_scale, scale);
  }
}

template <typename R, int N, int T, bool DOUT>
__global__ void __launch_bounds__((MixedCfg<R, N, T, DOUT>::NT), (MixedCfg<R, N, T, DOUT>::MINB))
    fft_mixed_static_kernel(const __grid_constant__ PassDesc d) {
  using Cfg = MixedCfg<R, N, T, DOUT>;
  using E = cx<R>;
  extern __shared__ __align__(16) unsigned char mixed_static_smem[];
  E* buf0 = reinterpret_cast<E*>(mixed_static_smem);
  E* buf1 = buf0 + (size_t)T * Cfg::PITCH;

  if (pass_aborted(d)) return;
  const int tid = threadIdx.x;
  const int tiles_t = (d.Tn + T - 1) / T;
  const int tt = blockIdx.x % tiles_t;
  const int o = blockIdx.x / tiles_t;
  const int b = blockIdx.y;
  const int t0 = tt * T;
  const bool inv = d.inverse != 0;
  const OutBase ob = out_base_for(d, o, b);
  const R scale = (R)d.scale;
  const bool do_scale = d.scale != 1.0;
  // row-wise layout: TPR consecutive threads serve one row
  MixedThreadMap m;
  m.row = tid / Cfg::TPR;
  m.j = tid - m.row * Cfg::TPR;
  m.active = m.row < T && t0 + m.row < d.Tn;
  {
    const int t = t0 + m.row;
    const int pt = d.split_axis == 2 ? t / d.Tl : 0;
    m.peer0 = ob.peer + pt;
    m.toff = ob.off + (long long)(t - pt * d.Tl) * d.os_t;
  }
  // layout of the last stage of a rotating pass: consecutive threads serve consecutive rows of the same
  // butterflies, so that the results of one column are stored by neighbouring lanes as one run
  MixedThreadMap ml = m;
  if constexpr (!DOUT) {
    ml.row = mixed_last_stage_row(T, Cfg::EB, tid);
    ml.j = mixed_last_stage_j(T, Cfg::EB, tid);
    ml.active = ml.j < Cfg::TPR && t0 + ml.row < d.Tn;
    const int t = t0 + ml.row;
    const int pt = d.split_axis == 2 ? t / d.Tl : 0;
    ml.peer0 = ob.peer + pt;
    ml.toff = ob.off + (long long)(t - pt * d.Tl) * d.os_t;
  }
  const E* gsrc = (const E*)d.in + ((long long)o * d.is_o + (long long)b * d.is_b + (long long)(t0 + m.row) * d.is_t);
  static_stages<Cfg, R, 0>(d, (const E*)d.twiddle, (const E*)d.tw_stage, buf0, buf1, gsrc, m, ml, inv, do_scale, scale);
}

template <typename R, int N, int T, bool DOUT>
static int launch_mixed_static_t(const PassDesc& d, cudaStream_t stream) {
  using Cfg = MixedCfg<R, N, T, DOUT>;
  auto kern = fft_mixed_static_kernel<R, N, T, DOUT>;
  static bool configured = false;  // one flag per template instantiation
  if (Cfg::SMEM > 48 * 1024 && !configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
    if (e != cudaSuccess) {
      set_last_error(cudaGetErrorString(e));
      return JD_ERR_CUDA;
    }
    configured = true;
  }
  const long long nblocks = (long long)((d.Tn + T - 1) / T) * d.On;
  if (nblocks > 2147483647LL || d.B > 65535) {
    set_last_error("mixed-radix pass: grid too large");
    return JD_ERR_INVALID_ARG;
  }
  kern<<<dim3((unsigned)nblocks, (unsigned)d.B, 1), Cfg::NT, Cfg::SMEM, stream>>>(d);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return JD_ERR_CUDA;
  }
  return JD_OK;
}

// JD_ERR_UNSUPPORTED: the descriptor does not match the specialised geometry (strided load, other tile height
// or pitch, unaligned transposed store): the caller uses the generic kernel.
template <typename R, int N>
static int launch_mixed_static_n(const PassDesc& d, cudaStream_t stream) {
  constexpr int EB = 2 * (int)sizeof(R);
  if (d.load_t_contig || d.is_c != 1 || d.M != N || d.tw_stage == nullptr) return JD_ERR_UNSUPPORTED;
  if (d.split_axis == 1 && d.Cl < 2) return JD_ERR_UNSUPPORTED;
  if (!d.store_t_contig) {
    constexpr int T = mixed_static_T(N, EB, false);
    if (d.os_c != 1 || d.T != T || d.pitch != mixed_static_pitch(N, EB, T)) return JD_ERR_UNSUPPORTED;
    return launch_mixed_static_t<R, N, T, true>(d, stream);
  }
  constexpr int T = mixed_static_T(N, EB, true);
  if (d.os_t != 1 || d.T != T || d.pitch != mixed_static_pitch(N, EB, T)) return JD_ERR_UNSUPPORTED;
  return launch_mixed_static_t<R, N, T, false>(d, stream);
}

}  // namespace jdb
