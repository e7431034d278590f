// Specialised tile pass for the hot case: power-of-two transform lengths
// 128..4096 read along the contiguous axis.  Same contract as the general
// kernel in fft_pass.cu (one PassDesc, rotated peer stores or plain stores),
// but every tile extent is a compile-time constant so that shared-memory
// offsets become immediates, and the data path is shortened:
//
//   * stage 0 takes its eight inputs straight from global memory into
//     registers (coalesced 8-byte loads along the pencil): no staging pass;
//   * the butterflies of a pencil are owned by a fixed group of M/8 threads,
//     which synchronise among themselves with a named barrier (or __syncwarp
//     when the group is a warp) instead of a block-wide barrier;
//   * twiddles come from per-stage tables laid out as eight consecutive
//     factors per butterfly: four 16-byte loads, no multiplications to derive them;
//   * a plain (non-rotating) pass writes the last stage's results directly to
//     global memory; a rotating pass goes through shared memory once more so
//     that each thread stores 16 contiguous bytes along the destination's
//     fastest axis, into the buffer of the peer that owns those columns.
//
//   * measured on B200, stores in runs shorter than 128 bytes reach only a
//     fraction of the NVLink (64-byte runs: 479 of 715 GB/s) and HBM (64-byte
//     runs: 3.2 of 6.2 TB/s) write bandwidth, so rotating passes use tiles of up
//     to 16384 elements handled by up to 1024 threads, which doubles the length
//     of every stored run (a thread-block-cluster variant that gathered the
//     rows of neighbouring blocks through distributed shared memory was
//     measured to be slower than single-block tiles and is not used).
//
// Shared-memory rows use the padded layout of fft_core.h (padidx), which keeps
// all exchange patterns free of bank conflicts for 8-byte elements.
#include <cuda_runtime.h>

#include <cstdlib>

#include "launch.h"
#include "tile_ops.h"

namespace jdb {

template <typename R, int LOGM_, int LOGT_, bool STORE_T_>
struct FastCfg {
  static constexpr int LOGM = LOGM_, LOGT = LOGT_;
  static constexpr bool STORE_T = STORE_T_;
  static constexpr int M = 1 << LOGM, T = 1 << LOGT;
  static constexpr int UPR = M / 8;            // butterflies (threads) per row
  static constexpr int LOGUPR = LOGM - 3;
  static constexpr int UNITS = T * UPR;
  // two butterflies per thread once the tile is large enough; at most 1024 (complex64) / 512 (complex128) threads
  static constexpr int NTMAX = sizeof(R) == 8 ? 512 : 1024;
  static constexpr int NTWANT = UNITS >= 1024 ? UNITS / 2 : UNITS;
  static constexpr int NT = NTWANT < NTMAX ? NTWANT : NTMAX;
  static constexpr int ITERS = UNITS / NT;
  // threads that synchronise together: whole rows, and at most eight groups per block (named barriers 1..8)
  static constexpr int GS = UPR > NT / 8 ? UPR : NT / 8;
  static constexpr int ROWS_PER_ROUND = NT / UPR;  // rows handled at once (>= 1 because UPR <= 512 <= ... see static_assert)
  static constexpr int ROWLEN = M + M / 8;
  static constexpr int PITCH = ROWLEN + 2;     // == 2 (mod 16): conflict-free transposed reads for 4 row pairs
  static constexpr int N8 = LOGM / 3;
  static constexpr int REM = LOGM - 3 * N8;    // log2 of the last, smaller radix (0 if none)
  static constexpr int NS = N8 + (REM ? 1 : 0);
  static constexpr int REGS = (sizeof(R) == 8 ? 2 : 1) * (ITERS <= 1 ? 40 : (ITERS == 2 ? 64 : 128));
  static constexpr int MINB_ = 65536 / (NT * REGS);
  static constexpr int MINB = MINB_ < 1 ? 1 : (MINB_ > 4 ? 4 : MINB_);
  static constexpr size_t SMEM = (size_t)T * PITCH * 2 * sizeof(R);
  static_assert(NT % UPR == 0, "a row must be owned by whole thread groups");
  static_assert(ITERS >= 1 && ITERS <= 4, "tile too large");
};

// Per-stage twiddle table: for stage s >= 1 (Ls = 8^s) entry [off_s + kk*8 + q] = exp(-2 pi i q kk / (8 Ls)).
__host__ __device__ constexpr int stage_table_offset(int s) {
  int off = 0, ls = 8;
  for (int i = 1; i < s; ++i) {
    off += 8 * ls;
    ls *= 8;
  }
  return off;
}

template <int UPR, int GS>
__device__ __forceinline__ void group_sync(int sync_group) {
  if constexpr (UPR <= 32) {
    __syncwarp();
  } else {
    asm volatile("bar.sync %0, %1;" ::"r"(sync_group + 1), "n"(GS) : "memory");
  }
}

template <typename R>
__device__ __forceinline__ cx<R> ldg_cx(const cx<R>* p) {
  if constexpr (sizeof(R) == 4) {
    const float2 v = __ldg(reinterpret_cast<const float2*>(p));
    return cx<R>{v.x, v.y};
  } else {
    const double2 v = __ldg(reinterpret_cast<const double2*>(p));
    return cx<R>{v.x, v.y};
  }
}

template <typename R>
__device__ __forceinline__ void load_tw8(const cx<R>* __restrict__ p, cx<R> w[8]) {
  if constexpr (sizeof(R) == 4) {
    const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = __ldg(q + i);
      w[2 * i] = cx<R>{v.x, v.y};
      w[2 * i + 1] = cx<R>{v.z, v.w};
    }
  } else {
    const double2* q = reinterpret_cast<const double2*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const double2 v = __ldg(q + i);
      w[i] = cx<R>{v.x, v.y};
    }
  }
}

template <typename Cfg, typename R, int S, int LOGLS>
__device__ __forceinline__ void fast_stage(cx<R>* sm, const int (&rbase)[Cfg::ITERS], const int (&rowoff)[Cfg::ITERS], int j,
                                           int sgroup, cx<R> (&a)[Cfg::ITERS][8], const cx<R>* __restrict__ tw,
                                           const cx<R>* __restrict__ stw, bool to_smem) {
  using E = cx<R>;
  constexpr int M = Cfg::M, LOGM = Cfg::LOGM, ITERS = Cfg::ITERS;
  constexpr int RL = S < Cfg::N8 ? 3 : Cfg::REM;
  constexpr int Ls = 1 << LOGLS;
  constexpr int QP = Cfg::UPR + Cfg::UPR / 8;  // padded distance between a thread's eight inputs
  if constexpr (S > 0) {
    // inputs of this stage: the eight values at j + k*M/8 of the row
#pragma unroll
    for (int it = 0; it < ITERS; ++it)
#pragma unroll
      for (int k = 0; k < 8; ++k) a[it][k] = sm[rbase[it] + k * QP];
    group_sync<Cfg::UPR, Cfg::GS>(sgroup);  // all reads of the group done before anyone overwrites
  }
  if constexpr (RL == 3) {
    const int kk = j & (Ls - 1);
    if constexpr (S > 0) {
      E w[8];
      load_tw8<R>(stw + stage_table_offset(S) + kk * 8, w);
#pragma unroll
      for (int it = 0; it < ITERS; ++it)
#pragma unroll
        for (int k = 1; k < 8; ++k) a[it][k] = cmul(a[it][k], w[k]);
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it) dft8(a[it]);
    if (to_smem) {
      const int base = ((j - kk) << 3) + kk;
      const int pb = padidx(base, 1);
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        E* p = sm + rowoff[it] + pb;
        if constexpr (LOGLS == 0) {
          cx2<R>* v = reinterpret_cast<cx2<R>*>(p);
#pragma unroll
          for (int k = 0; k < 4; ++k) v[k] = cx2<R>{a[it][2 * k], a[it][2 * k + 1]};
        } else if constexpr (LOGLS == 3) {
#pragma unroll
          for (int k = 0; k < 8; ++k) p[8 * k + 2 * (k >> 1)] = a[it][k];
        } else {
          constexpr int LP = Ls + Ls / 8;
#pragma unroll
          for (int k = 0; k < 8; ++k) p[k * LP] = a[it][k];
        }
      }
    }
  } else if constexpr (RL == 2) {
    // two radix-4 butterflies b = j + m*M/8 on (a[m], a[m+2], a[m+4], a[m+6]); Ls == M/4
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      const int bfly = j + m * Cfg::UPR;
      const E w1 = ldg_cx<R>(tw + bfly), w2 = ldg_cx<R>(tw + 2 * bfly);
      const E w3 = cmul(w1, w2);
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        E x0 = a[it][m], x1 = cmul(a[it][m + 2], w1), x2 = cmul(a[it][m + 4], w2), x3 = cmul(a[it][m + 6], w3);
        dft4(x0, x1, x2, x3);
        a[it][m] = x0; a[it][m + 2] = x1; a[it][m + 4] = x2; a[it][m + 6] = x3;
      }
    }
    if (to_smem) {
#pragma unroll
      for (int it = 0; it < ITERS; ++it)
#pragma unroll
        for (int k = 0; k < 8; ++k) sm[rbase[it] + k * QP] = a[it][k];  // output b + q*M/4 == j + (m + 2q)*M/8
    }
  } else if constexpr (RL == 1) {
    // four radix-2 butterflies b = j + m*M/8 on (a[m], a[m+4]); Ls == M/2
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const E w = ldg_cx<R>(tw + j + m * Cfg::UPR);
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        E x0 = a[it][m], x1 = cmul(a[it][m + 4], w);
        dft2(x0, x1);
        a[it][m] = x0;
        a[it][m + 4] = x1;
      }
    }
    if (to_smem) {
#pragma unroll
      for (int it = 0; it < ITERS; ++it)
#pragma unroll
        for (int k = 0; k < 8; ++k) sm[rbase[it] + k * QP] = a[it][k];
    }
  }
  if constexpr (S + 1 < Cfg::NS) {
    group_sync<Cfg::UPR, Cfg::GS>(sgroup);  // this stage's writes visible to the group
    fast_stage<Cfg, R, S + 1, LOGLS + RL>(sm, rbase, rowoff, j, sgroup, a, tw, stw, (S + 2 < Cfg::NS) || Cfg::STORE_T);
  }
}

template <typename R, int LOGM, int LOGT, bool STORE_T>
__global__ void __launch_bounds__((FastCfg<R, LOGM, LOGT, STORE_T>::NT), (FastCfg<R, LOGM, LOGT, STORE_T>::MINB))
    fft_fast_kernel(const __grid_constant__ PassDesc d) {
  using Cfg = FastCfg<R, LOGM, LOGT, STORE_T>;
  using E = cx<R>;
  constexpr int M = Cfg::M, T = Cfg::T, NT = Cfg::NT, ITERS = Cfg::ITERS, UPR = Cfg::UPR;
  extern __shared__ __align__(16) unsigned char fast_smem[];
  E* sm = reinterpret_cast<E*>(fast_smem);

  const int tid = threadIdx.x;
  const int tiles_t = d.Tn >> LOGT;
  const int tt = blockIdx.x % tiles_t;
  const int o = blockIdx.x / tiles_t;
  const int b = blockIdx.y;
  const int t0 = tt << LOGT;
  const bool inv = d.inverse != 0;

  const int j = tid & (UPR - 1);
  const int group = tid >> Cfg::LOGUPR;
  int rbase[ITERS], rowoff[ITERS];
  E a[ITERS][8];
  const E* __restrict__ in = (const E*)d.in + ((long long)o * d.is_o + (long long)b * d.is_b + (long long)t0 * d.is_t);
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int row = it * Cfg::ROWS_PER_ROUND + group;
    rowoff[it] = row * Cfg::PITCH;
    rbase[it] = rowoff[it] + padidx(j, 1);
    const E* src = in + (long long)row * d.is_t + j;
#pragma unroll
    for (int k = 0; k < 8; ++k) a[it][k] = src[k * UPR];
  }
  if (inv) {
#pragma unroll
    for (int it = 0; it < ITERS; ++it)
#pragma unroll
      for (int k = 0; k < 8; ++k) a[it][k] = cswap(a[it][k]);
  }
  const E* __restrict__ tw = (const E*)d.twiddle;
  const E* __restrict__ stw = (const E*)d.bhat;  // per-stage twiddle table travels in the (otherwise unused) bhat slot
  fast_stage<Cfg, R, 0, 0>(sm, rbase, rowoff, j, tid / Cfg::GS, a, tw, stw, Cfg::NS > 1 || STORE_T);

  const R scale = (R)d.scale;
  const bool do_scale = d.scale != 1.0;
  if constexpr (!STORE_T) {
    // results of the last stage sit in registers in natural order positions:
    // radix 8: j + k*M/8 holds output index base + k*Ls with Ls == M/8  -> column j + k*M/8
    // radix 4/2: same columns (see fast_stage).  Store them straight to global memory.
    const OutBase ob = out_base_for(d, o, b);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int t = t0 + it * Cfg::ROWS_PER_ROUND + group;
      const int pt = d.split_axis == 2 ? t / d.Tl : 0;
      const long long toff = ob.off + (long long)(t - pt * d.Tl) * d.os_t;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int c = j + k * UPR;
        E v = a[it][k];
        if (inv) v = cswap(v);
        if (do_scale) v = cscale(v, scale);
        const int pc = d.split_axis == 1 ? c / d.Cl : 0;
        ((E*)d.out[ob.peer + pc + pt])[toff + (c - pc * d.Cl)] = v;
      }
    }
  } else {
    __syncthreads();  // the transposed store reads every row of the tile
    constexpr int PER16 = 16 / (2 * (int)sizeof(R));  // elements per 16-byte store: 2 (complex64) or 1 (complex128)
    constexpr int TP = T / PER16;                    // threads that share one column
    constexpr int LOGTP = LOGT - (PER16 == 2 ? 1 : 0);
    constexpr int STEP = NT / TP;                    // columns advanced per iteration
    static_assert(STEP % 16 == 0, "column step must keep the padded index linear");
    constexpr int STEPP = STEP + STEP / 8;
    const int tp = tid & (TP - 1);
    const int t = tp * PER16;
    const int cs = tid >> LOGTP;
    const OutBase ob = out_base_for(d, o, b);
    const int tg = t0 + t;
    const int pt = d.split_axis == 2 ? tg / d.Tl : 0;
    const long long toff = ob.off + (long long)(tg - pt * d.Tl) * d.os_t;
    const E* src = sm + t * Cfg::PITCH + padidx(cs, 1);
    const int logCl = 31 - __clz(d.Cl);
#pragma unroll 4
    for (int i = 0; i < M / STEP; ++i) {
      const int c = cs + i * STEP;
      int pc = 0, cl = c;
      if (d.split_axis == 1) {
        pc = c >> logCl;
        cl = c & (d.Cl - 1);
      }
      E* dst = (E*)d.out[ob.peer + pc + pt] + (toff + (long long)cl * d.os_c);
      E v0 = src[i * STEPP];
      if (inv) v0 = cswap(v0);
      if (do_scale) v0 = cscale(v0, scale);
      if constexpr (PER16 == 2) {
        E v1 = src[Cfg::PITCH + i * STEPP];
        if (inv) v1 = cswap(v1);
        if (do_scale) v1 = cscale(v1, scale);
        *reinterpret_cast<cx2<R>*>(dst) = cx2<R>{v0, v1};
      } else {
        *dst = v0;
      }
    }
  }
}

// ---- host side --------------------------------------------------------------------------------------------------
static bool is_pow2(long long v) { return v > 0 && (v & (v - 1)) == 0; }

// The tile height the fast kernel is instantiated with for a given length and element size.
static bool big_tiles(const PassDesc& d) {
  // Large tiles (128 KiB of data, one block per SM) double the stored run length of rotating
  // passes.  Measured: they pay off when the stores cross NVLink (128-byte runs reach the full
  // peer-store bandwidth) and lose slightly for local passes, so they are the default only there.
  const char* env = std::getenv("JD_B200_BIGTILE");
  if (env && *env) return env[0] != '0';
  return d.store_t_contig != 0 && d.npeers > 1;
}

int fast_pass_logT(int logM, int elem_bytes, bool big) {
  // complex64: T*M = 8192 elements (64 KiB of data) or 16384 when big, T <= 32;
  // complex128: half as many elements, T <= 16
  const int budget = (elem_bytes == 8 ? 13 : 12) + (big ? 1 : 0);
  const int cap = elem_bytes == 8 ? 5 : 4;
  int lt = budget - logM;
  if (lt < 1) lt = 1;
  if (lt > cap) lt = cap;
  return lt;
}

bool fast_pass_eligible(const PassDesc& d) {
  if (d.fft_mode != JD_FFT_POW2) return false;
  if (d.elem_bytes != 8 && d.elem_bytes != 16) return false;
  if (d.M < 128 || d.M > (d.elem_bytes == 8 ? 4096 : 2048) || d.C != d.M) return false;
  if (d.load_t_contig || d.is_c != 1) return false;
  int logM = 0;
  while ((1 << logM) < d.M) ++logM;
  // the small tile height must divide the rows (the big variant is used only when it divides too)
  const int lt = fast_pass_logT(logM, d.elem_bytes, false);
  if (d.Tn % (1 << lt)) return false;
  if (!d.bhat) return false;  // per-stage twiddle table
  if (d.store_t_contig) {
    if (d.os_t != 1) return false;
    const int per16 = 16 / d.elem_bytes;
    if (per16 == 2) {
      if ((d.Tl & 1) || (d.out_base & 1) || (d.os_c & 1) || (d.os_o & 1) || (d.os_b & 1)) return false;
      for (int p = 0; p < d.npeers; ++p)
        if ((uintptr_t)d.out[p] % 16) return false;
    }
    if (d.split_axis == 1 && !is_pow2(d.Cl)) return false;
  } else {
    if (d.os_c != 1) return false;
  }
  return true;
}

template <typename R, int LOGM, int LOGT, bool STORE_T>
static int launch_fast_t(const PassDesc& d, cudaStream_t stream) {
  using Cfg = FastCfg<R, LOGM, LOGT, STORE_T>;
  auto kern = fft_fast_kernel<R, LOGM, LOGT, STORE_T>;
  static bool configured = false;
  if (!configured) {
    if (Cfg::SMEM > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
      if (e != cudaSuccess) {
        set_last_error(cudaGetErrorString(e));
        return JD_ERR_CUDA;
      }
    }
    configured = true;
  }
  const long long nblocks = (long long)(d.Tn >> LOGT) * d.On;
  if (nblocks > 2147483647LL || d.B > 65535) {
    set_last_error("fast pass: grid too large");
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

template <int LOGM, int BUDGET, int CAP>
struct TileLog {
  static constexpr int value = (BUDGET - LOGM) < 1 ? 1 : ((BUDGET - LOGM) > CAP ? CAP : (BUDGET - LOGM));
};

template <typename R, int LOGM>
static int launch_fast_m(const PassDesc& d, cudaStream_t stream) {
  constexpr int budget = sizeof(R) == 4 ? 13 : 12;
  constexpr int cap = sizeof(R) == 4 ? 5 : 4;
  constexpr int LT = TileLog<LOGM, budget, cap>::value;
  constexpr int LTB = TileLog<LOGM, budget + 1, cap>::value;
  if constexpr (LTB != LT) {
    if (big_tiles(d) && d.Tn % (1 << LTB) == 0) {
      if (d.store_t_contig) return launch_fast_t<R, LOGM, LTB, true>(d, stream);
      return launch_fast_t<R, LOGM, LTB, false>(d, stream);
    }
  }
  if (d.store_t_contig) return launch_fast_t<R, LOGM, LT, true>(d, stream);
  return launch_fast_t<R, LOGM, LT, false>(d, stream);
}

template <typename R>
static int launch_fast_r(const PassDesc& d, cudaStream_t stream) {
  switch (d.M) {
    case 128: return launch_fast_m<R, 7>(d, stream);
    case 256: return launch_fast_m<R, 8>(d, stream);
    case 512: return launch_fast_m<R, 9>(d, stream);
    case 1024: return launch_fast_m<R, 10>(d, stream);
    case 2048: return launch_fast_m<R, 11>(d, stream);
    case 4096:
      if constexpr (sizeof(R) == 4) return launch_fast_m<R, 12>(d, stream);
      return JD_ERR_UNSUPPORTED;
    default: return JD_ERR_UNSUPPORTED;
  }
}

int launch_fast_pass(const PassDesc& d, void* stream) {
  if (d.elem_bytes == 8) return launch_fast_r<float>(d, (cudaStream_t)stream);
  return launch_fast_r<double>(d, (cudaStream_t)stream);
}

}  // namespace jdb
