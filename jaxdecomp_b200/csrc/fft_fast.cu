// Specialised tile pass for the hot case: power-of-two transform lengths
// 128..4096 read along the contiguous axis.  Same contract as the general
// kernel in fft_pass.cu (one PassDesc, rotated peer stores or plain stores),
// but every tile extent is a compile-time constant so that shared-memory
// offsets become immediates, and the data path is shortened:
//
//   * every thread owns sixteen values of one pencil, row[j + k*M/16]; a stage
//     is a radix-16 butterfly on them or two radix-8 butterflies on interleaved
//     halves, so lengths up to 4096 need at most three stages
//     (128 = 16.8, 256 = 16.16, 512 = 8.8.8, 1024 = 16.8.8, 2048 = 16.16.8,
//     4096 = 16.16.16) and therefore at most two shared-memory exchanges
//     inside the transform -- profiles show the shared-memory data pipe, not
//     HBM, to be the limiter of these passes;
//   * stage 0 takes its inputs straight from global memory into registers
//     (coalesced 8-byte loads along the pencil): no staging pass;
//   * the butterflies of a pencil are owned by a fixed group of M/16 threads,
//     which synchronise among themselves with a named barrier (or __syncwarp
//     when the group fits in a warp) instead of a block-wide barrier;
//   * per butterfly only the factors w, w^2, w^4 (w^8) are read, as one contiguous
//     record of a per-stage table; the other powers are products of those (the
//     FP pipe has head-room, the load pipe has not);
//   * both kinds of pass write the last stage's results directly from registers
//     to global memory.  In a rotating pass the threads are re-assigned for the
//     last stage so that neighbouring lanes hold the same column of neighbouring
//     rows: their stores form runs of T elements along the destination's fastest
//     axis, in the buffer of the peer that owns those columns.  (An earlier
//     version transposed through shared memory once more; that exchange cost a
//     third of the shared-memory traffic of the pass.);
//   * measured on B200, stores in runs shorter than 128 bytes reach only a
//     fraction of the NVLink (64-byte runs: 479 of 715 GB/s) and HBM (64-byte
//     runs: 3.2 of 6.2 TB/s) write bandwidth, so passes whose stores cross
//     NVLink use tiles of 16384 elements handled by up to 1024 threads, which
//     doubles the length of every stored run (a thread-block-cluster variant
//     that gathered the rows of neighbouring blocks through distributed shared
//     memory, and a two-stage radix-32 variant with one warp per pencil, were
//     both measured to be slower and are not used).
//
// Shared-memory rows use the padded layout of fft_core.h (padidx), which keeps
// all exchange patterns free of bank conflicts for 8-byte elements.
#include <cuda_runtime.h>

#include <cstdlib>

#include "fft_fast_plan.h"
#include "fft_radix.h"
#include "launch.h"
#include "tile_ops.h"

namespace jdb {

// ---- stage plan: fft_fast_plan.h ----------------------------------------------------------------------------------
template <typename R, int LOGM_, int LOGT_, bool STORE_T_>
struct FastCfg {
  static constexpr int LOGM = LOGM_, LOGT = LOGT_;
  static constexpr bool STORE_T = STORE_T_;
  static constexpr int M = 1 << LOGM, T = 1 << LOGT;
  static constexpr int UPR = M / 16;           // threads per row
  static constexpr int LOGUPR = LOGM - 4;
  static constexpr int NT = T * UPR;           // one thread owns 16 values of one row
  // threads that synchronise together: whole rows, and at most eight groups per block (named barriers 1..8)
  static constexpr int GS = UPR > NT / 8 ? UPR : NT / 8;
  static constexpr int ROWLEN = M + M / 8;
  // Rotating passes: the last stage is done by threads laid out across the rows (see last_stage_map);
  // sixteen consecutive threads then read RH = min(T, 8) rows x 16/RH columns, which fall into
  // sixteen different 8-byte bank pairs when the pitch is 16/RH (mod 16).
  static constexpr int RH = T < 8 ? T : 8;
  static constexpr int CB = 16 / RH;
  static constexpr int PITCH = ROWLEN + CB;
  static constexpr int NS = plan_num_stages(LOGM);
  static constexpr int REGS = sizeof(R) == 8 ? 128 : 64;
  static constexpr int MINB_ = 65536 / (NT * REGS);
  static constexpr int MINB = MINB_ < 1 ? 1 : (MINB_ > 4 ? 4 : MINB_);
  static constexpr size_t SMEM = (size_t)T * PITCH * 2 * sizeof(R);
  static_assert(NT >= 32 && NT <= 1024, "tile does not map onto one thread block");
};

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

// a[FIRST + STRIDE*q] *= w^q for q = 1..N-1 (N = 8 or 16).  `rec` is the stage's record for this
// butterfly, {w, w^2, w^4, w^8} (fft_fast_plan.h), read with 16-byte loads; the other powers are
// products of at most four of them.  The kernel is limited by the L1/shared-memory data pipe, so
// deriving twiddles on the FP pipe is cheaper than loading a full row of factors per butterfly, and
// contiguous records are cheaper than scattered reads of the table of M roots.
template <typename R, int N, int FIRST, int STRIDE>
__device__ __forceinline__ void apply_tw(const cx<R>* __restrict__ rec, cx<R> (&a)[16]) {
  cx<R> w1, w2, w4, w8;
  if constexpr (sizeof(R) == 4) {
    const float4 lo = __ldg(reinterpret_cast<const float4*>(rec));
    w1 = cx<R>{lo.x, lo.y};
    w2 = cx<R>{lo.z, lo.w};
    if constexpr (N == 16) {
      const float4 hi = __ldg(reinterpret_cast<const float4*>(rec) + 1);
      w4 = cx<R>{hi.x, hi.y};
      w8 = cx<R>{hi.z, hi.w};
    } else {
      w4 = ldg_cx<R>(rec + 2);
    }
  } else {
    w1 = ldg_cx<R>(rec);
    w2 = ldg_cx<R>(rec + 1);
    w4 = ldg_cx<R>(rec + 2);
    if constexpr (N == 16) w8 = ldg_cx<R>(rec + 3);
  }
  const cx<R> w3 = cmul(w1, w2), w5 = cmul(w1, w4), w6 = cmul(w2, w4), w7 = cmul(w3, w4);
  a[FIRST + STRIDE * 1] = cmul(a[FIRST + STRIDE * 1], w1);
  a[FIRST + STRIDE * 2] = cmul(a[FIRST + STRIDE * 2], w2);
  a[FIRST + STRIDE * 3] = cmul(a[FIRST + STRIDE * 3], w3);
  a[FIRST + STRIDE * 4] = cmul(a[FIRST + STRIDE * 4], w4);
  a[FIRST + STRIDE * 5] = cmul(a[FIRST + STRIDE * 5], w5);
  a[FIRST + STRIDE * 6] = cmul(a[FIRST + STRIDE * 6], w6);
  a[FIRST + STRIDE * 7] = cmul(a[FIRST + STRIDE * 7], w7);
  if constexpr (N == 16) {
    a[FIRST + STRIDE * 8] = cmul(a[FIRST + STRIDE * 8], w8);
    a[FIRST + STRIDE * 9] = cmul(a[FIRST + STRIDE * 9], cmul(w1, w8));
    a[FIRST + STRIDE * 10] = cmul(a[FIRST + STRIDE * 10], cmul(w2, w8));
    a[FIRST + STRIDE * 11] = cmul(a[FIRST + STRIDE * 11], cmul(w3, w8));
    a[FIRST + STRIDE * 12] = cmul(a[FIRST + STRIDE * 12], cmul(w4, w8));
    a[FIRST + STRIDE * 13] = cmul(a[FIRST + STRIDE * 13], cmul(w5, w8));
    a[FIRST + STRIDE * 14] = cmul(a[FIRST + STRIDE * 14], cmul(w6, w8));
    a[FIRST + STRIDE * 15] = cmul(a[FIRST + STRIDE * 15], cmul(w7, w8));
  }
}

// Thread layout of the last stage of a rotating pass: consecutive threads own consecutive rows of the
// same butterfly index, so that the results of one column, which are contiguous in the destination,
// are stored by neighbouring lanes straight from registers (runs of T elements).
template <typename Cfg>
__device__ __forceinline__ void last_stage_map(int tid, int& row, int& j) {
  row = fast_last_stage_row(Cfg::T, tid);
  j = fast_last_stage_j(Cfg::T, tid);
}

// One stage on the sixteen values a[k] = row[j + k*M/16] of a thread.
template <typename Cfg, typename R, int S>
__device__ __forceinline__ void fast_stage(cx<R>* sm, cx<R>* rowp, int j, int sgroup, cx<R> (&a)[16],
                                           const cx<R>* __restrict__ stw, bool to_smem) {
  using E = cx<R>;
  constexpr int LOGM = Cfg::LOGM;
  constexpr int RL = plan_radix_log(LOGM, S);
  constexpr int LOGLS = plan_log_ls(LOGM, S);
  constexpr int Ls = 1 << LOGLS;
  constexpr int Q = Cfg::UPR;                  // distance between a thread's values
  if constexpr (S > 0) {
    if constexpr (Q >= 16) {
      constexpr int QP = Q + Q / 8;            // the padded distance is linear when Q is a multiple of 16
      const E* p = rowp + padidx(j, 1);
#pragma unroll
      for (int k = 0; k < 16; ++k) a[k] = p[k * QP];
    } else {
#pragma unroll
      for (int k = 0; k < 16; ++k) a[k] = rowp[padidx(j + k * Q, 1)];
    }
    // all reads of the group done before anyone overwrites (the last stage of a rotating pass writes nothing)
    if constexpr (!(Cfg::STORE_T && S + 1 == Cfg::NS)) group_sync<Cfg::UPR, Cfg::GS>(sgroup);
  }
  if constexpr (RL == 4) {
    const int kk = j & (Ls - 1);
    if constexpr (S > 0) apply_tw<R, 16, 0, 1>(stw + 4 * (plan_stage_record0(LOGM, S) + kk), a);
    dft16<R>(a);
    if (to_smem) {
      const int base = ((j - kk) << 4) + kk;
      if constexpr (LOGLS == 0) {
        // sixteen consecutive columns: one padded group, eight 2-element vector stores
        cx2<R>* v = reinterpret_cast<cx2<R>*>(rowp + padidx(base, 1));
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = cx2<R>{a[2 * k], a[2 * k + 1]};
      } else {
        // Ls >= 16 here (radix-16 stages come first): base + k*Ls stays linear in the padded layout
        E* p = rowp + padidx(base, 1);
        constexpr int LP = Ls + Ls / 8;
#pragma unroll
        for (int k = 0; k < 16; ++k) p[k * LP] = a[k];
      }
    }
  } else {
    // two radix-8 butterflies b = j + m*M/16 on the values k = m + 2q
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      const int bf = j + m * Q;
      const int kk = bf & (Ls - 1);
      if constexpr (S > 0) {
        if (m == 0) apply_tw<R, 8, 0, 2>(stw + 4 * (plan_stage_record0(LOGM, S) + kk), a);
        else apply_tw<R, 8, 1, 2>(stw + 4 * (plan_stage_record0(LOGM, S) + kk), a);
      }
      E x[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) x[q] = a[m + 2 * q];
      dft8(x);
      if (to_smem) {
        const int base = ((bf - kk) << 3) + kk;
        if constexpr (LOGLS == 0) {
          cx2<R>* v = reinterpret_cast<cx2<R>*>(rowp + padidx(base, 1));
#pragma unroll
          for (int q = 0; q < 4; ++q) v[q] = cx2<R>{x[2 * q], x[2 * q + 1]};
        } else if constexpr (LOGLS == 3) {
          E* p = rowp + padidx(base, 1);
#pragma unroll
          for (int q = 0; q < 8; ++q) p[8 * q + 2 * (q >> 1)] = x[q];
        } else {
          E* p = rowp + padidx(base, 1);
          constexpr int LP = Ls + Ls / 8;
#pragma unroll
          for (int q = 0; q < 8; ++q) p[q * LP] = x[q];
        }
      } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) a[m + 2 * q] = x[q];
      }
    }
  }
  if constexpr (S + 1 < Cfg::NS) {
    if constexpr (Cfg::STORE_T && S + 2 == Cfg::NS) {
      // the last stage of a rotating pass reads rows written by other thread groups
      __syncthreads();
      int row2, j2;
      last_stage_map<Cfg>(threadIdx.x, row2, j2);
      fast_stage<Cfg, R, S + 1>(sm, sm + row2 * Cfg::PITCH, j2, sgroup, a, stw, false);
    } else {
      group_sync<Cfg::UPR, Cfg::GS>(sgroup);  // this stage's writes visible to the group
      fast_stage<Cfg, R, S + 1>(sm, rowp, j, sgroup, a, stw, S + 2 < Cfg::NS);
    }
  }
}

// One tile: rows [t0, t0 + T) of (o, b).
template <typename Cfg, typename R, bool MUL = false>
__device__ __forceinline__ void fast_tile(const PassDesc& d, cx<R>* sm, int tile, int tiles_t, int tid, int b) {
  using E = cx<R>;
  constexpr int UPR = Cfg::UPR;
  constexpr bool STORE_T = Cfg::STORE_T;
  const int tt = tile % tiles_t;
  const int o = tile / tiles_t;
  const int t0 = tt << Cfg::LOGT;
  const bool inv = d.inverse != 0;

  const int j = tid & (UPR - 1);
  const int row = tid >> Cfg::LOGUPR;
  E* rowp = sm + row * Cfg::PITCH;
  E a[16];
  {
    const E* __restrict__ src =
        (const E*)d.in + ((long long)o * d.is_o + (long long)b * d.is_b + (long long)(t0 + row) * d.is_t + j);
#pragma unroll
    for (int k = 0; k < 16; ++k) a[k] = src[k * UPR];
  }
  if constexpr (MUL) {
    // fused Fourier-space multiplier (PassDesc::mul_mode), applied to the values as they arrive
    const MulRow<R> mr(d, t0 + row, o, b);
#pragma unroll
    for (int k = 0; k < 16; ++k) a[k] = mr.apply(a[k], j + k * UPR);
  }
  if (inv) {
#pragma unroll
    for (int k = 0; k < 16; ++k) a[k] = cswap(a[k]);
  }
  const E* __restrict__ stw = (const E*)d.tw_stage;  // per-stage twiddle records
  fast_stage<Cfg, R, 0>(sm, rowp, j, tid / Cfg::GS, a, stw, Cfg::NS > 1);

  const R scale = (R)d.scale;
  const bool do_scale = d.scale != 1.0;
  if constexpr (!STORE_T) {
    // After the last stage a[k] is the result for column j + k*M/16: store straight to global memory.
    const OutBase ob = out_base_for(d, o, b);
    const int t = t0 + row;
    const int pt = d.split_axis == 2 ? t / d.Tl : 0;
    const long long toff = ob.off + (long long)(t - pt * d.Tl) * d.os_t;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const int c = j + k * UPR;
      E v = a[k];
      if (inv) v = cswap(v);
      if (do_scale) v = cscale(v, scale);
      const int pc = d.split_axis == 1 ? c / d.Cl : 0;
      store_elem<E>(d, ob.peer + pc + pt, toff + (c - pc * d.Cl), v);
    }
  } else {
    // a[k] now is the result for column j2 + k*M/16 of row row2 (layout of last_stage_map): lanes that
    // hold the same column store neighbouring elements of the destination's fastest axis.
    int row2, j2;
    last_stage_map<Cfg>(tid, row2, j2);
    const OutBase ob = out_base_for(d, o, b);
    const int tg = t0 + row2;
    const int pt = d.split_axis == 2 ? tg / d.Tl : 0;
    const long long toff = ob.off + (long long)(tg - pt * d.Tl) * d.os_t;
    const int logCl = 31 - __clz(d.Cl);
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const int c = j2 + k * UPR;
      int pc = 0, cl = c;
      if (d.split_axis == 1) {
        pc = c >> logCl;
        cl = c & (d.Cl - 1);
      }
      E v = a[k];
      if (inv) v = cswap(v);
      if (do_scale) v = cscale(v, scale);
      store_elem<E>(d, ob.peer + pc + pt, toff + (long long)cl * d.os_c, v);
    }
  }
}

// Out-of-line copy of the tile body for the looping variant: as a real call the body gets the same
// register allocation as the one-tile kernel, and only the loop counters live across it (inlined into
// the loop, the compiler kept addresses of the next iteration live and spilled up to 190 bytes).
template <typename Cfg, typename R>
__device__ __noinline__ void fast_tile_call(const PassDesc& d, cx<R>* sm, int tile, int tiles_t) {
  fast_tile<Cfg, R>(d, sm, tile, tiles_t, threadIdx.x, blockIdx.y);
}

// VARIANT 0: one tile per block.  VARIANT 1: the grid is smaller than the number of tiles
// (PassDesc::grid_limit) and every block walks over several tiles, in launch order; such a pass leaves
// the other SMs to a pass that runs at the same time on another stream.  VARIANT 2: one tile per block with
// the fused input multiplier (a variant of its own so that the plain kernels keep their register allocation).
template <typename R, int LOGM, int LOGT, bool STORE_T, int VARIANT>
__global__ void __launch_bounds__((FastCfg<R, LOGM, LOGT, STORE_T>::NT), (FastCfg<R, LOGM, LOGT, STORE_T>::MINB))
    fft_fast_kernel(const __grid_constant__ PassDesc d) {
  using Cfg = FastCfg<R, LOGM, LOGT, STORE_T>;
  constexpr bool LOOP = VARIANT == 1;
  extern __shared__ __align__(16) unsigned char fast_smem[];
  cx<R>* sm = reinterpret_cast<cx<R>*>(fast_smem);
  if (pass_aborted(d)) return;
  const int tiles_t = d.Tn >> LOGT;
  if constexpr (VARIANT == 2) {
    // The batch entries of a fused pass read the same operand (is_b = 0) and differ only in the multiplier:
    // with the batch as the fastest block index the blocks of one tile run at the same time and the
    // operand comes from DRAM once, from L2 for the others.
    fast_tile<Cfg, R, true>(d, sm, blockIdx.x / d.B, tiles_t, threadIdx.x, blockIdx.x % d.B);
  } else if constexpr (!LOOP) {
    fast_tile<Cfg, R>(d, sm, blockIdx.x, tiles_t, threadIdx.x, blockIdx.y);
  } else {
    const int ntiles = tiles_t * d.On;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
      fast_tile_call<Cfg, R>(d, sm, tile, tiles_t);
      // the next tile's first stage overwrites rows that other threads may still be reading
      __syncthreads();
    }
  }
}

// ---- host side --------------------------------------------------------------------------------------------------
static bool is_pow2(long long v) { return v > 0 && (v & (v - 1)) == 0; }

static bool big_tiles(const PassDesc& d) {
  // Large tiles (128 KiB of data, one block per SM) double the stored run length of rotating
  // passes.  Measured: they pay off when the stores cross NVLink (128-byte runs reach the full
  // peer-store bandwidth) and lose slightly for local passes, so they are the default only there.
  const char* env = std::getenv("JD_B200_BIGTILE");
  if (env && *env) return env[0] != '0';
  if (!d.store_t_contig) return false;
  // local rotating passes: measured 1-2 % slower with large tiles at every length
  return d.npeers > 1;
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
  if (d.fft_mode != JD_FFT_POW2 || d.tw_stage == nullptr) return false;
  if (d.elem_bytes != 8 && d.elem_bytes != 16) return false;
  if (d.M < (d.elem_bytes == 8 ? 128 : 256) || d.M > (d.elem_bytes == 8 ? 4096 : 2048) || d.C != d.M) return false;
  if (d.load_t_contig || d.is_c != 1) return false;
  int logM = 0;
  while ((1 << logM) < d.M) ++logM;
  // the small tile height must divide the rows (the big variant is used only when it divides too)
  const int lt = fast_pass_logT(logM, d.elem_bytes, false);
  if (d.Tn % (1 << lt)) return false;
  if (d.store_t_contig) {
    if (d.os_t != 1) return false;
    if (d.split_axis == 1 && !is_pow2(d.Cl)) return false;
  } else {
    if (d.os_c != 1) return false;
  }
  return true;
}

template <typename R, int LOGM, int LOGT, bool STORE_T>
static int launch_fast_t(const PassDesc& d, cudaStream_t stream) {
  using Cfg = FastCfg<R, LOGM, LOGT, STORE_T>;
  const long long nblocks = (long long)(d.Tn >> LOGT) * d.On;
  if (nblocks * (d.mul_mode != JD_MUL_NONE ? d.B : 1) > 2147483647LL || d.B > 65535) {
    set_last_error("fast pass: grid too large");
    return JD_ERR_INVALID_ARG;
  }
  const bool mul = d.mul_mode != JD_MUL_NONE;
  const bool loop = !mul && d.grid_limit > 0 && d.grid_limit < nblocks;
  const int variant = mul ? 2 : (loop ? 1 : 0);
  auto kern = mul ? fft_fast_kernel<R, LOGM, LOGT, STORE_T, 2>
                  : (loop ? fft_fast_kernel<R, LOGM, LOGT, STORE_T, 1> : fft_fast_kernel<R, LOGM, LOGT, STORE_T, 0>);
  static bool configured[3] = {false, false, false};
  if (!configured[variant]) {
    if (Cfg::SMEM > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
      if (e != cudaSuccess) {
        set_last_error(cudaGetErrorString(e));
        return JD_ERR_CUDA;
      }
    }
    configured[variant] = true;
  }
  const long long grid = loop ? d.grid_limit : nblocks;
  const dim3 blocks = mul ? dim3((unsigned)(nblocks * d.B), 1, 1) : dim3((unsigned)grid, (unsigned)d.B, 1);
  kern<<<blocks, Cfg::NT, Cfg::SMEM, stream>>>(d);
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

// Small tiles (half the rows, twice the resident blocks): the load, compute and store phases of more,
// smaller blocks interleave better.  Measured on plain passes: 1024 points 2.89 -> 2.73 ms per 1024^3
// block (0.97 of the measured copy bandwidth), 512 points 0.386 -> 0.362 ms per 512^3.  Rotating passes
// only gain while the stored runs stay at 128 bytes or more (with 32-byte runs they lose up to 2x).
// JD_B200_SMALLTILE=1/0 forces the choice.
static bool small_tiles(const PassDesc& d, int small_run_bytes) {
  const char* env = std::getenv("JD_B200_SMALLTILE");
  if (env && *env) return env[0] != '0';
  if (!d.store_t_contig) return true;
  return small_run_bytes >= 128;
}

template <typename R, int LOGM>
static int launch_fast_m(const PassDesc& d, cudaStream_t stream) {
  constexpr int budget = sizeof(R) == 4 ? 13 : 12;
  constexpr int cap = sizeof(R) == 4 ? 5 : 4;
  constexpr int LT = TileLog<LOGM, budget, cap>::value;
  constexpr int LTB = TileLog<LOGM, budget + 1, cap>::value;
  constexpr int LTS = TileLog<LOGM, budget - 1, cap>::value;
  if constexpr (LTS != LT && (1 << LTS) * (1 << (LOGM - 4)) >= 64) {
    if (small_tiles(d, (1 << LTS) * 2 * (int)sizeof(R)) && !(big_tiles(d) && d.Tn % (1 << LTB) == 0)) {
      if (d.store_t_contig) return launch_fast_t<R, LOGM, LTS, true>(d, stream);
      return launch_fast_t<R, LOGM, LTS, false>(d, stream);
    }
  }
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
    case 128:
      if constexpr (sizeof(R) == 4) return launch_fast_m<R, 7>(d, stream);
      return JD_ERR_UNSUPPORTED;
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
