// Mixed-radix Stockham transform for lengths N = 2^a 3^b 5^c 7^d 11^e 13^f that
// are not handled by the power-of-two kernels: the stage plan (built on the
// host), the per-butterfly arithmetic shared by the CUDA kernel and the CPU
// emulation, and the emulation's row driver.
//
// A stage of radix r works on N/r butterflies per row.  Butterfly bf reads
// x[bf + q*N/r] (q < r), multiplies by the twiddles w_N^(q * kk * N/(Ls*r)),
// applies an r-point DFT and writes y[(bf/Ls)*Ls*r + kk + q*Ls], where Ls is
// the product of the earlier radices and kk = bf mod Ls.  Source and
// destination are different buffers (ping-pong), so one barrier per stage is
// enough.  Radices are the primes up to 13 and 4, 6, 8, 10, 12, 15, 16; where Ls
// is a power of two bf/Ls is a shift, elsewhere a multiply-high by a reciprocal.
//
// The reference covers such lengths through cuFFT plans (src/csrc/fft.cu:72-121).
#pragma once
#include "fft_radix.h"

#define JD_MIXED_MAX_STAGES 12

namespace jdb {

struct MixedStage {
  int32_t radix;
  int32_t nb;        // butterflies per row: N / radix
  int32_t ls;        // product of the earlier radices
  int32_t ls_log;    // log2(ls) when ls is a power of two, else -1
  int32_t tw_mul;    // N / (ls * radix): twiddle index of butterfly bf is (bf mod ls) * tw_mul
  uint32_t ls_magic; // floor(2^32 / ls) + 1: bf / ls == mulhi(bf, ls_magic) for bf, ls < 2^16
  int32_t rec0;      // index of this stage's first twiddle record (stages >= 1; one record per kk < ls)
};

struct MixedPlan {
  int32_t n;
  int32_t ns;
  int32_t nb_min;    // butterflies per row of the stage with the largest radix
  int32_t nrec;      // twiddle records of all stages: {w, w^2, w^4, w^8} with w = exp(-2 pi i kk tw_mul / n)
  MixedStage st[JD_MIXED_MAX_STAGES];
};

// Stage radices for lengths that profit from composite butterflies (fewer stages, or stages whose
// butterfly counts divide evenly among the threads of a row).  Found by an exhaustive search over the
// factorisations into radices <= 16, scored by padded work per stage plus a fixed cost per stage.
struct MixedRadices {
  int32_t n;
  int32_t r[4];
};
constexpr MixedRadices kMixedRadixTable[] = {
    {96, {12, 8, 0, 0}},    {192, {8, 8, 3, 0}},    {384, {8, 8, 6, 0}},     {1536, {16, 16, 6, 0}},
    {3072, {16, 16, 12, 0}}, {288, {12, 6, 4, 0}},   {576, {12, 12, 4, 0}},   {1152, {12, 12, 8, 0}},
    {2304, {16, 12, 12, 0}}, {160, {16, 10, 0, 0}},  {2560, {16, 16, 10, 0}}, {400, {10, 10, 4, 0}},
    {800, {10, 10, 8, 0}},   {1600, {16, 10, 10, 0}}, {250, {10, 5, 5, 0}},    {500, {10, 10, 5, 0}},
    {1000, {10, 10, 10, 0}}, {2000, {10, 10, 5, 4}}, {240, {16, 15, 0, 0}},   {480, {12, 10, 4, 0}},
    {960, {15, 8, 8, 0}},    {1920, {16, 15, 8, 0}},
};

// The plan for length n; ns == 0 when n has a prime factor above 13, is below 2, or needs too many
// stages.  constexpr so that kernels specialised on the length can fold every stage constant.
constexpr MixedPlan mixed_plan_of(int n) {
  MixedPlan pl{};
  if (n < 2 || n > 65535) return pl;
  int radices[32] = {};
  int ns = 0;
  for (const MixedRadices& e : kMixedRadixTable)
    if (e.n == n)
      for (int i = 0; i < 4 && e.r[i] > 0; ++i) radices[ns++] = e.r[i];
  if (ns == 0) {
    int m = n, a = 0;
    while (m % 2 == 0) {
      m /= 2;
      ++a;
    }
    // power-of-two part: ceil(a/4) stages of nearly equal size, largest first
    if (a > 0) {
      const int k = (a + 3) / 4;
      for (int i = 0; i < k; ++i) {
        const int bits = a / k + (i < a % k ? 1 : 0);
        radices[ns++] = 1 << bits;
      }
    }
    const int primes[5] = {3, 5, 7, 11, 13};
    for (int pi = 0; pi < 5; ++pi) {
      const int p = primes[pi];
      while (m % p == 0) {
        if (ns >= 32) return pl;
        m /= p;
        radices[ns++] = p;
      }
    }
    if (m != 1 || ns > JD_MIXED_MAX_STAGES) return pl;
  }
  pl.n = n;
  pl.ns = ns;
  int ls = 1, rmax = 1, nrec = 0;
  for (int s = 0; s < ns; ++s) {
    pl.st[s].rec0 = nrec;
    if (s > 0) nrec += ls;
    pl.st[s].radix = radices[s];
    pl.st[s].nb = n / radices[s];
    pl.st[s].ls = ls;
    pl.st[s].ls_log = -1;
    for (int l = 0; l < 31; ++l)
      if ((1 << l) == ls) pl.st[s].ls_log = l;
    pl.st[s].tw_mul = n / (ls * radices[s]);
    pl.st[s].ls_magic = ls == 1 ? 0u : (uint32_t)((0x100000000ULL / (unsigned long long)ls) + 1ULL);
    ls *= radices[s];
    if (radices[s] > rmax) rmax = radices[s];
  }
  pl.nb_min = n / rmax;
  pl.nrec = nrec;
  return pl;
}

inline bool make_mixed_plan(int n, MixedPlan* out) {
  const MixedPlan pl = mixed_plan_of(n);
  if (pl.ns == 0) return false;
  *out = pl;
  return true;
}

// Threads per row for tiles of T rows (0: impossible).  Between three quarters of the block size that the
// register budget allows and all of it, the count that wastes the fewest butterfly slots
// (sum over stages of ceil(nb / tpr) * tpr / nb); ties go to the larger count.
constexpr int mixed_threads_per_row(const MixedPlan& pl, int T, int elem_bytes) {
  const int cap = elem_bytes == 8 ? 512 : 256;
  int hi = cap / T;
  if (hi < 1 || pl.ns < 1) return 0;
  int nbmax = 1;
  for (int s = 0; s < pl.ns; ++s)
    if (pl.st[s].nb > nbmax) nbmax = pl.st[s].nb;
  if (hi > nbmax) hi = nbmax;
  int lo = (3 * cap / 4 + T - 1) / T;
  if (lo > hi) lo = hi;
  if (lo < 1) lo = 1;
  int best = hi;
  long long best_cost = -1;
  for (int tpr = hi; tpr >= lo; --tpr) {
    long long cost = 0;
    for (int s = 0; s < pl.ns; ++s) {
      const int nb = pl.st[s].nb;
      cost += (long long)((nb + tpr - 1) / tpr) * tpr * 65536 / nb;
    }
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = tpr;
    }
  }
  return best;
}

// Geometry rules of the length-specialised kernels (fft_mixed_static.h); ops/passes.py::choose_tiling applies
// the same ones, and the launcher falls back to the generic kernel when a descriptor was tiled differently.  The tile height follows from the shared-memory
// budget with the pitch of tall tiles; the final pitch then makes the reads of the last stage of a rotating
// pass conflict-free: the threads of one shared-memory wavefront (16 lanes of 8-byte elements, 8 lanes of
// 16-byte ones) cover RH = min(T, 8) rows x CB columns, which needs pitch == CB modulo the wavefront width.
constexpr int mixed_rowlen(int n) { return n + 2 * ((n + 15) / 16); }
constexpr int mixed_pitch_mod(int rowlen, int want, int mod) { return rowlen + (((want - rowlen) % mod) + mod) % mod; }
constexpr int mixed_static_T(int n, int elem_bytes, bool store_t) {
  const int pitch = elem_bytes == 8 ? mixed_pitch_mod(mixed_rowlen(n), 2, 16) : mixed_pitch_mod(mixed_rowlen(n), 1, 8);
  int T = 1;
  while (T < 32 && 2 * (2 * T) * pitch * elem_bytes <= 110 * 1024) T *= 2;
  if (store_t)
    while (T * elem_bytes < 64 && 2 * (2 * T) * pitch * elem_bytes <= 220 * 1024) T *= 2;
  return T;
}
constexpr int mixed_static_pitch(int n, int elem_bytes, int T) {
  const int lanes = elem_bytes == 8 ? 16 : 8;
  const int rh = T < 8 ? T : 8;
  return mixed_pitch_mod(mixed_rowlen(n), lanes / rh, lanes);
}

// Thread layout of the last stage of a rotating pass in the specialised kernels: the threads of one
// shared-memory wavefront cover RH = min(T, 8) consecutive rows x CB = lanes/RH consecutive butterfly indices.
constexpr int mixed_last_stage_row(int T, int elem_bytes, int tid) {
  const int lanes = elem_bytes == 8 ? 16 : 8;
  const int rh = T < 8 ? T : 8;
  return tid % rh + rh * ((tid / lanes) % (T / rh));
}
constexpr int mixed_last_stage_j(int T, int elem_bytes, int tid) {
  const int lanes = elem_bytes == 8 ? 16 : 8;
  const int rh = T < 8 ? T : 8;
  const int cb = lanes / rh;
  return cb * ((tid / lanes) / (T / rh)) + (tid / rh) % cb;
}

JD_HD uint32_t jd_mulhi(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
  return __umulhi(a, b);
#else
  return (uint32_t)(((uint64_t)a * (uint64_t)b) >> 32);
#endif
}

// Twiddle + DFT of one butterfly held in a[]; returns the index of output 0
// (output q goes to that index + q * st.ls).
// `tws`: the per-stage twiddle records, or null (then the table `tw` of n roots is used).
template <typename R, int RADIX>
JD_HD int mixed_butterfly(const MixedStage& st, const cx<R>* tw, const cx<R>* tws, int bf, cx<R> (&a)[RADIX]) {
  int kk = 0, blk = bf;
  if (st.ls > 1) {
    if (st.ls_log >= 0) {
      kk = bf & (st.ls - 1);
      blk = bf >> st.ls_log;
    } else {
      blk = (int)jd_mulhi((uint32_t)bf, st.ls_magic);
      kk = bf - blk * st.ls;
    }
    if (tws != nullptr)
      twiddle_record<R, RADIX>(tws + 4 * (st.rec0 + kk), a);
    else
      twiddle_powers<R, RADIX>(tw, kk * st.tw_mul, a);
  }
  dft_any<R, RADIX>(a);
  return blk * st.ls * RADIX + kk;
}

// One stage on one row, smem/host buffer to buffer (both in the padded layout of padidx).
template <typename R, int RADIX>
JD_HD void mixed_stage_row(const MixedStage& st, const cx<R>* tw, const cx<R>* tws, const cx<R>* src, cx<R>* dst,
                           int first, int step) {
  for (int bf = first; bf < st.nb; bf += step) {
    cx<R> a[RADIX];
#pragma unroll
    for (int q = 0; q < RADIX; ++q) a[q] = src[padidx(bf + q * st.nb, 1)];
    const int base = mixed_butterfly<R, RADIX>(st, tw, tws, bf, a);
#pragma unroll
    for (int q = 0; q < RADIX; ++q) dst[padidx(base + q * st.ls, 1)] = a[q];
  }
}

// Calls f.template run<RADIX>() for the stage's radix.
template <typename F>
JD_HD void mixed_dispatch(int radix, F&& f) {
  switch (radix) {
    case 2: f.template run<2>(); break;
    case 3: f.template run<3>(); break;
    case 4: f.template run<4>(); break;
    case 5: f.template run<5>(); break;
    case 6: f.template run<6>(); break;
    case 7: f.template run<7>(); break;
    case 8: f.template run<8>(); break;
    case 10: f.template run<10>(); break;
    case 11: f.template run<11>(); break;
    case 12: f.template run<12>(); break;
    case 13: f.template run<13>(); break;
    case 15: f.template run<15>(); break;
    case 16: f.template run<16>(); break;
    default: break;
  }
}

}  // namespace jdb
