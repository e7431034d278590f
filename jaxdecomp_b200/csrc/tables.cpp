// Constant tables for the FFT kernels, computed once on the host in extended
// precision and cached per (length, element size, memory space):
//   twiddle[n] = exp(-2*pi*i*n/M), n < M
//   tw_stage   = per-stage records {w, w^2, w^4, w^8} of the specialised power-of-two kernel (fft_fast_plan.h)
//   chirp[n]   = exp(-i*pi*n^2/C), n < C                      (Bluestein)
//   bhat[m]    = FFT_M(b)[m] / M with b[m] = b[M-m] = conj(chirp[m]), m < C   (Bluestein)
// The reference keeps cuFFT plans in its descriptor manager for the same
// purpose (src/csrc/grid_descriptor_mgr.cc:29-66).
#include <cuda_runtime.h>

#include <cmath>
#include <complex>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include <tuple>
#include <vector>

#include "fft_fast_plan.h"
#include "fft_mixed.h"
#include "runtime.h"

namespace jdb {

using cld = std::complex<long double>;
static const long double kPi = 3.141592653589793238462643383279502884L;

static void host_fft_pow2(std::vector<cld>& a) {
  const size_t n = a.size();
  for (size_t i = 1, j = 0; i < n; ++i) {
    size_t bit = n >> 1;
    for (; j & bit; bit >>= 1) j ^= bit;
    j ^= bit;
    if (i < j) std::swap(a[i], a[j]);
  }
  for (size_t len = 2; len <= n; len <<= 1) {
    std::vector<cld> w(len / 2);
    for (size_t k = 0; k < len / 2; ++k) {
      const long double ang = -2.0L * kPi * (long double)k / (long double)len;
      w[k] = cld(cosl(ang), sinl(ang));
    }
    for (size_t i = 0; i < n; i += len)
      for (size_t k = 0; k < len / 2; ++k) {
        const cld u = a[i + k], v = a[i + k + len / 2] * w[k];
        a[i + k] = u + v;
        a[i + k + len / 2] = u - v;
      }
  }
}

static void* upload(const std::vector<cld>& v, int elem_bytes, bool device) {
  const size_t n = v.size();
  std::vector<unsigned char> raw(n * (size_t)elem_bytes);
  if (elem_bytes == 8) {
    float* p = reinterpret_cast<float*>(raw.data());
    for (size_t i = 0; i < n; ++i) {
      p[2 * i] = (float)v[i].real();
      p[2 * i + 1] = (float)v[i].imag();
    }
  } else {
    double* p = reinterpret_cast<double*>(raw.data());
    for (size_t i = 0; i < n; ++i) {
      p[2 * i] = (double)v[i].real();
      p[2 * i + 1] = (double)v[i].imag();
    }
  }
  void* out = nullptr;
  if (device) {
    if (cudaMalloc(&out, raw.size()) != cudaSuccess) throw std::runtime_error("tables: cudaMalloc failed");
    if (cudaMemcpy(out, raw.data(), raw.size(), cudaMemcpyHostToDevice) != cudaSuccess)
      throw std::runtime_error("tables: cudaMemcpy failed");
  } else {
    out = std::malloc(raw.size());
    std::memcpy(out, raw.data(), raw.size());
  }
  return out;
}

struct TableSet {
  int ordinal = -1;  // GPU that owns the device copies
  void* twiddle = nullptr;
  void* tw_stage = nullptr;
  void* chirp = nullptr;
  void* bhat = nullptr;
  bool device = false;
};

static std::mutex g_mu;
// (C, M, elem_bytes, device ordinal or -1 for host tables): device tables live in the memory of the GPU that
// was current when they were built, so every GPU of a multi-device process gets its own set
static std::map<std::tuple<int, int, int, int>, TableSet> g_tables;

FftTables get_fft_tables(int C, int M, int elem_bytes, bool device) {
  if (elem_bytes != 8 && elem_bytes != 16) throw std::runtime_error("tables: complex64/complex128 only");
  // a table of M roots alone (mixed-radix transforms) may have any length; Bluestein needs a power of two
  if (C != M && (M < 8 || (M & (M - 1)))) throw std::runtime_error("tables: M must be a power of two >= 8");
  if (M < 1) throw std::runtime_error("tables: empty table");
  std::lock_guard<std::mutex> lk(g_mu);
  int ordinal = -1;
  if (device && cudaGetDevice(&ordinal) != cudaSuccess) {
    cudaGetLastError();
    throw std::runtime_error("tables: no current CUDA device");
  }
  auto key = std::make_tuple(C, M, elem_bytes, ordinal);
  auto it = g_tables.find(key);
  if (it == g_tables.end()) {
    TableSet ts;
    ts.device = device;
    ts.ordinal = ordinal;
    std::vector<cld> tw(M);
    for (int n = 0; n < M; ++n) {
      const long double ang = -2.0L * kPi * (long double)n / (long double)M;
      tw[n] = cld(cosl(ang), sinl(ang));
    }
    ts.twiddle = upload(tw, elem_bytes, device);
    int logm = 0;
    while ((1 << logm) < M) ++logm;
    if (C == M && (1 << logm) == M && logm >= kFastMinLog && logm <= kFastMaxLog) {
      // records {w, w^2, w^4, w^8} per stage >= 1 and kk < Ls, w = exp(-2 pi i kk / (Ls * radix))
      std::vector<cld> rec((size_t)plan_stage_records(logm) * 4);
      for (int s = 1; s < plan_num_stages(logm); ++s) {
        const int ls = 1 << plan_log_ls(logm, s);
        const int span = ls << plan_radix_log(logm, s);
        for (int kk = 0; kk < ls; ++kk)
          for (int p = 0; p < 4; ++p) {
            const long double ang = -2.0L * kPi * (long double)(kk << p) / (long double)span;
            rec[((size_t)plan_stage_record0(logm, s) + kk) * 4 + p] = cld(cosl(ang), sinl(ang));
          }
      }
      ts.tw_stage = upload(rec, elem_bytes, device);
    } else if (C == M) {
      // mixed-radix plan: records {w, w^2, w^4, w^8} per stage >= 1 and kk < ls, w = exp(-2 pi i kk tw_mul / M)
      const MixedPlan pl = mixed_plan_of(M);
      if (pl.ns > 0 && pl.nrec > 0) {
        std::vector<cld> rec((size_t)pl.nrec * 4);
        for (int s = 1; s < pl.ns; ++s)
          for (int kk = 0; kk < pl.st[s].ls; ++kk)
            for (int p = 0; p < 4; ++p) {
              const long long e = ((long long)kk * pl.st[s].tw_mul * (1LL << p)) % M;
              const long double ang = -2.0L * kPi * (long double)e / (long double)M;
              rec[((size_t)pl.st[s].rec0 + kk) * 4 + p] = cld(cosl(ang), sinl(ang));
            }
        ts.tw_stage = upload(rec, elem_bytes, device);
      }
    }
    if (C != M) {
      if (M < 2 * C - 1) throw std::runtime_error("tables: Bluestein length too short");
      std::vector<cld> chirp(C), b(M, cld(0, 0));
      for (int n = 0; n < C; ++n) {
        const long long r = ((long long)n * n) % (2LL * C);  // exact reduction of n^2 mod 2C
        const long double ang = -kPi * (long double)r / (long double)C;
        chirp[n] = cld(cosl(ang), sinl(ang));
      }
      for (int n = 0; n < C; ++n) {
        b[n] = std::conj(chirp[n]);
        if (n) b[M - n] = std::conj(chirp[n]);
      }
      host_fft_pow2(b);
      for (auto& z : b) z /= (long double)M;
      ts.chirp = upload(chirp, elem_bytes, device);
      ts.bhat = upload(b, elem_bytes, device);
    }
    it = g_tables.emplace(key, ts).first;
  }
  FftTables out;
  out.twiddle = it->second.twiddle;
  out.tw_stage = it->second.tw_stage;
  out.chirp = it->second.chirp;
  out.bhat = it->second.bhat;
  return out;
}

void clear_fft_tables() {
  std::lock_guard<std::mutex> lk(g_mu);
  int cur = -1;
  cudaGetDevice(&cur);
  for (auto& kv : g_tables) {
    TableSet& ts = kv.second;
    if (ts.device && ts.ordinal >= 0) cudaSetDevice(ts.ordinal);
    for (void* p : {ts.twiddle, ts.tw_stage, ts.chirp, ts.bhat}) {
      if (!p) continue;
      if (ts.device)
        cudaFree(p);
      else
        std::free(p);
    }
  }
  g_tables.clear();
  if (cur >= 0) cudaSetDevice(cur);
  cudaGetLastError();
}

}  // namespace jdb
