// Register-resident butterflies beyond radix 8: the 16-point DFT of the
// specialised power-of-two kernel, prime-length DFTs (3, 5, 7, 11, 13) and small
// composite ones (6, 10, 12, 15) for the mixed-radix kernel, and the
// in-register twiddle multiplication they share.
// Only the forward direction exp(-2*pi*i*..) exists; callers obtain the
// inverse by swapping real and imaginary parts on the way in and out.
// The reference leaves all of this to cuFFT (src/csrc/fft.cu:72-121).
#pragma once
#include "fft_core.h"

namespace jdb {

// ---- constants evaluated by the compiler -----------------------------------------------------------------
// cos / sin of 2*pi*num/den, by Taylor series after reduction to [-pi, pi]
constexpr double jd_sincos_2pi(int num, int den, bool want_sin) {
  num %= den;
  double x = 6.283185307179586476925286766559 * (double)num / (double)den;
  if (x > 3.14159265358979323846264338327950288) x -= 6.283185307179586476925286766559;
  const double x2 = x * x;
  double term = want_sin ? x : 1.0, sum = term;
  for (int k = want_sin ? 1 : 0; k < 40; k += 2) {
    term *= -x2 / (double)((k + 1) * (k + 2));
    sum += term;
  }
  return sum;
}

// a * exp(-2 pi i K / 16), trivial cases resolved at compile time
template <typename R, int K>
JD_HD cx<R> mulw16(cx<R> a) {
  constexpr int k = K & 15;
  constexpr R c1 = (R)0.92387953251128673848, s1 = (R)0.38268343236508978178, h = (R)0.70710678118654752440;
  if constexpr (k == 0) {
    return a;
  } else if constexpr (k == 4) {
    return cx<R>{a.y, -a.x};
  } else if constexpr (k == 8) {
    return cx<R>{-a.x, -a.y};
  } else if constexpr (k == 12) {
    return cx<R>{-a.y, a.x};
  } else if constexpr (k == 2) {
    return cx<R>{(a.x + a.y) * h, (a.y - a.x) * h};
  } else if constexpr (k == 6) {
    return cx<R>{(a.y - a.x) * h, -(a.x + a.y) * h};
  } else if constexpr (k == 10) {
    return cx<R>{-(a.x + a.y) * h, (a.x - a.y) * h};
  } else if constexpr (k == 14) {
    return cx<R>{(a.x - a.y) * h, (a.x + a.y) * h};
  } else {
    // W = wr + i wi with wr = cos(pi k / 8), wi = -sin(pi k / 8)
    constexpr R wr = (k == 1 || k == 15) ? c1 : (k == 3 || k == 13) ? s1 : (k == 5 || k == 11) ? -s1 : -c1;
    constexpr R wi = (k == 1 || k == 7) ? -s1 : (k == 3 || k == 5) ? -c1 : (k == 9 || k == 15) ? s1 : c1;
    return cx<R>{a.x * wr - a.y * wi, a.x * wi + a.y * wr};
  }
}

// 16-point DFT in registers, natural order in and out (4 x 4 decomposition):
// X[k1 + 4 k2] = sum_n W16^(n k1) W4^(n k2) sum_m x[n + 4 m] W4^(m k1)
template <typename R>
JD_HD void dft16(cx<R> (&a)[16]) {
#pragma unroll
  for (int n = 0; n < 4; ++n) dft4(a[n], a[n + 4], a[n + 8], a[n + 12]);  // a[n + 4 k1] = y_n[k1]
  a[1 + 4] = mulw16<R, 1>(a[1 + 4]); a[1 + 8] = mulw16<R, 2>(a[1 + 8]); a[1 + 12] = mulw16<R, 3>(a[1 + 12]);
  a[2 + 4] = mulw16<R, 2>(a[2 + 4]); a[2 + 8] = mulw16<R, 4>(a[2 + 8]); a[2 + 12] = mulw16<R, 6>(a[2 + 12]);
  a[3 + 4] = mulw16<R, 3>(a[3 + 4]); a[3 + 8] = mulw16<R, 6>(a[3 + 8]); a[3 + 12] = mulw16<R, 9>(a[3 + 12]);
  // second layer over n for each k1: inputs a[n + 4 k1], outputs X[k1 + 4 k2]
  cx<R> t[16];
#pragma unroll
  for (int k1 = 0; k1 < 4; ++k1) {
    cx<R> x0 = a[4 * k1], x1 = a[4 * k1 + 1], x2 = a[4 * k1 + 2], x3 = a[4 * k1 + 3];
    dft4(x0, x1, x2, x3);
    t[k1] = x0; t[k1 + 4] = x1; t[k1 + 8] = x2; t[k1 + 12] = x3;
  }
#pragma unroll
  for (int k = 0; k < 16; ++k) a[k] = t[k];
}

// ---- prime lengths ---------------------------------------------------------------------------------------------
// With s_k = x_k + x_{P-k} and d_k = x_k - x_{P-k} (k = 1..H, H = (P-1)/2):
//   X_m     = x_0 + sum_k cos(2 pi m k / P) s_k  -  i sum_k sin(2 pi m k / P) d_k
//   X_{P-m} = x_0 + sum_k cos(2 pi m k / P) s_k  +  i sum_k sin(2 pi m k / P) d_k
template <typename R, int P, int M, int K>
JD_HD void prime_term(cx<R>& re, cx<R>& im, const cx<R>* s, const cx<R>* d) {
  constexpr R c = (R)jd_sincos_2pi(M * K, P, false);
  constexpr R sn = (R)jd_sincos_2pi(M * K, P, true);
  re.x += c * s[K - 1].x;
  re.y += c * s[K - 1].y;
  im.x += sn * d[K - 1].x;
  im.y += sn * d[K - 1].y;
}

template <typename R, int P, int M, int K = 1>
JD_HD void prime_row(cx<R>& re, cx<R>& im, const cx<R>* s, const cx<R>* d) {
  prime_term<R, P, M, K>(re, im, s, d);
  if constexpr (K < (P - 1) / 2) prime_row<R, P, M, K + 1>(re, im, s, d);
}

template <typename R, int P, int M = 1>
JD_HD void prime_rows(cx<R> x0, const cx<R>* s, const cx<R>* d, cx<R>* a) {
  cx<R> re = x0, im = cx<R>{(R)0, (R)0};
  prime_row<R, P, M>(re, im, s, d);
  a[M] = cx<R>{re.x + im.y, re.y - im.x};
  a[P - M] = cx<R>{re.x - im.y, re.y + im.x};
  if constexpr (M < (P - 1) / 2) prime_rows<R, P, M + 1>(x0, s, d, a);
}

template <typename R, int P>
JD_HD void dft_prime(cx<R> (&a)[P]) {
  constexpr int H = (P - 1) / 2;
  cx<R> s[H], d[H];
#pragma unroll
  for (int k = 0; k < H; ++k) {
    s[k] = cadd(a[k + 1], a[P - 1 - k]);
    d[k] = csub(a[k + 1], a[P - 1 - k]);
  }
  const cx<R> x0 = a[0];
  cx<R> sum = x0;
#pragma unroll
  for (int k = 0; k < H; ++k) sum = cadd(sum, s[k]);
  prime_rows<R, P>(x0, s, d, a);
  a[0] = sum;
}

template <typename R, int RADIX>
JD_HD void dft_any(cx<R> (&a)[RADIX]);

// ---- composite lengths (6, 10, 12, 15) ---------------------------------------------------------------
// a * exp(-2 pi i NUM / DEN) with the constant folded by the compiler
template <typename R, int NUM, int DEN>
JD_HD cx<R> mul_root(cx<R> a) {
  constexpr int k = NUM % DEN;
  if constexpr (k == 0) {
    return a;
  } else if constexpr (4 * k == DEN) {
    return cx<R>{a.y, -a.x};
  } else if constexpr (2 * k == DEN) {
    return cx<R>{-a.x, -a.y};
  } else if constexpr (4 * k == 3 * DEN) {
    return cx<R>{-a.y, a.x};
  } else {
    constexpr R c = (R)jd_sincos_2pi(k, DEN, false), s = (R)jd_sincos_2pi(k, DEN, true);
    return cx<R>{a.x * c + a.y * s, a.y * c - a.x * s};
  }
}

template <typename R, int A, int B, int N_, int K1>
JD_HD void comp_twiddle(cx<R> (&t)[A]) {
  t[K1] = mul_root<R, N_ * K1, A * B>(t[K1]);
  if constexpr (K1 + 1 < A) comp_twiddle<R, A, B, N_, K1 + 1>(t);
}

// first layer of an (A x B)-point DFT on x[n + B m]: A-point DFTs over m for column n, then W_AB^(n k1)
template <typename R, int A, int B, int N_>
JD_HD void comp_columns(cx<R> (&a)[A * B]) {
  cx<R> t[A];
#pragma unroll
  for (int m = 0; m < A; ++m) t[m] = a[N_ + B * m];
  dft_any<R, A>(t);
  if constexpr (N_ > 0) comp_twiddle<R, A, B, N_, 1>(t);
#pragma unroll
  for (int k1 = 0; k1 < A; ++k1) a[N_ + B * k1] = t[k1];
  if constexpr (N_ + 1 < B) comp_columns<R, A, B, N_ + 1>(a);
}

// X[k1 + A k2] = sum_n W_B^(n k2) W_AB^(n k1) sum_m x[n + B m] W_A^(m k1)
template <typename R, int A, int B>
JD_HD void dft_composite(cx<R> (&a)[A * B]) {
  comp_columns<R, A, B, 0>(a);
  cx<R> out[A * B];
#pragma unroll
  for (int k1 = 0; k1 < A; ++k1) {
    cx<R> t[B];
#pragma unroll
    for (int n = 0; n < B; ++n) t[n] = a[n + B * k1];
    dft_any<R, B>(t);
#pragma unroll
    for (int k2 = 0; k2 < B; ++k2) out[k1 + A * k2] = t[k2];
  }
#pragma unroll
  for (int k = 0; k < A * B; ++k) a[k] = out[k];
}

// DFT of RADIX values held in registers, natural order in and out
template <typename R, int RADIX>
JD_HD void dft_any(cx<R> (&a)[RADIX]) {
  if constexpr (RADIX == 6) {
    dft_composite<R, 2, 3>(a);
  } else if constexpr (RADIX == 10) {
    dft_composite<R, 2, 5>(a);
  } else if constexpr (RADIX == 12) {
    dft_composite<R, 4, 3>(a);
  } else if constexpr (RADIX == 15) {
    dft_composite<R, 3, 5>(a);
  } else if constexpr (RADIX == 2) {
    dft2(a[0], a[1]);
  } else if constexpr (RADIX == 4) {
    dft4(a[0], a[1], a[2], a[3]);
  } else if constexpr (RADIX == 8) {
    dft8(a);
  } else if constexpr (RADIX == 16) {
    dft16(a);
  } else {
    dft_prime<R, RADIX>(a);
  }
}

// ---- twiddles -------------------------------------------------------------------------------------------------
template <typename R>
JD_HD cx<R> tw_load(const cx<R>* p) {
#if defined(__CUDA_ARCH__)
  if constexpr (sizeof(R) == 4) {
    const float2 v = __ldg(reinterpret_cast<const float2*>(p));
    return cx<R>{v.x, v.y};
  } else {
    const double2 v = __ldg(reinterpret_cast<const double2*>(p));
    return cx<R>{v.x, v.y};
  }
#else
  return *p;
#endif
}

// a[q] *= w^q for q = 1..RADIX-1 given w, w^2, w^4 and w^8 (only those below RADIX are used); the
// other powers are products of them.
template <typename R, int RADIX>
JD_HD void twiddle_apply(cx<R> w1, cx<R> w2, cx<R> w4, cx<R> w8, cx<R> (&a)[RADIX]) {
  cx<R> w[RADIX < 8 ? RADIX : 8];
  w[1] = w1;
  a[1] = cmul(a[1], w[1]);
  if constexpr (RADIX > 2) {
    w[2] = w2;
    a[2] = cmul(a[2], w[2]);
  }
  if constexpr (RADIX > 3) {
    w[3] = cmul(w[1], w[2]);
    a[3] = cmul(a[3], w[3]);
  }
  if constexpr (RADIX > 4) {
    w[4] = w4;
    a[4] = cmul(a[4], w[4]);
  }
  if constexpr (RADIX > 5) {
    w[5] = cmul(w[1], w[4]);
    a[5] = cmul(a[5], w[5]);
  }
  if constexpr (RADIX > 6) {
    w[6] = cmul(w[2], w[4]);
    a[6] = cmul(a[6], w[6]);
  }
  if constexpr (RADIX > 7) {
    w[7] = cmul(w[3], w[4]);
    a[7] = cmul(a[7], w[7]);
  }
  if constexpr (RADIX > 8) {
    a[8] = cmul(a[8], w8);
#pragma unroll
    for (int q = 9; q < RADIX; ++q) a[q] = cmul(a[q], cmul(w[q - 8], w8));
  }
}

// Twiddles from the table of N roots: w = tw[ti]; w^2, w^4, w^8 are read from the table as well (the
// caller guarantees (RADIX-1)*ti < table length).
template <typename R, int RADIX>
JD_HD void twiddle_powers(const cx<R>* tw, int ti, cx<R> (&a)[RADIX]) {
  const cx<R> w1 = tw_load(tw + ti);
  cx<R> w2 = w1, w4 = w1, w8 = w1;
  if constexpr (RADIX > 2) w2 = tw_load(tw + 2 * ti);
  if constexpr (RADIX > 4) w4 = tw_load(tw + 4 * ti);
  if constexpr (RADIX > 8) w8 = tw_load(tw + 8 * ti);
  twiddle_apply<R, RADIX>(w1, w2, w4, w8, a);
}

// Twiddles from a per-stage record {w, w^2, w^4, w^8} (32 bytes for complex64, read as two 16-byte words):
// the records of consecutive butterflies are contiguous, so a warp's reads coalesce.
template <typename R, int RADIX>
JD_HD void twiddle_record(const cx<R>* rec, cx<R> (&a)[RADIX]) {
  cx<R> w1, w2, w4, w8;
#if defined(__CUDA_ARCH__)
  if constexpr (sizeof(R) == 4) {
    const float4 lo = __ldg(reinterpret_cast<const float4*>(rec));
    w1 = cx<R>{lo.x, lo.y};
    w2 = cx<R>{lo.z, lo.w};
    w4 = w1;
    w8 = w1;
    if constexpr (RADIX > 4) {
      const float4 hi = __ldg(reinterpret_cast<const float4*>(rec) + 1);
      w4 = cx<R>{hi.x, hi.y};
      w8 = cx<R>{hi.z, hi.w};
    }
  } else {
    w1 = tw_load(rec);
    w2 = tw_load(rec + 1);
    w4 = w1;
    w8 = w1;
    if constexpr (RADIX > 4) w4 = tw_load(rec + 2);
    if constexpr (RADIX > 8) w8 = tw_load(rec + 3);
  }
#else
  w1 = rec[0];
  w2 = rec[1];
  w4 = rec[2];
  w8 = rec[3];
#endif
  twiddle_apply<R, RADIX>(w1, w2, w4, w8, a);
}

}  // namespace jdb
