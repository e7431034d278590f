// In-place Stockham FFT on rows held in fast memory (shared memory on the GPU,
// ordinary memory in the CPU emulation).
//
// A row of M = 2^L complex values (M >= 8) is transformed by ceil(L/3) stages.
// In every stage a work item j in [0, M/8) owns the eight values
// row[j + k*M/8], k = 0..7.  A radix-8 stage applies one 8-point DFT to them;
// a radix-4 (radix-2) stage applies two (four) smaller DFTs to interleaved
// subsets of the same eight values, so the register footprint and the access
// pattern are identical for all radices.  Results are written back in
// autosorted (Stockham) order, so no bit reversal is needed; all reads of a
// stage must complete before its writes (one barrier in between).
//
// Only the forward direction exp(-2*pi*i*..) is implemented: the inverse is
// obtained by swapping real and imaginary parts on the way in and out.
//
// This replaces the batched 1-D cuFFT plans of the reference
// (src/csrc/fft.cu:72-121).  The code is shared by the CUDA kernels and by the
// CPU emulation that the unit tests use.
#pragma once
#include "tile_map.h"

namespace jdb {

template <typename R>
struct alignas(2 * sizeof(R)) cx {
  R x, y;
};

template <typename R>
JD_HD cx<R> cadd(cx<R> a, cx<R> b) { return cx<R>{a.x + b.x, a.y + b.y}; }
template <typename R>
JD_HD cx<R> csub(cx<R> a, cx<R> b) { return cx<R>{a.x - b.x, a.y - b.y}; }
template <typename R>
JD_HD cx<R> cmul(cx<R> a, cx<R> b) { return cx<R>{a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x}; }
template <typename R>
JD_HD cx<R> cswap(cx<R> a) { return cx<R>{a.y, a.x}; }
template <typename R>
JD_HD cx<R> cscale(cx<R> a, R s) { return cx<R>{a.x * s, a.y * s}; }
// multiply by -i
template <typename R>
JD_HD cx<R> cmul_mi(cx<R> a) { return cx<R>{a.y, -a.x}; }

template <typename R>
JD_HD void dft2(cx<R>& a, cx<R>& b) {
  cx<R> t = a;
  a = cadd(t, b);
  b = csub(t, b);
}

// natural order in, natural order out
template <typename R>
JD_HD void dft4(cx<R>& x0, cx<R>& x1, cx<R>& x2, cx<R>& x3) {
  cx<R> p0 = cadd(x0, x2), q0 = csub(x0, x2);
  cx<R> p1 = cadd(x1, x3), q1 = cmul_mi(csub(x1, x3));
  x0 = cadd(p0, p1);
  x2 = csub(p0, p1);
  x1 = cadd(q0, q1);
  x3 = csub(q0, q1);
}

template <typename R>
JD_HD void dft8(cx<R> a[8]) {
  const R h = (R)0.70710678118654752440;
  cx<R> s0 = cadd(a[0], a[4]), d0 = csub(a[0], a[4]);
  cx<R> s1 = cadd(a[1], a[5]), d1 = csub(a[1], a[5]);
  cx<R> s2 = cadd(a[2], a[6]), d2 = cmul_mi(csub(a[2], a[6]));
  cx<R> s3 = cadd(a[3], a[7]), d3 = csub(a[3], a[7]);
  // d1 *= (1 - i)/sqrt2 ; d3 *= (-1 - i)/sqrt2
  d1 = cx<R>{(d1.x + d1.y) * h, (d1.y - d1.x) * h};
  d3 = cx<R>{(d3.y - d3.x) * h, -(d3.x + d3.y) * h};
  dft4(s0, s1, s2, s3);
  dft4(d0, d1, d2, d3);
  a[0] = s0; a[2] = s1; a[4] = s2; a[6] = s3;
  a[1] = d0; a[3] = d1; a[5] = d2; a[7] = d3;
}

// Number of stages and the radix of stage s for M = 2^logM (logM >= 3):
// radix-8 stages first, then one radix-4 or radix-2 stage if needed.
JD_HD int fft_num_stages(int logM) { return (logM + 2) / 3; }
JD_HD int fft_stage_radix_log(int logM, int s) {
  const int n8 = logM / 3;
  return s < n8 ? 3 : (logM - 3 * n8);
}

// Column index -> position inside a shared-memory row.  With `pad` set, two
// unused slots follow every 16 columns.  This makes all three exchange
// patterns of the radix-8 stages free of bank conflicts for 8-byte elements:
// eight consecutive outputs per thread (first stage, written as 16-byte
// vectors), stride-8 groups (second stage) and unit stride (reads, later stages).
JD_HD int padidx(int n, int pad) { return pad ? n + ((n >> 4) << 1) : n; }
JD_HD int padded_row_length(int M, int pad) { return pad ? M + (((M + 15) >> 4) << 1) : M; }

template <typename R>
JD_HD void stage_read(const cx<R>* row, int M, int j, cx<R> a[8], int pad) {
  const int q = M >> 3;
  if (pad) {  // q is a multiple of 16 here, so the padded offset is linear in k
    const cx<R>* p = row + padidx(j, 1);
    const int qp = q + (q >> 3);
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = p[k * qp];
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = row[j + k * q];
  }
}

template <typename R>
struct alignas(4 * sizeof(R)) cx2 {
  cx<R> a, b;
};

// Ls = 2^logLs: length of the sub-transforms already done (product of earlier radices).
// tw: table of M roots exp(-2*pi*i*n/M).
template <typename R>
JD_HD void stage_compute_write(cx<R>* row, int logM, int j, int logLs, int radix_log, const cx<R>* tw, cx<R> a[8],
                               int pad) {
  const int M = 1 << logM;
  const int Ls = 1 << logLs;
  const int q8 = M >> 3;
  if (radix_log == 3) {
    const int kk = j & (Ls - 1);
    if (logLs > 0) {
      const int ti = kk << (logM - logLs - 3);
      const cx<R> w1 = tw[ti], w2 = tw[2 * ti], w4 = tw[4 * ti];
      const cx<R> w3 = cmul(w1, w2), w5 = cmul(w1, w4), w6 = cmul(w2, w4);
      const cx<R> w7 = cmul(w3, w4);
      a[1] = cmul(a[1], w1); a[2] = cmul(a[2], w2); a[3] = cmul(a[3], w3); a[4] = cmul(a[4], w4);
      a[5] = cmul(a[5], w5); a[6] = cmul(a[6], w6); a[7] = cmul(a[7], w7);
    }
    dft8(a);
    const int base = ((j - kk) << 3) + kk;
    if (!pad) {
#pragma unroll
      for (int k = 0; k < 8; ++k) row[base + (k << logLs)] = a[k];
    } else if (logLs == 0) {
      // eight consecutive columns inside one 16-column group: four 2-element vector stores
      cx2<R>* p = reinterpret_cast<cx2<R>*>(row + padidx(base, 1));
#pragma unroll
      for (int k = 0; k < 4; ++k) p[k] = cx2<R>{a[2 * k], a[2 * k + 1]};
    } else if (logLs == 3) {
      cx<R>* p = row + padidx(base, 1);
#pragma unroll
      for (int k = 0; k < 8; ++k) p[8 * k + 2 * (k >> 1)] = a[k];
    } else if (logLs >= 4) {
      cx<R>* p = row + padidx(base, 1);
      const int lp = Ls + (Ls >> 3);
#pragma unroll
      for (int k = 0; k < 8; ++k) p[k * lp] = a[k];
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) row[padidx(base + (k << logLs), 1)] = a[k];
    }
  } else if (radix_log == 2) {
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      const int b = j + m * q8;
      const int kk = b & (Ls - 1);
      cx<R> x0 = a[m], x1 = a[m + 2], x2 = a[m + 4], x3 = a[m + 6];
      if (logLs > 0) {
        const int ti = kk << (logM - logLs - 2);
        const cx<R> w1 = tw[ti], w2 = tw[2 * ti];
        const cx<R> w3 = cmul(w1, w2);
        x1 = cmul(x1, w1); x2 = cmul(x2, w2); x3 = cmul(x3, w3);
      }
      dft4(x0, x1, x2, x3);
      const int base = ((b - kk) << 2) + kk;
      row[padidx(base, pad)] = x0;
      row[padidx(base + Ls, pad)] = x1;
      row[padidx(base + 2 * Ls, pad)] = x2;
      row[padidx(base + 3 * Ls, pad)] = x3;
    }
  } else {
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const int b = j + m * q8;
      const int kk = b & (Ls - 1);
      cx<R> x0 = a[m], x1 = a[m + 4];
      if (logLs > 0) x1 = cmul(x1, tw[kk << (logM - logLs - 1)]);
      dft2(x0, x1);
      const int base = ((b - kk) << 1) + kk;
      row[padidx(base, pad)] = x0;
      row[padidx(base + Ls, pad)] = x1;
    }
  }
}

}  // namespace jdb
