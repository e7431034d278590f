// Tile movement shared by the CUDA kernel and the CPU emulation: global -> tile
// load, tile -> (peer) global store, and the pointwise steps of Bluestein's
// algorithm.  All functions take (tid, nthreads) and stride over the tile, so
// the emulation calls them with (0, 1).
//
// The tile is row-major [T rows][pitch], row = index along t, column = index
// along c.  In copy mode a tile covers Cc columns starting at c0; in the FFT
// modes it covers the whole transform axis (c0 == 0) and M >= C columns.
#pragma once
#include "fft_core.h"

namespace jdb {

template <typename E>
struct elem_traits {
  static constexpr bool is_complex = false;
};
template <typename R>
struct elem_traits<cx<R>> {
  static constexpr bool is_complex = true;
  using real = R;
};

template <typename E>
struct alignas(2 * sizeof(E)) pair_of {
  E a, b;
};

// ---- load ---------------------------------------------------------------------------------
// Rows t >= Tn (ragged last tile) and columns >= C are filled with zeros.
template <typename E>
JD_HD void tile_load(const PassDesc& d, E* tile, int o, int t0, int c0, int b, int tid, int nt) {
  const E* in = (const E*)d.in;
  const int T = d.T;
  const int W = (d.fft_mode == JD_COPY) ? d.Cc : d.M;  // columns held per row
  const int cols = (d.fft_mode == JD_COPY) ? ((d.C - c0) < d.Cc ? (d.C - c0) : d.Cc) : d.C;
  const long long base = (long long)o * d.is_o + (long long)b * d.is_b;
  E zero;
  {
    unsigned char* z = (unsigned char*)&zero;
    for (unsigned i = 0; i < sizeof(E); ++i) z[i] = 0;
  }
  const bool blue = d.fft_mode == JD_FFT_BLUESTEIN;
  const bool swp = d.inverse != 0;
  if (d.load_t_contig) {
    // lanes run along t (contiguous in memory), then along c
    if (d.vec_in && sizeof(E) == 8) {
      const int Th = T >> 1;
      for (int e = tid; e < Th * W; e += nt) {
        const int c = e / Th, t = (e - c * Th) * 2;
        E v0 = zero, v1 = zero;
        if (c < cols && t0 + t < d.Tn) {
          const pair_of<E> p = *(const pair_of<E>*)(in + base + (long long)(c0 + c) * d.is_c + (t0 + t));
          v0 = p.a;
          v1 = p.b;
          if constexpr (elem_traits<E>::is_complex) {
            if (swp) { v0 = cswap(v0); v1 = cswap(v1); }
            if (blue) {
              const E ch = ((const E*)d.chirp)[c];
              v0 = cmul(v0, ch);
              v1 = cmul(v1, ch);
            }
          }
        }
        tile[(long long)t * d.pitch + c] = v0;
        tile[(long long)(t + 1) * d.pitch + c] = v1;
      }
    } else {
      for (int e = tid; e < T * W; e += nt) {
        const int c = e / T, t = e - c * T;
        E v = zero;
        if (c < cols && t0 + t < d.Tn) {
          v = in[base + (long long)(c0 + c) * d.is_c + (long long)(t0 + t) * d.is_t];
          if constexpr (elem_traits<E>::is_complex) {
            if (swp) v = cswap(v);
            if (blue) v = cmul(v, ((const E*)d.chirp)[c]);
          }
        }
        tile[(long long)t * d.pitch + c] = v;
      }
    }
  } else {
    // lanes run along c (contiguous in memory)
    if (d.vec_in && sizeof(E) == 8) {
      const int Wh = W >> 1;
      for (int e = tid; e < T * Wh; e += nt) {
        const int t = e / Wh, c = (e - t * Wh) * 2;
        pair_of<E> p;
        p.a = zero;
        p.b = zero;
        if (c < cols && t0 + t < d.Tn) {
          p = *(const pair_of<E>*)(in + base + (long long)(t0 + t) * d.is_t + (c0 + c));
          if constexpr (elem_traits<E>::is_complex) {
            if (swp) { p.a = cswap(p.a); p.b = cswap(p.b); }
            if (blue) {
              p.a = cmul(p.a, ((const E*)d.chirp)[c]);
              p.b = cmul(p.b, ((const E*)d.chirp)[c + 1]);
            }
          }
        }
        *(pair_of<E>*)(tile + (long long)t * d.pitch + c) = p;
      }
    } else {
      for (int e = tid; e < T * W; e += nt) {
        const int t = e / W, c = e - t * W;
        E v = zero;
        if (c < cols && t0 + t < d.Tn) {
          v = in[base + (long long)(t0 + t) * d.is_t + (long long)(c0 + c) * d.is_c];
          if constexpr (elem_traits<E>::is_complex) {
            if (swp) v = cswap(v);
            if (blue) v = cmul(v, ((const E*)d.chirp)[c]);
          }
        }
        tile[(long long)t * d.pitch + c] = v;
      }
    }
  }
}

// After a bulk (asynchronous, unmodified) fetch of the rows: apply what
// tile_load would have applied on the fly.  Only needed for inverse transforms.
template <typename E>
JD_HD void tile_fixup_after_bulk(const PassDesc& d, E* tile, int tid, int nt) {
  if constexpr (elem_traits<E>::is_complex) {
    if (d.inverse) {
      for (int e = tid; e < d.T * d.C; e += nt) {
        const int t = e / d.C, c = e - t * d.C;
        E* p = tile + (long long)t * d.pitch + c;
        *p = cswap(*p);
      }
    }
  }
}

// ---- Bluestein pointwise steps ------------------------------------------------------------------
// After the first length-M transform: multiply by the filter spectrum and swap
// re/im so that the second forward transform acts as an inverse one.
template <typename E>
JD_HD void bluestein_filter(const PassDesc& d, E* tile, int tid, int nt) {
  if constexpr (elem_traits<E>::is_complex) {
    const E* bh = (const E*)d.bhat;
    for (int e = tid; e < d.T * d.M; e += nt) {
      const int t = e / d.M, m = e - t * d.M;
      E* p = tile + (long long)t * d.pitch + m;
      *p = cswap(cmul(*p, bh[m]));
    }
  }
}

// ---- store --------------------------------------------------------------------------------------
template <typename E>
JD_HD E finish_value(const PassDesc& d, E v, int c) {
  if constexpr (elem_traits<E>::is_complex) {
    using R = typename elem_traits<E>::real;
    if (d.fft_mode == JD_FFT_BLUESTEIN) v = cmul(cswap(v), ((const E*)d.chirp)[c]);
    if (d.inverse) v = cswap(v);
    if (d.fft_mode != JD_COPY && d.scale != 1.0) v = cscale(v, (R)d.scale);
  }
  return v;
}

template <typename E>
JD_HD void tile_store(const PassDesc& d, const E* tile, int o, int t0, int c0, int b, int tid, int nt) {
  const int T = d.T;
  const int cols = (d.fft_mode == JD_COPY) ? ((d.C - c0) < d.Cc ? (d.C - c0) : d.Cc) : d.C;
  if (d.store_t_contig) {
    if (d.vec_out && sizeof(E) == 8) {
      const int Th = T >> 1;
      for (int e = tid; e < Th * cols; e += nt) {
        const int c = e / Th, t = (e - c * Th) * 2;
        if (t0 + t >= d.Tn) continue;
        pair_of<E> p;
        p.a = finish_value(d, tile[(long long)t * d.pitch + c], c0 + c);
        p.b = finish_value(d, tile[(long long)(t + 1) * d.pitch + c], c0 + c);
        int peer;
        long long off;
        out_location(d, c0 + c, t0 + t, o, b, peer, off);
        *(pair_of<E>*)((E*)d.out[peer] + off) = p;
      }
    } else {
      for (int e = tid; e < T * cols; e += nt) {
        const int c = e / T, t = e - c * T;
        if (t0 + t >= d.Tn) continue;
        int peer;
        long long off;
        out_location(d, c0 + c, t0 + t, o, b, peer, off);
        ((E*)d.out[peer])[off] = finish_value(d, tile[(long long)t * d.pitch + c], c0 + c);
      }
    }
  } else {
    if (d.vec_out && sizeof(E) == 8) {
      const int Ch = cols >> 1;
      for (int e = tid; e < T * Ch; e += nt) {
        const int t = e / Ch, c = (e - t * Ch) * 2;
        if (t0 + t >= d.Tn) continue;
        pair_of<E> p = *(const pair_of<E>*)(tile + (long long)t * d.pitch + c);
        p.a = finish_value(d, p.a, c0 + c);
        p.b = finish_value(d, p.b, c0 + c + 1);
        int peer;
        long long off;
        out_location(d, c0 + c, t0 + t, o, b, peer, off);
        *(pair_of<E>*)((E*)d.out[peer] + off) = p;
      }
    } else {
      for (int e = tid; e < T * cols; e += nt) {
        const int t = e / cols, c = e - t * cols;
        if (t0 + t >= d.Tn) continue;
        int peer;
        long long off;
        out_location(d, c0 + c, t0 + t, o, b, peer, off);
        ((E*)d.out[peer])[off] = finish_value(d, tile[(long long)t * d.pitch + c], c0 + c);
      }
    }
  }
}

}  // namespace jdb
