// Tile movement shared by the CUDA kernel and the CPU emulation: global -> tile
// load, tile -> (peer) global store, and the pointwise steps of Bluestein's
// algorithm.  All functions take (tid, nthreads) and stride over the tile, so
// the emulation calls them with (0, 1).
//
// The tile is row-major [T rows][pitch], row = index along t, column = index
// along c (through padidx() when the rows carry intra-row padding).  In copy
// mode a tile covers Cc columns starting at c0; in the FFT modes it covers the
// whole transform axis (c0 == 0) and M >= C columns.  T and the number of
// columns per row are powers of two, so tile coordinates come from shifts.
#pragma once
#include "fft_core.h"
#include "status.h"

#ifndef JD_BOUNDS_CHECK
#define JD_BOUNDS_CHECK 0
#endif

namespace jdb {

// ---- checked stores -------------------------------------------------------------------------
// Every store of a pass goes through store_elem / store_pair.  In a normal GPU build they are plain
// stores.  The CPU emulation, and GPU builds compiled with -DJD_BOUNDS_CHECK=1 (the library variant
// that JD_B200_BOUNDS=1 selects), first compare the destination with the size of the destination
// buffer; a miss is recorded as JD_ERR_BOUNDS -- in the status block on the GPU, in a per-thread
// record on the host -- and the access is skipped, so a wrong descriptor is reported instead of
// corrupting a peer's memory.  (The reference relies on cuDecomp and XLA for its index arithmetic and
// has no such mode.)
struct BoundsMiss {
  int32_t hit;
  int32_t peer;
  long long off, limit;
};
#if !defined(__CUDA_ARCH__)
inline BoundsMiss& host_bounds_miss() {
  static thread_local BoundsMiss m = {0, 0, 0, 0};
  return m;
}
#endif

JD_HD bool store_in_bounds(const PassDesc& d, int peer, long long off, int count) {
#if JD_BOUNDS_CHECK || !defined(__CUDA_ARCH__)
  if (d.out_limit <= 0) return true;
  if (peer >= 0 && peer < d.npeers && off >= 0 && off + count <= d.out_limit) return true;
#if defined(__CUDA_ARCH__)
  StatusBlock* st = (StatusBlock*)d.status;
  if (st != nullptr && atomicCAS(&st->code, 0, (int)JD_ERR_BOUNDS) == 0) {
    st->peer = peer;
    st->expected = (int32_t)(d.out_limit > 2147483647LL ? 2147483647LL : d.out_limit);
    st->seen = (int32_t)(off > 2147483647LL ? 2147483647LL : (off < -2147483647LL ? -2147483647LL : off));
    st->where = 200;
    __threadfence_system();
  }
#else
  BoundsMiss& m = host_bounds_miss();
  if (!m.hit) m = BoundsMiss{1, peer, off, d.out_limit};
#endif
  return false;
#else
  return true;
#endif
}

// True when a cross-rank wait failed earlier on this rank or on a peer (signal.cu sets the word): the
// data in the exchange buffers is then incomplete, and every block of every later pass returns at once.
JD_HD bool pass_aborted(const PassDesc& d) {
#if defined(__CUDA_ARCH__)
  return d.abort_word != nullptr && *(const volatile uint32_t*)d.abort_word != 0;
#else
  return d.abort_word != nullptr && *d.abort_word != 0;
#endif
}

template <typename E>
JD_HD void store_elem(const PassDesc& d, int peer, long long off, const E& v) {
  if (!store_in_bounds(d, peer, off, 1)) return;
  ((E*)d.out[peer])[off] = v;
}

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

template <typename E>
JD_HD void store_pair(const PassDesc& d, int peer, long long off, const pair_of<E>& v) {
  if (!store_in_bounds(d, peer, off, 2)) return;
  *(pair_of<E>*)((E*)d.out[peer] + off) = v;
}

template <typename E>
JD_HD E zero_elem() {
  E z;
  unsigned char* p = (unsigned char*)&z;
  for (unsigned i = 0; i < sizeof(E); ++i) p[i] = 0;
  return z;
}

JD_HD int tile_cols(const PassDesc& d, int c0) {
  if (d.fft_mode != JD_COPY) return d.C;
  return (d.C - c0) < d.Cc ? (d.C - c0) : d.Cc;
}

// Fused input multiplier (PassDesc::mul_mode) for the element at local indices (c, t, o) of batch b.
template <typename E>
JD_HD E apply_mul(const PassDesc& d, E v, int c, int t, int o, int b) {
  if constexpr (elem_traits<E>::is_complex) {
    using R = typename elem_traits<E>::real;
    if (d.mul_mode == JD_MUL_DISPLACEMENT) {
      const MulDesc& m = d.mul;
      const int idx[3] = {c, t, o};
      R kv[3] = {0, 0, 0};
      R kk = 0;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
      for (int r = 0; r < 3; ++r) {
        const int a = m.axis[r];
        const int g = m.off[r] + idx[r];
        const int f = g < (m.n[a] + 1) / 2 ? g : g - m.n[a];
        const R k = (R)m.kfac[a] * (R)f;
        kv[a] = k;
        kk += k * k;
      }
      const R s = kk > (R)0 ? kv[b] / kk : (R)0;
      // i * s * (x + i y) = s * (-y + i x)
      v = E{-v.y * s, v.x * s};
    }
  }
  return v;
}

// The same multiplier with everything that does not depend on the column hoisted out: one object per
// (row t, plane o, batch entry b) of a thread, then a compare, a convert, two FMAs, a reciprocal and three
// multiplies per element.  (The general form above costs about forty instructions per element, which made
// a fused pass twice as slow as a plain one; this form keeps it at the speed of the plain pass.)
template <typename R>
struct MulRow {
  R base;      // k_t^2 + k_o^2
  R fixed;     // k_b when component b runs along t or o
  R kf;        // 2*pi / box of the axis that c runs along
  int off, n, half;
  bool along_c;  // component b runs along c

  JD_HD MulRow(const PassDesc& d, int t, int o, int b) {
    const MulDesc& m = d.mul;
    const R k_t = wave(m, m.axis[1], m.off[1] + t), k_o = wave(m, m.axis[2], m.off[2] + o);
    base = k_t * k_t + k_o * k_o;
    const int ac = m.axis[0];
    along_c = b == ac;
    fixed = b == m.axis[1] ? k_t : k_o;
    kf = (R)(ac == 0 ? m.kfac[0] : (ac == 1 ? m.kfac[1] : m.kfac[2]));
    off = m.off[0];
    n = ac == 0 ? m.n[0] : (ac == 1 ? m.n[1] : m.n[2]);
    half = (n + 1) / 2;
  }

  static JD_HD R wave(const MulDesc& m, int a, int g) {
    const int na = a == 0 ? m.n[0] : (a == 1 ? m.n[1] : m.n[2]);
    const double kf_a = a == 0 ? m.kfac[0] : (a == 1 ? m.kfac[1] : m.kfac[2]);
    const int f = g < (na + 1) / 2 ? g : g - na;
    return (R)kf_a * (R)f;
  }

  JD_HD cx<R> apply(cx<R> v, int c) const {
    const int g = off + c;
    const int f = g < half ? g : g - n;
    const R kc = kf * (R)f;
    const R kk = base + kc * kc;
    const R num = along_c ? kc : fixed;
    R s;
#if defined(__CUDA_ARCH__)
    if constexpr (sizeof(R) == 4) s = kk > (R)0 ? num * __frcp_rn(kk) : (R)0;
    else s = kk > (R)0 ? num / kk : (R)0;
#else
    s = kk > (R)0 ? num / kk : (R)0;
#endif
    return cx<R>{-v.y * s, v.x * s};
  }
};

// What a freshly loaded element goes through before it enters the tile: the fused multiplier (on the true
// value), the conjugation trick of inverse transforms, the chirp of Bluestein's algorithm.
template <typename E>
JD_HD E prepare_value(const PassDesc& d, E v, int c, int t, int o, int b) {
  if (d.mul_mode != JD_MUL_NONE) v = apply_mul(d, v, c, t, o, b);
  if constexpr (elem_traits<E>::is_complex) {
    if (d.inverse) v = cswap(v);
    if (d.fft_mode == JD_FFT_BLUESTEIN) v = cmul(v, ((const E*)d.chirp)[c]);
  }
  return v;
}

// ---- load ---------------------------------------------------------------------------------
// Rows t >= Tn (ragged last tile) and columns >= C are filled with zeros.
template <typename E>
JD_HD void tile_load(const PassDesc& d, E* tile, int o, int t0, int c0, int b, int tid, int nt) {
  const E* in = (const E*)d.in + ((long long)o * d.is_o + (long long)b * d.is_b);
  const int T = d.T, logT = d.logT, logW = d.logW, W = 1 << logW;
  const int cols = tile_cols(d, c0);
  const int pad = d.intra_pad;
  const E zero = zero_elem<E>();
  // mixed-radix rows hold exactly C columns: nothing is stored past them
  const int wlim = d.fft_mode == JD_FFT_MIXED ? cols : W;
  if (d.load_t_contig) {
    // lanes run along t (contiguous in memory), then along c
    if (d.vec_in && sizeof(E) == 8) {
      const int lh = logT - 1, Th = T >> 1;
      for (int e = tid; e < (W << lh); e += nt) {
        const int c = e >> lh, t = (e & (Th - 1)) << 1;
        if (c >= wlim) continue;
        E v0 = zero, v1 = zero;
        if (c < cols && t0 + t < d.Tn) {
          const pair_of<E> p = *(const pair_of<E>*)(in + (long long)(c0 + c) * d.is_c + (t0 + t));
          v0 = prepare_value(d, p.a, c0 + c, t0 + t, o, b);
          v1 = prepare_value(d, p.b, c0 + c, t0 + t + 1, o, b);
        }
        const int col = padidx(c, pad);
        tile[t * d.pitch + col] = v0;
        tile[(t + 1) * d.pitch + col] = v1;
      }
    } else {
      for (int e = tid; e < (W << logT); e += nt) {
        const int c = e >> logT, t = e & (T - 1);
        if (c >= wlim) continue;
        E v = zero;
        if (c < cols && t0 + t < d.Tn)
          v = prepare_value(d, in[(long long)(c0 + c) * d.is_c + (long long)(t0 + t) * d.is_t], c0 + c, t0 + t, o, b);
        tile[t * d.pitch + padidx(c, pad)] = v;
      }
    }
  } else {
    // lanes run along c (contiguous in memory)
    if (d.vec_in && sizeof(E) == 8) {
      const int lh = logW - 1, Wh = W >> 1;
      for (int e = tid; e < (T << lh); e += nt) {
        const int t = e >> lh, c = (e & (Wh - 1)) << 1;
        if (c >= wlim) continue;
        pair_of<E> p;
        p.a = zero;
        p.b = zero;
        if (c < cols && t0 + t < d.Tn) {
          p = *(const pair_of<E>*)(in + (long long)(t0 + t) * d.is_t + (c0 + c));
          p.a = prepare_value(d, p.a, c0 + c, t0 + t, o, b);
          p.b = prepare_value(d, p.b, c0 + c + 1, t0 + t, o, b);
        }
        *(pair_of<E>*)(tile + t * d.pitch + padidx(c, pad)) = p;
      }
    } else {
      for (int e = tid; e < (T << logW); e += nt) {
        const int t = e >> logW, c = e & (W - 1);
        if (c >= wlim) continue;
        E v = zero;
        if (c < cols && t0 + t < d.Tn)
          v = prepare_value(d, in[(long long)(t0 + t) * d.is_t + (long long)(c0 + c) * d.is_c], c0 + c, t0 + t, o, b);
        tile[t * d.pitch + padidx(c, pad)] = v;
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
      for (int e = tid; e < (d.T << d.logW); e += nt) {
        const int t = e >> d.logW, c = e & ((1 << d.logW) - 1);
        E* p = tile + t * d.pitch + c;
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
    for (int e = tid; e < (d.T << d.logW); e += nt) {
      const int t = e >> d.logW, m = e & ((1 << d.logW) - 1);
      E* p = tile + t * d.pitch + padidx(m, d.intra_pad);
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

// Destination of column c / row t, given the part contributed by (o, b).
struct OutBase {
  long long off;  // out_base + o-part + b-part
  int peer;       // peer contribution of o
};

JD_HD OutBase out_base_for(const PassDesc& d, int o, int b) {
  OutBase r;
  const int po = d.split_axis == 3 ? o / d.Ol : 0;
  r.peer = po;
  r.off = d.out_base + (long long)(o - po * d.Ol) * d.os_o + (long long)b * d.os_b;
  return r;
}

// peer and element offset of (c, t) given the (o, b) part
JD_HD long long out_offset(const PassDesc& d, const OutBase& ob, int c, int t, int& peer) {
  const int pc = d.split_axis == 1 ? c / d.Cl : 0;
  const int pt = d.split_axis == 2 ? t / d.Tl : 0;
  peer = ob.peer + pc + pt;
  return ob.off + (long long)(c - pc * d.Cl) * d.os_c + (long long)(t - pt * d.Tl) * d.os_t;
}

template <typename E>
JD_HD void tile_store(const PassDesc& d, const E* tile, int o, int t0, int c0, int b, int tid, int nt) {
  const int T = d.T, logT = d.logT, logW = d.logW, W = 1 << logW;
  const int cols = tile_cols(d, c0);
  const int pad = d.intra_pad;
  const OutBase ob = out_base_for(d, o, b);
  if (d.store_t_contig) {
    // every thread keeps its t and walks down the columns: the peer of a column
    // is tracked incrementally instead of dividing per element
    const bool vec = d.vec_out && sizeof(E) == 8;
    const int lt = vec ? logT - 1 : logT;
    const int per_col = 1 << lt;           // threads that share one column
    if (nt % per_col == 0) {
      const int step = nt >> lt;
      const int tsub = tid & (per_col - 1);
      const int t = vec ? (tsub << 1) : tsub;
      if (t0 + t < d.Tn) {
        const int pt = d.split_axis == 2 ? (t0 + t) / d.Tl : 0;
        const long long toff = ob.off + (long long)(t0 + t - pt * d.Tl) * d.os_t;
        int c = tid >> lt;
        int pc = d.split_axis == 1 ? (c0 + c) / d.Cl : 0;
        int cl = c0 + c - pc * d.Cl;
        const E* src = tile + t * d.pitch;
        for (; c < cols; c += step) {
          const long long doff = toff + (long long)cl * d.os_c;
          const int col = padidx(c, pad);
          if (vec) {
            pair_of<E> p;
            p.a = finish_value(d, src[col], c0 + c);
            p.b = finish_value(d, src[d.pitch + col], c0 + c);
            store_pair<E>(d, ob.peer + pc + pt, doff, p);
          } else {
            store_elem<E>(d, ob.peer + pc + pt, doff, finish_value(d, src[col], c0 + c));
          }
          cl += step;
          if (d.split_axis == 1)
            while (cl >= d.Cl) {
              cl -= d.Cl;
              ++pc;
            }
        }
      }
    } else {
      for (int e = tid; e < (cols << logT); e += nt) {
        const int c = e >> logT, t = e & (T - 1);
        if (t0 + t >= d.Tn) continue;
        int peer;
        const long long doff = out_offset(d, ob, c0 + c, t0 + t, peer);
        store_elem<E>(d, peer, doff, finish_value(d, tile[t * d.pitch + padidx(c, pad)], c0 + c));
      }
    }
  } else {
    if (d.vec_out && sizeof(E) == 8) {
      const int lh = logW - 1, Wh = W >> 1;
      for (int e = tid; e < (T << lh); e += nt) {
        const int t = e >> lh, c = (e & (Wh - 1)) << 1;
        if (c >= cols || t0 + t >= d.Tn) continue;
        pair_of<E> p = *(const pair_of<E>*)(tile + t * d.pitch + padidx(c, pad));
        p.a = finish_value(d, p.a, c0 + c);
        p.b = finish_value(d, p.b, c0 + c + 1);
        int peer;
        const long long doff = out_offset(d, ob, c0 + c, t0 + t, peer);
        store_pair<E>(d, peer, doff, p);
      }
    } else {
      for (int e = tid; e < (T << logW); e += nt) {
        const int t = e >> logW, c = e & (W - 1);
        if (c >= cols || t0 + t >= d.Tn) continue;
        int peer;
        const long long doff = out_offset(d, ob, c0 + c, t0 + t, peer);
        store_elem<E>(d, peer, doff, finish_value(d, tile[t * d.pitch + padidx(c, pad)], c0 + c));
      }
    }
  }
}

}  // namespace jdb
