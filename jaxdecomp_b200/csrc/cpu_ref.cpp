// CPU emulation of the tile pass: the same descriptor, the same index
// arithmetic (tile_map.h), the same tile movement (tile_ops.h) and the same
// butterflies (fft_core.h) as the CUDA kernel, executed one tile at a time.
// It lets the planner, the peer addressing and the FFT numerics be tested on a
// machine without a GPU, with the buffers of all emulated ranks living in one
// process.  It is a test vehicle, not a product path.
#include <cstring>
#include <vector>

#include "fft_mixed.h"
#include <cstdio>

#include "launch.h"
#include "tile_ops.h"  // also brings fft_core.h

namespace jdb {

template <typename E>
static void fft_rows_host(const PassDesc& d, E* tile) {
  if constexpr (elem_traits<E>::is_complex) {
    int logM = 0;
    while ((1 << logM) < d.M) ++logM;
    const int upr = d.M >> 3;
    const int units = d.T * upr;
    std::vector<E> regs((size_t)units * 8);
    const int ns = fft_num_stages(logM);
    int logLs = 0;
    for (int s = 0; s < ns; ++s) {
      const int rl = fft_stage_radix_log(logM, s);
      for (int u = 0; u < units; ++u)
        stage_read(tile + (long long)(u / upr) * d.pitch, d.M, u % upr, &regs[(size_t)u * 8], d.intra_pad);
      for (int u = 0; u < units; ++u)
        stage_compute_write(tile + (long long)(u / upr) * d.pitch, logM, u % upr, logLs, rl, (const E*)d.twiddle,
                            &regs[(size_t)u * 8], d.intra_pad);
      logLs += rl;
    }
  }
}

template <typename R>
struct HostStage {
  const MixedStage& st;
  const cx<R>* tw;
  const cx<R>* tws;
  const cx<R>* src;
  cx<R>* dst;
  template <int RADIX>
  void run() {
    mixed_stage_row<R, RADIX>(st, tw, tws, src, dst, 0, 1);
  }
};

// Mixed-radix rows: ping-pong between `tile` and `other`; returns the buffer that holds the result.
template <typename E>
static E* mixed_rows_host(const PassDesc& d, const MixedPlan& pl, E* tile, E* other) {
  if constexpr (elem_traits<E>::is_complex) {
    using R = typename elem_traits<E>::real;
    for (int s = 0; s < pl.ns; ++s) {
      for (int r = 0; r < d.T; ++r) {
        HostStage<R> hs{pl.st[s], (const E*)d.twiddle, (const E*)d.tw_stage, tile + (long long)r * d.pitch,
                        other + (long long)r * d.pitch};
        mixed_dispatch(pl.st[s].radix, hs);
      }
      E* tmp = tile;
      tile = other;
      other = tmp;
    }
  }
  return tile;
}

template <typename E>
static int run_pass_host_t(const PassDesc& d) {
  const bool fft = d.fft_mode != JD_COPY;
  if (d.fft_mode == JD_FFT_MIXED) {
    MixedPlan pl;
    if (!make_mixed_plan(d.M, &pl)) return JD_ERR_INVALID_ARG;
    const int tiles = (d.Tn + d.T - 1) / d.T;
    std::vector<E> bufa((size_t)d.T * d.pitch), bufb((size_t)d.T * d.pitch);
    const int NT = 64;
    for (int b = 0; b < d.B; ++b)
      for (int o = 0; o < d.On; ++o)
        for (int tt = 0; tt < tiles; ++tt) {
          const int t0 = tt * d.T;
          for (int tid = 0; tid < NT; ++tid) tile_load<E>(d, bufa.data(), o, t0, 0, b, tid, NT);
          const E* res = mixed_rows_host<E>(d, pl, bufa.data(), bufb.data());
          for (int tid = 0; tid < NT; ++tid) tile_store<E>(d, res, o, t0, 0, b, tid, NT);
        }
    return JD_OK;
  }
  const int tiles_t = (d.Tn + d.T - 1) / d.T;
  const int tiles_c = fft ? 1 : (d.C + d.Cc - 1) / d.Cc;
  std::vector<E> tile((size_t)d.T * d.pitch);
  for (int b = 0; b < d.B; ++b)
    for (int o = 0; o < d.On; ++o)
      for (int tt = 0; tt < tiles_t; ++tt)
        for (int cc = 0; cc < tiles_c; ++cc) {
          const int t0 = tt * d.T, c0 = cc * d.Cc;
          // the data-movement phases run as an emulated block of NT threads so that
          // the same per-thread code paths as on the GPU are exercised
          const int NT = 64;
          for (int tid = 0; tid < NT; ++tid) tile_load<E>(d, tile.data(), o, t0, c0, b, tid, NT);
          if (fft) {
            fft_rows_host<E>(d, tile.data());
            if (d.fft_mode == JD_FFT_BLUESTEIN) {
              for (int tid = 0; tid < NT; ++tid) bluestein_filter<E>(d, tile.data(), tid, NT);
              fft_rows_host<E>(d, tile.data());
            }
          }
          for (int tid = 0; tid < NT; ++tid) tile_store<E>(d, tile.data(), o, t0, c0, b, tid, NT);
        }
  return JD_OK;
}

static int run_pass_host_dispatch(const PassDesc& d) {
  if (d.fft_mode == JD_COPY) {
    if (d.elem_bytes == 4) return run_pass_host_t<float>(d);
    if (d.elem_bytes == 8) return run_pass_host_t<cx<float>>(d);
    if (d.elem_bytes == 16) return run_pass_host_t<cx<double>>(d);
    return JD_ERR_INVALID_ARG;
  }
  if (d.elem_bytes == 8) return run_pass_host_t<cx<float>>(d);
  if (d.elem_bytes == 16) return run_pass_host_t<cx<double>>(d);
  return JD_ERR_INVALID_ARG;
}

// The emulation always checks every store against PassDesc::out_limit (tile_ops.h): a store that would
// leave the destination buffer is skipped and the pass returns JD_ERR_BOUNDS with the first miss in the
// error message.
int run_pass_host(const PassDesc& d) {
  int rc = validate_pass(d);
  if (rc != JD_OK) return rc;
  if (pass_aborted(d)) return JD_OK;
  host_bounds_miss() = BoundsMiss{0, 0, 0, 0};
  rc = run_pass_host_dispatch(d);
  if (rc != JD_OK) return rc;
  const BoundsMiss m = host_bounds_miss();
  if (m.hit) {
    char msg[160];
    std::snprintf(msg, sizeof(msg), "store outside the destination buffer: peer %d, element offset %lld, buffer of %lld elements",
                  m.peer, m.off, m.limit);
    set_last_error(msg);
    return JD_ERR_BOUNDS;
  }
  return JD_OK;
}

// Structural checks shared by the host emulation and the CUDA launcher.
int validate_pass(const PassDesc& d) {
  if (d.C < 1 || d.Tn < 1 || d.On < 1 || d.B < 1) return JD_ERR_INVALID_ARG;
  if (d.Cl < 1 || d.Tl < 1 || d.Ol < 1) return JD_ERR_INVALID_ARG;
  if (d.C % d.Cl || d.Tn % d.Tl || d.On % d.Ol) return JD_ERR_INVALID_ARG;
  const int np = (d.C / d.Cl) + (d.Tn / d.Tl) + (d.On / d.Ol) - 2;
  if (np != d.npeers || np < 1 || np > JD_MAX_PEERS) return JD_ERR_INVALID_ARG;
  if (d.T < 1 || d.pitch < 1 || d.logT < 0 || d.T != (1 << d.logT)) return JD_ERR_INVALID_ARG;
  if (d.fft_mode == JD_FFT_MIXED) {
    // logW: log2 of the next power of two >= M
    if (d.logW < 0 || (1 << d.logW) < d.M || (d.logW > 0 && (1 << (d.logW - 1)) >= d.M)) return JD_ERR_INVALID_ARG;
  } else if (d.logW < 0 || (1 << d.logW) != (d.fft_mode == JD_COPY ? d.Cc : d.M)) {
    return JD_ERR_INVALID_ARG;
  }
  if (d.split_axis < 0 || d.split_axis > 3) return JD_ERR_INVALID_ARG;
  {
    const int want = d.Cl != d.C ? 1 : (d.Tl != d.Tn ? 2 : (d.Ol != d.On ? 3 : 0));
    if (want != d.split_axis) return JD_ERR_INVALID_ARG;
  }
  if (d.fft_mode == JD_FFT_MIXED) {
    if (!d.intra_pad || d.use_bulk) return JD_ERR_INVALID_ARG;  // mixed-radix rows always use the padded layout
  } else if (d.intra_pad && (d.fft_mode == JD_COPY || d.M < 128 || d.use_bulk)) {
    return JD_ERR_INVALID_ARG;
  }
  if (d.elem_bytes != 4 && d.elem_bytes != 8 && d.elem_bytes != 16) return JD_ERR_INVALID_ARG;
  if (d.mul_mode != JD_MUL_NONE) {
    // fused input multiplier: complex data, three batch entries (one per displacement component), rows read
    // element by element (no bulk fetch, no direct-from-global first stage of the mixed-radix kernels)
    if (d.mul_mode != JD_MUL_DISPLACEMENT || d.elem_bytes == 4 || d.B != 3 || d.use_bulk || d.fft_mode == JD_COPY ||
        d.fft_mode == JD_FFT_MIXED)
      return JD_ERR_INVALID_ARG;
    int seen = 0;
    for (int r = 0; r < 3; ++r) {
      if (d.mul.axis[r] < 0 || d.mul.axis[r] > 2 || d.mul.n[r] < 1 || d.mul.off[r] < 0) return JD_ERR_INVALID_ARG;
      seen |= 1 << d.mul.axis[r];
    }
    if (seen != 7) return JD_ERR_INVALID_ARG;
  }
  if (d.load_t_contig ? d.is_t != 1 : d.is_c != 1) return JD_ERR_INVALID_ARG;
  if (d.store_t_contig ? d.os_t != 1 : d.os_c != 1) return JD_ERR_INVALID_ARG;
  if (d.fft_mode == JD_COPY) {
    if (d.Cc < 1 || d.pitch < d.Cc) return JD_ERR_INVALID_ARG;
  } else {
    if (d.elem_bytes == 4) return JD_ERR_INVALID_ARG;
    if (d.fft_mode == JD_FFT_MIXED) {
      MixedPlan pl;
      if (d.M != d.C || !make_mixed_plan(d.M, &pl)) return JD_ERR_INVALID_ARG;
    } else if (d.M < 8 || (d.M & (d.M - 1))) {
      return JD_ERR_INVALID_ARG;
    }
    if (d.pitch < padded_row_length(d.M, d.intra_pad) || !d.twiddle) return JD_ERR_INVALID_ARG;
    if (d.fft_mode == JD_FFT_POW2 && d.M != d.C) return JD_ERR_INVALID_ARG;
    if (d.fft_mode == JD_FFT_BLUESTEIN && (d.M < 2 * d.C - 1 || !d.chirp || !d.bhat)) return JD_ERR_INVALID_ARG;
  }
  if (d.vec_in || d.vec_out) {
    if (d.elem_bytes != 8 || (d.pitch & 1)) return JD_ERR_INVALID_ARG;
  }
  for (int p = 0; p < d.npeers; ++p)
    if (!d.out[p]) return JD_ERR_INVALID_ARG;
  if (!d.in) return JD_ERR_INVALID_ARG;
  return JD_OK;
}

}  // namespace jdb
