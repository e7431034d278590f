// CPU emulation of the tile pass: the same descriptor, the same index
// arithmetic (tile_map.h), the same tile movement (tile_ops.h) and the same
// butterflies (fft_core.h) as the CUDA kernel, executed one tile at a time.
// It lets the planner, the peer addressing and the FFT numerics be tested on a
// machine without a GPU, with the buffers of all emulated ranks living in one
// process.  It is a test vehicle, not a product path.
#include <cstdint>
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

// ---- host twin of the rotating copy kernels ---------------------------------------------------------------
// copy_rotate8_kernel / copy_rotate16_kernel (copy_fast.cu) restated for the host: the same decomposition
// into blocks, warps and lanes, the same swizzled (or odd-pitch) shared-memory tile, the same destination
// arithmetic, executed serially -- so that their addressing on every mesh shape, including the peers of a
// column or of a tile's rows, is tested against the general pass without a GPU.  A restatement, not shared
// code: it has to be kept in step with the kernels by hand.
namespace {

struct Unit16 {
  uint64_t lo, hi;
};

struct HostTile {
  int c0, t0, o, b;
};

HostTile host_tile_of_block(const PassDesc& d, long long bid, int b, int TC, int TT) {
  const int tiles_c = d.C / TC, tiles_t = d.Tn / TT;
  HostTile tc;
  tc.c0 = (int)(bid % tiles_c) * TC;
  bid /= tiles_c;
  tc.t0 = (int)(bid % tiles_t) * TT;
  tc.o = (int)(bid / tiles_t);
  tc.b = b;
  return tc;
}

// count elements of EB bytes each at element offset off of peer's buffer
template <typename T>
void host_checked_store(const PassDesc& d, int peer, long long off, const T* src, int count) {
  if (!store_in_bounds(d, peer, off, count)) return;
  std::memcpy((T*)d.out[peer] + off, src, sizeof(T) * (size_t)count);
}

void copy_rotate8_host(const PassDesc& d) {
  constexpr int TC = 64, TT = 64, UNITS = TT / 2, WARPS = 8;
  const long long nblocks = (long long)(d.C / TC) * (d.Tn / TT) * d.On;
  std::vector<Unit16> sm((size_t)TC * UNITS);
  for (int b = 0; b < d.B; ++b)
    for (long long bid = 0; bid < nblocks; ++bid) {
      const HostTile tc = host_tile_of_block(d, bid, b, TC, TT);
      for (int warp = 0; warp < WARPS; ++warp)
        for (int lane = 0; lane < 32; ++lane) {
          const uint64_t* in = (const uint64_t*)d.in + ((long long)tc.o * d.is_o + (long long)tc.b * d.is_b +
                                                        (long long)tc.t0 * d.is_t + tc.c0 + 2 * lane);
          const int sw_w = lane & 7;
          for (int it = 0; it < 4; ++it) {
            const int tp = it * 8 + warp;
            const uint64_t* p = in + (long long)(2 * tp) * d.is_t;
            const uint64_t r00 = p[0], r01 = p[1], r10 = p[d.is_t], r11 = p[d.is_t + 1];
            sm[(size_t)(2 * lane) * UNITS + (tp ^ sw_w)] = Unit16{r00, r10};
            sm[(size_t)(2 * lane + 1) * UNITS + (tp ^ sw_w)] = Unit16{r01, r11};
          }
        }
      const OutBase ob = out_base_for(d, tc.o, tc.b);
      const int pt = d.split_axis == 2 ? tc.t0 / d.Tl : 0;
      for (int warp = 0; warp < WARPS; ++warp)
        for (int lane = 0; lane < 32; ++lane) {
          const long long toff = ob.off + (long long)(tc.t0 - pt * d.Tl + 2 * lane);
          for (int it = 0; it < 8; ++it) {
            const int c = it * 8 + warp;
            const Unit16 v = sm[(size_t)c * UNITS + (lane ^ ((c >> 1) & 7))];
            const int gc = tc.c0 + c;
            const int pc = d.split_axis == 1 ? gc / d.Cl : 0;
            const uint64_t pair[2] = {v.lo, v.hi};
            host_checked_store<uint64_t>(d, ob.peer + pc + pt, toff + (long long)(gc - pc * d.Cl) * d.os_c, pair, 2);
          }
        }
    }
}

void copy_rotate16_host(const PassDesc& d) {
  constexpr int TC = 32, TT = 32, PITCH = TC + 1, WARPS = 8;
  const long long nblocks = (long long)(d.C / TC) * (d.Tn / TT) * d.On;
  std::vector<Unit16> sm((size_t)TT * PITCH);
  for (int b = 0; b < d.B; ++b)
    for (long long bid = 0; bid < nblocks; ++bid) {
      const HostTile tc = host_tile_of_block(d, bid, b, TC, TT);
      for (int warp = 0; warp < WARPS; ++warp)
        for (int lane = 0; lane < 32; ++lane) {
          const Unit16* in = (const Unit16*)d.in + ((long long)tc.o * d.is_o + (long long)tc.b * d.is_b +
                                                    (long long)tc.t0 * d.is_t + tc.c0 + lane);
          for (int it = 0; it < 4; ++it) sm[(size_t)(it * 8 + warp) * PITCH + lane] = in[(long long)(it * 8 + warp) * d.is_t];
        }
      const OutBase ob = out_base_for(d, tc.o, tc.b);
      const int pt = d.split_axis == 2 ? tc.t0 / d.Tl : 0;
      for (int warp = 0; warp < WARPS; ++warp)
        for (int lane = 0; lane < 32; ++lane) {
          const long long toff = ob.off + (long long)(tc.t0 - pt * d.Tl + lane);
          for (int it = 0; it < 4; ++it) {
            const int c = it * 8 + warp;
            const Unit16 v = sm[(size_t)lane * PITCH + c];
            const int gc = tc.c0 + c;
            const int pc = d.split_axis == 1 ? gc / d.Cl : 0;
            host_checked_store<Unit16>(d, ob.peer + pc + pt, toff + (long long)(gc - pc * d.Cl) * d.os_c, &v, 1);
          }
        }
    }
}

}  // namespace

// Runs the host twin on a descriptor that copy_fast_eligible() accepted (the caller checks).
int run_copy_fast_host(const PassDesc& d) {
  int rc = validate_pass(d);
  if (rc != JD_OK) return rc;
  if (d.fft_mode != JD_COPY || (d.elem_bytes != 8 && d.elem_bytes != 16)) return JD_ERR_INVALID_ARG;
  if (pass_aborted(d)) return JD_OK;
  host_bounds_miss() = BoundsMiss{0, 0, 0, 0};
  if (d.elem_bytes == 8)
    copy_rotate8_host(d);
  else
    copy_rotate16_host(d);
  if (host_bounds_miss().hit) {
    set_last_error("rotating copy pass: store outside the destination buffer");
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
