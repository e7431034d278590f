// Descriptor of one "tile pass" and the index arithmetic that maps an element
// of a rank's local block to (destination peer, offset in that peer's buffer).
//
// A pass reads a local 3-D block (plus an optional batch dimension) through
// arbitrary strides, optionally Fourier-transforms it along one axis, and
// scatters the result into up to JD_MAX_PEERS destination buffers.  The three
// local axes are given roles:
//   c  the transform axis (or, in copy mode, the axis that is contiguous in the input),
//   t  the axis that is tiled together with c (contiguous on the output side
//      for a rotating pass, or on the input side for a strided transform),
//   o  the remaining axis: one value per thread block.
// A tiled all-to-all over P ranks that splits one of the axes is expressed by
// that axis's chunk extent (Cl, Tl or Ol = extent / P): element index / chunk
// selects the peer, index % chunk is the coordinate on the peer, and out_base
// holds this rank's constant offset along the concatenation axis.  Local axis
// permutations are folded into the output strides.  One descriptor therefore
// covers every step group of the distributed FFT, the six pencil transposes in
// both layout modes, and purely local passes (npeers == 1).
//
// This is the device-side counterpart of what the reference delegates to
// cudecompTranspose* + cufftXtExec (src/csrc/fft.cu:460-535) or to XLA's
// all_to_all + transpose (src/jaxdecomp/_src/jax/fft.py:94-135).
//
// The header is plain C++ so that the CPU emulation used by the unit tests
// shares the exact arithmetic of the kernels.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define JD_HD __host__ __device__ __forceinline__
#else
#define JD_HD inline
#endif

#define JD_MAX_PEERS 16

namespace jdb {

// JD_FFT_MIXED: M == C is a product of the primes 2..13, transformed by the mixed-radix kernel; logW is
// then the log2 of the next power of two >= M (only used to split loop counters into row and column).
enum FftMode : int32_t { JD_COPY = 0, JD_FFT_POW2 = 1, JD_FFT_BLUESTEIN = 2, JD_FFT_MIXED = 3 };

// Pointwise Fourier-space multiplier applied to the input of a pass, so that an operator such as
// "i k_d / k^2" costs no pass over memory of its own (the reference gets the same effect from XLA
// fusing the element-wise expression of examples/lpt_nbody_demo.py:120-133 into its neighbours).
// The wave number along original axis a at global index g is kfac[a] * (g < (n[a]+1)/2 ? g : g - n[a]).
struct MulDesc {
  int32_t n[3];     // global extents of the original axes 0, 1, 2
  int32_t off[3];   // global index of local index 0 along the role axes c, t, o
  int32_t axis[3];  // original axis that the role axes c, t, o run along
  double kfac[3];   // 2*pi / box length of the original axes
};

enum MulMode : int32_t {
  JD_MUL_NONE = 0,
  JD_MUL_DISPLACEMENT = 1,  // batch entry b (0..2) of the pass reads in * i * k_b / |k|^2 (0 at k = 0)
};

struct PassDesc {
  // strides in elements
  long long is_c, is_t, is_o, is_b;
  long long os_c, os_t, os_o, os_b;
  long long out_base;
  int32_t C, Tn, On, B;   // extents of c, t, o and batch
  int32_t Cl, Tl, Ol;     // per-peer chunk extents (== full extent when the axis is not split)
  int32_t npeers;
  int32_t fft_mode;       // FftMode
  int32_t M;              // transform length held in shared memory (C, or the Bluestein length)
  int32_t inverse;        // 1: conjugate (inverse-direction) transform
  int32_t T, Cc;          // tile extents along t and c (Cc == M-row in fft modes)
  int32_t pitch;          // shared-memory row pitch in elements
  int32_t elem_bytes;     // 4, 8 or 16
  int32_t load_t_contig;  // 1: input is contiguous along t (is_t == 1), else along c
  int32_t store_t_contig; // 1: output is contiguous along t (os_t == 1), else along c
  int32_t use_bulk;       // 1: fetch rows with bulk async copies (needs 16-byte aligned rows)
  int32_t mul_mode;       // MulMode: pointwise multiplier applied to every element as it is read
  int32_t vec_in;         // 1: 8-byte elements may be loaded two at a time (16-byte accesses)
  int32_t vec_out;        // 1: 8-byte elements may be stored two at a time
  int32_t intra_pad;      // 1: rows carry two unused slots after every 16 columns (bank-conflict-free FFT exchanges)
  int32_t logT;           // T == 1 << logT
  int32_t logW;           // columns held per row (M in fft modes, Cc in copy mode) == 1 << logW
  int32_t split_axis;     // which axis selects the peer: 0 none, 1 c, 2 t, 3 o
  int32_t grid_limit;     // > 0: launch at most this many blocks, each looping over tiles (leaves the other
                          // SMs to a pass that runs concurrently on another stream); 0: one block per tile
  double scale;
  const void* in;
  void* out[JD_MAX_PEERS];
  const void* twiddle;    // M entries: exp(-2*pi*i*n/M)
  const void* tw_stage;   // per-stage twiddle records of the specialised power-of-two kernel (fft_fast_plan.h), or null
  const void* chirp;      // Bluestein: C entries exp(-i*pi*n^2/C)
  const void* bhat;       // Bluestein: M entries FFT_M(conj chirp, wrapped) / M
  MulDesc mul;            // geometry for mul_mode != JD_MUL_NONE
  const uint32_t* abort_word;  // device word of this rank that a failed cross-rank wait sets (signal.cu); blocks
                               // return at entry when it is non-zero; null: not checked
  long long out_limit;    // elements each destination buffer holds; checked per store by the CPU emulation and by
                          // kernels compiled with JD_BOUNDS_CHECK (0: unknown, not checked)
  void* status;           // StatusBlock* for the bounds check of JD_BOUNDS_CHECK builds, or null
};

// (c, t, o, b) of the local block -> destination peer and element offset there.
JD_HD void out_location(const PassDesc& d, int c, int t, int o, int b, int& peer, long long& off) {
  const int pc = c / d.Cl, pt = t / d.Tl, po = o / d.Ol;
  peer = pc + pt + po;
  off = d.out_base + (long long)(c - pc * d.Cl) * d.os_c + (long long)(t - pt * d.Tl) * d.os_t +
        (long long)(o - po * d.Ol) * d.os_o + (long long)b * d.os_b;
}

// Restrict a pass to the rows [lo, lo + len) of its t axis (role == 2) or its o axis (role == 3).
// The restricted pass reads and writes exactly the elements that the full pass touches for those
// indices, so running it for a partition of the axis is equivalent to the full pass.  Used to cut a
// pass into chunks that are pipelined with the pass that consumes them.  Requirements: the axis must
// not select the destination peer, and a t range must start and end on a tile boundary (so that tiles,
// and with them the vector-access alignment rules, are those of the full pass).  The pointer `in`
// must already be set.  Returns false (descriptor unchanged) when the range is not admissible.
inline bool restrict_pass(PassDesc& d, int role, int lo, int len) {
  if (role != 2 && role != 3) return false;
  if (d.split_axis == role || lo < 0 || len <= 0) return false;
  const int ext = role == 2 ? d.Tn : d.On;
  if (lo + len > ext) return false;
  if (role == 2) {
    // tile heights are powers of two up to 32 (the specialised kernels pick theirs from Tn's divisibility)
    const int align = d.T > 32 ? d.T : 32;
    if ((lo % align) != 0 || ((len % align) != 0 && lo + len != ext)) return false;
    d.in = static_cast<const char*>(d.in) + (long long)lo * d.is_t * d.elem_bytes;
    d.out_base += (long long)lo * d.os_t;
    d.Tn = len;
    d.Tl = len;
  } else {
    d.in = static_cast<const char*>(d.in) + (long long)lo * d.is_o * d.elem_bytes;
    d.out_base += (long long)lo * d.os_o;
    d.On = len;
    d.Ol = len;
  }
  return true;
}

JD_HD long long in_location(const PassDesc& d, int c, int t, int o, int b) {
  return (long long)c * d.is_c + (long long)t * d.is_t + (long long)o * d.is_o + (long long)b * d.is_b;
}

}  // namespace jdb
