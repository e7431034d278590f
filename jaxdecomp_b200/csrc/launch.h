// Host-side entry points of the native core (declarations).
#pragma once
#include <cstddef>
#include <cstdint>

#include "status.h"
#include "tile_map.h"

namespace jdb {

// ---- tile pass (fft_pass.cu / cpu_ref.cpp) ---------------------------------------------------------
int validate_pass(const PassDesc& d);
int run_pass_host(const PassDesc& d);
// Rotating copy passes of 8- and 16-byte elements whose extents are multiples of the tile (copy_fast.cu):
// launch_pass uses them instead of the general kernel's copy mode.  Eligibility looks at the addresses too
// (16-byte alignment), so it is decided at launch time.  JD_B200_COPY_FAST=0 switches them off.
bool copy_fast_eligible(const PassDesc& d);
int launch_copy_fast(const PassDesc& d, void* stream);
// Host restatement of those kernels (cpu_ref.cpp), for tests of their addressing without a GPU.
int run_copy_fast_host(const PassDesc& d);
// Launch on `stream`.  Returns a Status; CUDA launch errors are reported as JD_ERR_CUDA
// and the message is available from last_error_message().
int launch_pass(const PassDesc& d, void* stream, StatusBlock* status);
// Threads per block the launcher will use for this descriptor (0 if invalid).
int pass_threads(const PassDesc& d);
size_t pass_smem_bytes(const PassDesc& d);
// Specialised kernel for power-of-two lengths 128..4096 (fft_fast.cu)
bool fast_pass_eligible(const PassDesc& d);
int launch_fast_pass(const PassDesc& d, void* stream);
// Mixed-radix kernel for lengths with prime factors up to 13 (fft_mixed.cu)
int launch_mixed_pass(const PassDesc& d, void* stream);
// Length-specialised variants (fft_mixed_s*.cu); JD_ERR_UNSUPPORTED when the length or the tiling is not theirs
int launch_mixed_static_a(const PassDesc& d, void* stream);
int launch_mixed_static_b(const PassDesc& d, void* stream);
int launch_mixed_static_c(const PassDesc& d, void* stream);

// ---- cross-rank signalling (signal.cu) ---------------------------------------------------------------
// Words of a rank's flag region (uint32): [0, JD_MAX_PEERS) epoch slots, one per peer; the rank's own
// barrier counter; the abort word (0, or 1 + the rank whose wait failed).
constexpr int kFlagEpochCounterWord = 64;
constexpr int kFlagAbortWord = 65;
struct PeerFlags {
  uint32_t* flags[JD_MAX_PEERS];  // flags[p]: base of peer p's flag array (its own for p == me)
};
// Stream-ordered barrier over n ranks: writes the epoch into slot `me` of every
// peer's flag array, then waits (bounded by timeout_ns) until all n slots of
// this rank's own array have reached it.  The epoch is *epoch_counter + 1 (and
// the counter is advanced) when epoch_counter is a device pointer, else `epoch`.
int launch_signal_barrier(const PeerFlags& pf, int me, int n, uint32_t* epoch_counter, uint32_t epoch,
                          long long timeout_ns, void* stream, StatusBlock* status);
// Only the waiting half, for tests of the time-out path (nothing signals).
int launch_wait_only(uint32_t* my_flags, int n, uint32_t epoch, long long timeout_ns, void* stream,
                     StatusBlock* status);

// ---- halo kernels (halo.cu) ---------------------------------------------------------------------------
struct HaloRegion {
  // region of the local padded block, [lo0,hi0) x [lo1,hi1) x full last axis
  int32_t lo0, hi0, lo1, hi1;
  int32_t peer;         // index into HaloDesc::stage (destination or source), -1: none (zero fill / skip)
  long long stage_off;  // element offset of this region's slab inside the staging buffer
  int32_t dlo0, dlo1;   // direct pushes: first row / column of the region this slab lands in on the peer
};
struct HaloDesc {
  int32_t S0, S1, S2, B;   // padded local block (B = batch)
  int32_t elem_bytes;      // 4, 8, 16
  int32_t nregions;
  int32_t accumulate;      // unpack: 0 overwrite, 1 add
  int32_t is_f64;          // accumulate arithmetic: 1 = float64/complex128, 0 = float32/complex64
  int32_t direct;          // pack only: 1 = stage[p] is peer p's *block* (same shape as this rank's) and every
                           // slab is stored at its final place there, rows [dlo0..) x columns [dlo1..)
  HaloRegion reg[8];
  void* stage[JD_MAX_PEERS];  // staging buffers (peer-visible)
  const void* src;            // local block read by pack
  void* dst;                  // local block written by unpack
};
// pack: for every region copy src[region] -> stage[reg.peer] + stage_off (peer stores), or, in direct mode,
// straight into the neighbour's padded block
int launch_halo_pack(const HaloDesc& d, void* stream);
// unpack: for every region dst[region] (=|+=) stage[reg.peer] + stage_off (local loads); peer == -1 -> zero (overwrite mode)
int launch_halo_unpack(const HaloDesc& d, void* stream);

// ---- particle-mesh kernels (cic.cu) ---------------------------------------------------------------------
struct CicArgs {
  long long n;               // number of particles
  int32_t S0, S1, S2;        // local (padded) mesh block
  int32_t wrap0, wrap1, wrap2;
  int32_t g0, g1, g2;        // lattice of initial positions (grid mode: pos holds displacements), or 0
  float o0, o1, o2;          // offset of the lattice inside the block
  float wscalar;             // weight of every particle when no per-particle weights are given
  int32_t planar;            // 0: pos is [n, 3]; 1: pos is three planes [3, n] (gradients use the same layout)
};
// pos: [n,3] (or, planar, [3,n]) float32 positions (or displacements in grid mode) in cell units
int launch_cic_paint(const CicArgs& a, const float* pos, const float* weight, float* mesh, void* stream);
int launch_cic_readout(const CicArgs& a, const float* pos, const float* mesh, float* out, void* stream);
int launch_cic_paint_grad_pos(const CicArgs& a, const float* pos, const float* weight, const float* gmesh, float* gpos,
                              void* stream);

// ---- k-space elementwise kernels (kspace.cu) --------------------------------------------------------------
struct KSpaceDesc {
  // local block of the rotated FFT output: dims (L0, L1, L2) hold original axes (1, 2, 0)
  int32_t L0, L1, L2;
  int32_t off0, off1, off2;  // global index of the first local element on each dim
  int32_t N0, N1, N2;        // global extents of the *original* axes 0, 1, 2
  int32_t mode;              // see kspace.cu
  int32_t ntable;            // mode 1: number of samples of the power-spectrum table
  float box0, box1, box2;    // physical box lengths along original axes
  float p0, p1, p2, p3;      // mode 0: amplitude, index, cut-off, normalisation; mode 1: log k0, d log k, -, normalisation
};
int launch_kspace(const KSpaceDesc& d, const void* in, void* out0, void* out1, void* out2, const float* table,
                  void* stream);

// ---- misc --------------------------------------------------------------------------------------------
const char* last_error_message();
void set_last_error(const char* msg);

}  // namespace jdb
