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
// Launch on `stream`.  Returns a Status; CUDA launch errors are reported as JD_ERR_CUDA
// and the message is available from last_error_message().
int launch_pass(const PassDesc& d, void* stream, StatusBlock* status);
// Threads per block the launcher will use for this descriptor (0 if invalid).
int pass_threads(const PassDesc& d);
size_t pass_smem_bytes(const PassDesc& d);
// Specialised kernel for power-of-two lengths 128..4096 (fft_fast.cu)
bool fast_pass_eligible(const PassDesc& d);
int launch_fast_pass(const PassDesc& d, void* stream);

// ---- cross-rank signalling (signal.cu) ---------------------------------------------------------------
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
};
struct HaloDesc {
  int32_t S0, S1, S2, B;   // padded local block (B = batch)
  int32_t elem_bytes;      // 4, 8, 16
  int32_t nregions;
  int32_t accumulate;      // unpack: 0 overwrite, 1 add
  int32_t is_f64;          // accumulate arithmetic: 1 = float64/complex128, 0 = float32/complex64
  HaloRegion reg[8];
  void* stage[JD_MAX_PEERS];  // staging buffers (peer-visible)
  const void* src;            // local block read by pack
  void* dst;                  // local block written by unpack
};
// pack: for every region copy src[region] -> stage[reg.peer] + stage_off (peer stores)
int launch_halo_pack(const HaloDesc& d, void* stream);
// unpack: for every region dst[region] (=|+=) stage[reg.peer] + stage_off (local loads); peer == -1 -> zero (overwrite mode)
int launch_halo_unpack(const HaloDesc& d, void* stream);

// ---- particle-mesh kernels (cic.cu) ---------------------------------------------------------------------
// pos: [n,3] positions in units of cells relative to the origin of the local (padded) mesh
int launch_cic_paint(const float* pos, const float* weight, long long n, float* mesh, int S0, int S1, int S2,
                     int wrap0, int wrap1, int wrap2, void* stream);
int launch_cic_readout(const float* pos, long long n, const float* mesh, float* out, int S0, int S1, int S2, int wrap0,
                       int wrap1, int wrap2, void* stream);
// gradient of paint w.r.t. positions: gpos[n,3] = sum over 8 cells of gmesh * d(weight)/d(pos) * w
int launch_cic_paint_grad_pos(const float* pos, const float* weight, long long n, const float* gmesh, float* gpos,
                              int S0, int S1, int S2, int wrap0, int wrap1, int wrap2, void* stream);

// ---- k-space elementwise kernels (kspace.cu) --------------------------------------------------------------
struct KSpaceDesc {
  // local block of the rotated FFT output: dims (L0, L1, L2) hold original axes (1, 2, 0)
  int32_t L0, L1, L2;
  int32_t off0, off1, off2;  // global index of the first local element on each dim
  int32_t N0, N1, N2;        // global extents of the *original* axes 0, 1, 2
  int32_t mode;              // see kspace.cu
  float box0, box1, box2;    // physical box lengths along original axes
  float p0, p1, p2, p3;      // mode-specific parameters
};
int launch_kspace(const KSpaceDesc& d, const void* in, void* out0, void* out1, void* out2, void* stream);

// ---- misc --------------------------------------------------------------------------------------------
const char* last_error_message();
void set_last_error(const char* msg);

}  // namespace jdb
