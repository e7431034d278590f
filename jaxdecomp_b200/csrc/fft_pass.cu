// The tile-pass kernel for sm_100a: strided tile load -> batched 1-D FFT in
// shared memory -> scatter into the destination layout on the destination
// rank.  One kernel covers
//   * the three transform passes of pfft3d / pifft3d, each fused with the
//     pencil transpose that follows it: result tiles are written with plain
//     peer stores straight into the next pencil buffer of the owning GPU
//     (NVLink / NVSwitch), at their final, rotated position -- there is no
//     pack buffer, no all-to-all call and no separate transpose kernel;
//   * strided transforms for the non-contiguous layout mode;
//   * arbitrary lengths through Bluestein's algorithm done entirely in shared memory;
//   * the stand-alone pencil transposes (copy mode).
// The reference does the same work with cufftXtExec + cudecompTranspose* calls
// (src/csrc/fft.cu:460-535) or XLA's fft + all_to_all + transpose
// (src/jaxdecomp/_src/jax/fft.py:94-135).
//
// Rows are fetched either with ordinary coalesced loads or, when the rows are
// 16-byte aligned and contiguous, with bulk asynchronous copies
// (cp.async.bulk, the 1-D TMA path) that complete on an mbarrier; the wait on
// that barrier is bounded and reports through the status block.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <string>

#include "launch.h"
#include "tile_ops.h"

namespace jdb {

static thread_local std::string g_last_error;
const char* last_error_message() { return g_last_error.c_str(); }
void set_last_error(const char* msg) { g_last_error = msg ? msg : ""; }

__device__ __forceinline__ void report_status(StatusBlock* st, int code, int peer, int expected, int seen, int where) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0, code) == 0) {
    st->peer = peer;
    st->expected = expected;
    st->seen = seen;
    st->where = where;
    __threadfence_system();
  }
}

// ---- bulk asynchronous row fetch ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Fetch the rows of a tile with one bulk copy per row.  Returns false if the
// bounded wait expired (the status block then holds JD_ERR_TIMEOUT_MBARRIER).
template <typename E>
__device__ bool tile_load_bulk(const PassDesc& d, E* tile, uint64_t* bar, int o, int t0, int b, StatusBlock* st) {
  const int rows = min(d.T, d.Tn - t0);
  const uint32_t row_bytes = (uint32_t)d.C * sizeof(E);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_expect_tx(bar, row_bytes * (uint32_t)rows);
    const E* in = (const E*)d.in + (long long)o * d.is_o + (long long)b * d.is_b;
    for (int r = 0; r < rows; ++r) bulk_g2s(tile + (long long)r * d.pitch, in + (long long)(t0 + r) * d.is_t, row_bytes, bar);
  }
  // ragged last tile: rows past the end are zero
  if (rows < d.T) {
    E zero;
    memset(&zero, 0, sizeof(E));
    for (int e = threadIdx.x; e < (d.T - rows) * d.C; e += blockDim.x) {
      const int r = rows + e / d.C, c = e % d.C;
      tile[(long long)r * d.pitch + c] = zero;
    }
  }
  // bounded wait: ~2^22 polls with back-off is several hundred milliseconds
  bool done = false;
  for (int spin = 0; spin < (1 << 22); ++spin) {
    if (mbar_try_wait(bar, 0)) {
      done = true;
      break;
    }
    if (spin > 64) __nanosleep(64);
  }
  if (!done) {
    report_status(st, JD_ERR_TIMEOUT_MBARRIER, -1, (int)(row_bytes * rows), 0, 1);
    // give copies still in flight a last, bounded chance to land before the block leaves
    for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(bar, 0); ++spin) __nanosleep(256);
  }
  // the whole block takes the same decision
  return __syncthreads_and(done ? 1 : 0) != 0;
}

// ---- the transform on the tile ----------------------------------------------------------------------------
template <typename E, int ITERS>
__device__ __forceinline__ void fft_rows(const PassDesc& d, E* tile) {
  const int M = d.M;
  const int logM = d.logW;
  const int upr = M >> 3;
  const int lupr = logM - 3;
  const int units = d.T * upr;
  const int pad = d.intra_pad;
  const E* __restrict__ tw = (const E*)d.twiddle;
  const int ns = fft_num_stages(logM);
  // the (row, butterfly) a thread owns is the same in every stage
  E* rowp[ITERS];
  int jj[ITERS];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int u = it * blockDim.x + threadIdx.x;
    rowp[it] = tile + (u >> lupr) * d.pitch;
    jj[it] = u < units ? (u & (upr - 1)) : -1;
  }
  int logLs = 0;
  for (int s = 0; s < ns; ++s) {
    const int rl = fft_stage_radix_log(logM, s);
    E a[ITERS][8];
#pragma unroll
    for (int it = 0; it < ITERS; ++it)
      if (jj[it] >= 0) stage_read(rowp[it], M, jj[it], a[it], pad);
    __syncthreads();
#pragma unroll
    for (int it = 0; it < ITERS; ++it)
      if (jj[it] >= 0) stage_compute_write(rowp[it], logM, jj[it], logLs, rl, tw, a[it], pad);
    __syncthreads();
    logLs += rl;
  }
}

template <typename E, bool FFT, int ITERS>
__global__ void __launch_bounds__(FFT ? (sizeof(E) == 16 ? 256 : 512) : 256,
                                  FFT ? (ITERS == 1 ? 3 : (ITERS == 2 ? 2 : 1)) : 4) tile_pass_kernel(const __grid_constant__ PassDesc d, StatusBlock* status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ uint64_t bar;
  E* tile = (E*)smem_raw;
  if (pass_aborted(d)) return;

  const int tiles_t = (d.Tn + d.T - 1) / d.T;
  const int tiles_c = FFT ? 1 : (d.C + d.Cc - 1) / d.Cc;
  long long bid = blockIdx.x;
  const int cc = (int)(bid % tiles_c);
  bid /= tiles_c;
  const int tt = (int)(bid % tiles_t);
  const int o = (int)(bid / tiles_t);
  const int b = blockIdx.y;
  const int t0 = tt * d.T, c0 = cc * d.Cc;

  if (FFT && d.use_bulk) {
    if (!tile_load_bulk<E>(d, tile, &bar, o, t0, b, status)) return;
    tile_fixup_after_bulk<E>(d, tile, threadIdx.x, blockDim.x);
  } else {
    tile_load<E>(d, tile, o, t0, c0, b, threadIdx.x, blockDim.x);
  }
  __syncthreads();
  if constexpr (FFT) {
    fft_rows<E, ITERS>(d, tile);
    if (d.fft_mode == JD_FFT_BLUESTEIN) {
      bluestein_filter<E>(d, tile, threadIdx.x, blockDim.x);
      __syncthreads();
      fft_rows<E, ITERS>(d, tile);
    }
  }
  tile_store<E>(d, tile, o, t0, c0, b, threadIdx.x, blockDim.x);
}

// ---- host side ------------------------------------------------------------------------------------------------
// Threads per block: T*M/8 butterflies spread over 1, 2 or 4 rounds per thread,
// at most 512 threads for 8-byte elements and 256 for 16-byte ones (register budget).
static int fft_iters(const PassDesc& d) {
  const long long units = (long long)d.T * (d.M >> 3);
  const long long cap = d.elem_bytes == 16 ? 256 : 512;
  for (int it : {1, 2, 4}) {
    const long long nt = (units + it - 1) / it;
    if (nt <= cap) return it;
  }
  return 0;
}

int pass_threads(const PassDesc& d) {
  if (d.fft_mode == JD_COPY) return 256;
  const long long units = (long long)d.T * (d.M >> 3);
  const int it = fft_iters(d);
  if (it == 0) return 0;
  long long nt = (units + it - 1) / it;
  nt = (nt + 31) / 32 * 32;
  return (int)nt;
}

size_t pass_smem_bytes(const PassDesc& d) { return (size_t)d.T * d.pitch * d.elem_bytes; }

template <typename E, bool FFT, int ITERS>
static int launch_t(const PassDesc& d, cudaStream_t stream, StatusBlock* status) {
  const int nt = pass_threads(d);
  if (nt <= 0) {
    set_last_error("tile pass: tile too large for one thread block (reduce T)");
    return JD_ERR_INVALID_ARG;
  }
  const size_t smem = pass_smem_bytes(d);
  // 227 KB is the per-block limit including the kernel's small static part
  constexpr size_t kMaxDynSmem = 226 * 1024;
  if (smem > kMaxDynSmem) {
    set_last_error("tile pass: tile exceeds the shared memory of one block");
    return JD_ERR_INVALID_ARG;
  }
  auto kern = tile_pass_kernel<E, FFT, ITERS>;
  static bool configured = false;  // one flag per template instantiation
  if (smem > 48 * 1024 && !configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxDynSmem);
    if (e != cudaSuccess) {
      set_last_error(cudaGetErrorString(e));
      return JD_ERR_CUDA;
    }
    configured = true;
  }
  const long long tiles_t = (d.Tn + d.T - 1) / d.T;
  const long long tiles_c = FFT ? 1 : (d.C + d.Cc - 1) / d.Cc;
  const long long nblocks = tiles_t * tiles_c * d.On;
  if (nblocks > 2147483647LL || d.B > 65535) {
    set_last_error("tile pass: grid too large");
    return JD_ERR_INVALID_ARG;
  }
  dim3 grid((unsigned)nblocks, (unsigned)d.B, 1);
  kern<<<grid, nt, smem, stream>>>(d, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return JD_ERR_CUDA;
  }
  return JD_OK;
}

int launch_pass(const PassDesc& d, void* stream_, StatusBlock* status) {
  int rc = validate_pass(d);
  if (rc != JD_OK) {
    set_last_error("tile pass: invalid descriptor");
    return rc;
  }
  cudaStream_t stream = (cudaStream_t)stream_;
  if (fast_pass_eligible(d)) {
    const char* off = std::getenv("JD_B200_FAST");
    if (!(off && off[0] == '0')) return launch_fast_pass(d, stream_);
  }
  if (d.fft_mode == JD_FFT_MIXED) return launch_mixed_pass(d, stream_);
  if (d.fft_mode == JD_COPY) {
    if (copy_fast_eligible(d)) {
      const char* off = std::getenv("JD_B200_COPY_FAST");
      if (!(off && off[0] == '0')) return launch_copy_fast(d, stream_);
    }
    if (d.elem_bytes == 4) return launch_t<float, false, 1>(d, stream, status);
    if (d.elem_bytes == 8) return launch_t<cx<float>, false, 1>(d, stream, status);
    return launch_t<cx<double>, false, 1>(d, stream, status);
  }
  const int it = fft_iters(d);
  if (d.elem_bytes == 8) {
    if (it == 1) return launch_t<cx<float>, true, 1>(d, stream, status);
    if (it == 2) return launch_t<cx<float>, true, 2>(d, stream, status);
    return launch_t<cx<float>, true, 4>(d, stream, status);
  }
  if (it == 1) return launch_t<cx<double>, true, 1>(d, stream, status);
  if (it == 2) return launch_t<cx<double>, true, 2>(d, stream, status);
  return launch_t<cx<double>, true, 4>(d, stream, status);
}

}  // namespace jdb
