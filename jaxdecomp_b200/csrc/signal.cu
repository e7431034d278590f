// Stream-ordered cross-GPU barrier built from plain peer stores and bounded
// polling.  The reference gets its ordering implicitly from NCCL/MPI
// collectives (cudecompTranspose*, lax.all_to_all); the fused kernels of this
// library write directly into peer memory, so the only synchronisation needed
// is "everyone's stores of the previous pass have landed", which this provides.
//
// Protocol: every rank owns an array of 32-bit epoch slots, one per peer, in
// peer-visible memory.  A barrier with epoch e stores e into slot `me` of every
// peer (release, system scope) and then polls its own slots until each holds a
// value >= e (acquire, system scope).  Epochs only grow, so slots are never
// reset.  The wait is bounded by a wall-clock budget read from %globaltimer;
// when it expires the kernel records {TIMEOUT_PEER_SIGNAL, peer, expected,
// seen} in the status block, sets the abort word of every rank (so that no
// pass runs on incomplete data and every rank raises) and returns normally.
// It never traps or spins forever.
#include <cuda_runtime.h>

#include "launch.h"

namespace jdb {

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Result of a bounded wait: 0 when the slot reached the epoch, else the Status that ended it.
//   * TIMEOUT_PEER_SIGNAL: the wall-clock budget ran out;
//   * STALE_EPOCH: the slot is more than one barrier ahead of the epoch waited for.  A peer signals
//     barrier e+1 only after it left barrier e, and it cannot leave barrier e+1 before this rank
//     signalled e+1, so a healthy slot is never ahead by more than one: a larger lead means that the
//     ranks no longer count the same barriers (a replayed or skipped barrier, a corrupted slot);
//   * PEER_ABORTED: the rank's abort word was set by a peer whose own wait failed.
__device__ int bounded_wait(const uint32_t* slot, uint32_t epoch, long long timeout_ns, const uint32_t* abort_word,
                            uint32_t* seen_out) {
  const unsigned long long t0 = globaltimer_ns();
  uint32_t seen = 0;
  unsigned spins = 0;
  int rc = JD_ERR_TIMEOUT_PEER_SIGNAL;
  for (;;) {
    seen = ld_acquire_sys(slot);
    const int32_t lead = (int32_t)(seen - epoch);
    if (lead > 1) {
      rc = JD_ERR_STALE_EPOCH;
      break;
    }
    if (lead >= 0) {
      rc = JD_OK;
      break;
    }
    if ((++spins & 15u) == 0) {
      if (abort_word != nullptr && ld_acquire_sys(abort_word) != 0) {
        rc = JD_ERR_PEER_ABORTED;
        break;
      }
      if ((long long)(globaltimer_ns() - t0) > timeout_ns) break;
      __nanosleep(100);
    }
  }
  *seen_out = seen;
  return rc;
}

__device__ void record_status(StatusBlock* st, int code, int peer, uint32_t expected, uint32_t seen, int where) {
  if (st != nullptr && atomicCAS(&st->code, 0, code) == 0) {
    st->peer = peer;
    st->expected = (int32_t)expected;
    st->seen = (int32_t)seen;
    st->where = where;
    __threadfence_system();
  }
}

__global__ void signal_barrier_kernel(PeerFlags pf, int me, int n, uint32_t* epoch_counter, uint32_t epoch_arg,
                                      long long timeout_ns, StatusBlock* st) {
  const int p = threadIdx.x;
  uint32_t* abort_word = pf.flags[me] + kFlagAbortWord;
  // The epoch normally lives in device memory and is advanced by the barrier
  // itself, so that a captured CUDA graph can be replayed: every rank runs the
  // same sequence of barriers and therefore counts identically.
  uint32_t epoch = epoch_arg;
  if (epoch_counter != nullptr) {
    epoch = *epoch_counter + 1;
    __syncwarp();
    if (p == 0) *epoch_counter = epoch;
  }
  // A rank whose wait failed earlier (here or on a peer) takes no further part: its kernels return at
  // entry, it signals nothing, and the host raises at its next status check.
  const uint32_t aborted = ld_acquire_sys(abort_word);
  if (aborted != 0) {
    if (p == 0) record_status(st, JD_ERR_PEER_ABORTED, (int)aborted - 1, epoch, 0, 101);
    return;
  }
  if (p >= n) return;
  // everything this stream did before (including peer stores of the previous
  // kernel) is ordered before the flag
  __threadfence_system();
  st_release_sys(pf.flags[p] + me, epoch);
  uint32_t seen = 0;
  const int rc = bounded_wait(pf.flags[me] + p, epoch, timeout_ns, abort_word, &seen);
  if (rc != JD_OK) {
    record_status(st, rc, rc == JD_ERR_PEER_ABORTED ? (int)ld_acquire_sys(abort_word) - 1 : p, epoch, seen, 100);
    // The data this barrier was guarding is incomplete.  Mark this rank and every peer as aborted so
    // that no later pass computes on it and no rank returns a result as if nothing had happened.
    if (rc != JD_ERR_PEER_ABORTED)
      for (int q = 0; q < n; ++q) st_release_sys(pf.flags[q] + kFlagAbortWord, (uint32_t)me + 1);
  }
}

__global__ void wait_only_kernel(uint32_t* my_flags, int n, uint32_t epoch, long long timeout_ns, StatusBlock* st) {
  const int p = threadIdx.x;
  if (p >= n) return;
  uint32_t seen = 0;
  const int rc = bounded_wait(my_flags + p, epoch, timeout_ns, nullptr, &seen);
  if (rc != JD_OK) record_status(st, rc, p, epoch, seen, 100);
}

static int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return JD_ERR_CUDA;
  }
  return JD_OK;
}

int launch_signal_barrier(const PeerFlags& pf, int me, int n, uint32_t* epoch_counter, uint32_t epoch,
                          long long timeout_ns, void* stream, StatusBlock* status) {
  if (n < 1 || n > JD_MAX_PEERS || me < 0 || me >= n) return JD_ERR_INVALID_ARG;
  signal_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(pf, me, n, epoch_counter, epoch, timeout_ns, status);
  return check_launch();
}

int launch_wait_only(uint32_t* my_flags, int n, uint32_t epoch, long long timeout_ns, void* stream,
                     StatusBlock* status) {
  if (n < 1 || n > JD_MAX_PEERS) return JD_ERR_INVALID_ARG;
  wait_only_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(my_flags, n, epoch, timeout_ns, status);
  return check_launch();
}

}  // namespace jdb
