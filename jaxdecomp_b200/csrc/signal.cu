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
// seen} in the status block and returns normally.  It never traps or spins forever.
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

__device__ void bounded_wait(const uint32_t* slot, uint32_t epoch, long long timeout_ns, int peer, StatusBlock* st) {
  const unsigned long long t0 = globaltimer_ns();
  uint32_t seen = 0;
  unsigned spins = 0;
  for (;;) {
    seen = ld_acquire_sys(slot);
    if ((int32_t)(seen - epoch) >= 0) return;
    if ((++spins & 15u) == 0) {
      if ((long long)(globaltimer_ns() - t0) > timeout_ns) break;
      __nanosleep(100);
    }
  }
  if (st != nullptr && atomicCAS(&st->code, 0, (int)JD_ERR_TIMEOUT_PEER_SIGNAL) == 0) {
    st->peer = peer;
    st->expected = (int32_t)epoch;
    st->seen = (int32_t)seen;
    st->where = 100;
    __threadfence_system();
  }
}

__global__ void signal_barrier_kernel(PeerFlags pf, int me, int n, uint32_t* epoch_counter, uint32_t epoch_arg,
                                      long long timeout_ns, StatusBlock* st) {
  const int p = threadIdx.x;
  // The epoch normally lives in device memory and is advanced by the barrier
  // itself, so that a captured CUDA graph can be replayed: every rank runs the
  // same sequence of barriers and therefore counts identically.
  uint32_t epoch = epoch_arg;
  if (epoch_counter != nullptr) {
    epoch = *epoch_counter + 1;
    __syncwarp();
    if (p == 0) *epoch_counter = epoch;
  }
  if (p >= n) return;
  // everything this stream did before (including peer stores of the previous
  // kernel) is ordered before the flag
  __threadfence_system();
  st_release_sys(pf.flags[p] + me, epoch);
  bounded_wait(pf.flags[me] + p, epoch, timeout_ns, p, st);
}

__global__ void wait_only_kernel(uint32_t* my_flags, int n, uint32_t epoch, long long timeout_ns, StatusBlock* st) {
  const int p = threadIdx.x;
  if (p >= n) return;
  bounded_wait(my_flags + p, epoch, timeout_ns, p, st);
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
