// Status codes shared by host code and kernels.
//
// The reference library reports failures with COM-style HRESULT values and
// terminates the process on CUDA or MPI errors (src/csrc/include/checks.h:6-72).
// Here a kernel that detects a problem writes one of these codes into a status
// block and returns; the host turns it into a Python exception.  Nothing in
// this library calls exit() or traps on the device.
#pragma once
#include <cstdint>

namespace jdb {

enum Status : int32_t {
  JD_OK = 0,
  JD_CACHE_HIT = 1,          // informational: a plan was found in the cache
  JD_ERR_INVALID_ARG = -1,
  JD_ERR_CUDA = -2,
  JD_ERR_TIMEOUT_PEER_SIGNAL = -3,  // bounded wait on a peer's flag expired
  JD_ERR_STALE_EPOCH = -4,          // a flag is more than one barrier ahead of the epoch waited for
  JD_ERR_BOUNDS = -5,               // debug bounds check failed; access skipped
  JD_ERR_TIMEOUT_MBARRIER = -6,     // bounded wait on a local bulk-copy barrier expired
  JD_ERR_UNSUPPORTED = -7,
  JD_ERR_PEER_ABORTED = -8,         // a peer's bounded wait failed and it marked the whole group as aborted
};

inline const char* status_name(int32_t s) {
  switch (s) {
    case JD_OK: return "OK";
    case JD_CACHE_HIT: return "CACHE_HIT";
    case JD_ERR_INVALID_ARG: return "INVALID_ARG";
    case JD_ERR_CUDA: return "CUDA_ERROR";
    case JD_ERR_TIMEOUT_PEER_SIGNAL: return "TIMEOUT_PEER_SIGNAL";
    case JD_ERR_STALE_EPOCH: return "STALE_EPOCH";
    case JD_ERR_BOUNDS: return "BOUNDS";
    case JD_ERR_TIMEOUT_MBARRIER: return "TIMEOUT_MBARRIER";
    case JD_ERR_UNSUPPORTED: return "UNSUPPORTED";
    case JD_ERR_PEER_ABORTED: return "PEER_ABORTED";
    default: return "UNKNOWN";
  }
}

// One per process, in device memory that the host reads back after a stream
// synchronise.  A kernel records only the first failure (atomicCAS on code).
struct StatusBlock {
  int32_t code;      // Status
  int32_t peer;      // peer index involved, or -1
  int32_t expected;  // epoch or index expected
  int32_t seen;      // epoch or index observed
  int32_t where;     // kernel-specific location tag
  int32_t pad[3];
};

}  // namespace jdb
