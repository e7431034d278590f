// Peer-visible ("symmetric") device memory for one process per GPU on one node.
//
// Every rank allocates a data region and a small flag region with cudaMalloc,
// exports both as CUDA IPC handles, and opens the handles of all other ranks.
// The result is a table of device pointers -- one per rank -- that kernels use
// for plain peer loads/stores over NVLink.  This plays the role that cuDecomp's
// internal NCCL/NVSHMEM work buffers play in the reference
// (src/csrc/grid_descriptor_mgr.cc:15-27, src/csrc/fft.cu:14-70): it is created
// once, cached, and torn down in finalize().
//
// The status block is mapped pinned host memory: kernels write an error record
// into it directly, and the host can look at it without synchronising a stream.
#include <cuda_runtime.h>

#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "arena.h"

namespace jdb {

static void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    // clear the sticky-free error so that later calls report their own status
    cudaGetLastError();
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
  }
}

SymmetricArena::SymmetricArena(size_t bytes, int world, int me) : bytes_(bytes), world_(world), me_(me) {
  if (world < 1 || world > JD_MAX_PEERS || me < 0 || me >= world) throw std::runtime_error("arena: bad world/rank");
  data_.assign(world, nullptr);
  flags_.assign(world, nullptr);
  // 2 MiB granularity keeps every carve-out generously aligned
  bytes_ = (bytes + ((size_t)2 << 20) - 1) / ((size_t)2 << 20) * ((size_t)2 << 20);
  check(cudaMalloc(&data_[me], bytes_), "cudaMalloc(arena data)");
  check(cudaMalloc(&flags_[me], kFlagBytes), "cudaMalloc(arena flags)");
  check(cudaMemset(flags_[me], 0, kFlagBytes), "cudaMemset(arena flags)");
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
}

std::string SymmetricArena::export_handles() const {
  exported_ = true;
  cudaIpcMemHandle_t h[2];
  check(cudaIpcGetMemHandle(&h[0], data_[me_]), "cudaIpcGetMemHandle(data)");
  check(cudaIpcGetMemHandle(&h[1], flags_[me_]), "cudaIpcGetMemHandle(flags)");
  return std::string(reinterpret_cast<const char*>(h), sizeof(h));
}

void SymmetricArena::open_peers(const std::vector<std::string>& handles) {
  if ((int)handles.size() != world_) throw std::runtime_error("arena: need one handle blob per rank");
  for (int p = 0; p < world_; ++p) {
    if (p == me_) continue;
    if (handles[p].size() != 2 * sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("arena: malformed handle blob");
    cudaIpcMemHandle_t h[2];
    std::memcpy(h, handles[p].data(), sizeof(h));
    check(cudaIpcOpenMemHandle(&data_[p], h[0], cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle(data)");
    check(cudaIpcOpenMemHandle(&flags_[p], h[1], cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle(flags)");
    opened_ = true;
  }
}

void SymmetricArena::close_peers() {
  // Importers must close their mappings before the owner frees the memory, so
  // tear-down is two-phase: every rank closes its peers' handles, the ranks
  // synchronise on the host, and only then does each rank free its own block.
  cudaDeviceSynchronize();
  for (int p = 0; p < world_; ++p) {
    if (p == me_) continue;
    if (data_[p]) cudaIpcCloseMemHandle(data_[p]);
    if (flags_[p]) cudaIpcCloseMemHandle(flags_[p]);
    data_[p] = flags_[p] = nullptr;
  }
  cudaGetLastError();
}

void SymmetricArena::close(bool free_own) {
  if (closed_) return;
  closed_ = true;
  close_peers();
  // Peers may still have this rank's blocks mapped (and be storing into them or polling the flags)
  // unless the ranks synchronised on the host after phase 1.  Freeing exported memory that an importer
  // still uses is undefined, so without that guarantee the blocks are left to process tear-down.
  if (free_own || world_ == 1 || !exported_) {
    if (data_[me_]) cudaFree(data_[me_]);
    if (flags_[me_]) cudaFree(flags_[me_]);
  }
  data_[me_] = flags_[me_] = nullptr;
  cudaGetLastError();
}

SymmetricArena::~SymmetricArena() { close(false); }

HostStatus::HostStatus() {
  void* h = nullptr;
  check(cudaHostAlloc(&h, sizeof(StatusBlock), cudaHostAllocMapped), "cudaHostAlloc(status)");
  host_ = static_cast<StatusBlock*>(h);
  std::memset(host_, 0, sizeof(StatusBlock));
  void* d = nullptr;
  check(cudaHostGetDevicePointer(&d, h, 0), "cudaHostGetDevicePointer(status)");
  dev_ = static_cast<StatusBlock*>(d);
}

HostStatus::~HostStatus() {
  if (host_) cudaFreeHost(host_);
  cudaGetLastError();
}

void HostStatus::clear() { std::memset(host_, 0, sizeof(StatusBlock)); }

}  // namespace jdb
