// Peer-visible device memory and the host-mapped status block (see arena.cpp).
#pragma once
#include <cstddef>
#include <string>
#include <vector>

#include "status.h"
#include "tile_map.h"

namespace jdb {

class SymmetricArena {
 public:
  static constexpr size_t kFlagBytes = 4096;
  SymmetricArena(size_t bytes, int world, int me);
  ~SymmetricArena();
  SymmetricArena(const SymmetricArena&) = delete;
  SymmetricArena& operator=(const SymmetricArena&) = delete;

  std::string export_handles() const;                         // opaque blob to all-gather
  void open_peers(const std::vector<std::string>& handles);  // blobs of all ranks, indexed by rank
  void close_peers();  // phase 1 of tear-down: unmap the other ranks' memory
  // phase 2: free this rank's memory (also runs phase 1 if still needed).  Freeing is only safe once every
  // importer has unmapped the block, i.e. after the ranks met on the host; a rank that leaves on its own
  // passes free_own = false and lets process tear-down reclaim the memory.
  void close(bool free_own = true);

  size_t bytes() const { return bytes_; }
  int world() const { return world_; }
  int me() const { return me_; }
  void* data(int peer) const { return data_.at(peer); }
  void* flags(int peer) const { return flags_.at(peer); }

 private:
  size_t bytes_;
  int world_, me_;
  bool opened_ = false, closed_ = false;
  mutable bool exported_ = false;  // handles were handed out: other processes may map this rank's blocks
  std::vector<void*> data_, flags_;
};

class HostStatus {
 public:
  HostStatus();
  ~HostStatus();
  HostStatus(const HostStatus&) = delete;
  HostStatus& operator=(const HostStatus&) = delete;
  StatusBlock* host() const { return host_; }
  StatusBlock* device() const { return dev_; }
  void clear();

 private:
  StatusBlock* host_ = nullptr;
  StatusBlock* dev_ = nullptr;
};

}  // namespace jdb
