// Process-wide runtime of the native backend: the peer-visible arena, the
// status block, the FFT tables and the plan cache with its executor.
//
// Counterpart of the reference's GridDescriptorManager singleton, which caches
// one executor per (gdims, pdims, precision, layout, backend) descriptor and
// owns the cuDecomp handle and workspaces
// (src/csrc/grid_descriptor_mgr.cc:15-144, include/grid_descriptor_mgr.h:20-67).
// Here a cached plan is a list of tile passes with symbolic buffer bindings;
// executing it is one call from Python that launches every pass and every
// cross-rank barrier on the caller's stream.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "arena.h"
#include "launch.h"

namespace jdb {

struct FftTables {
  const void* twiddle = nullptr;
  const void* tw_stage = nullptr;
  const void* chirp = nullptr;
  const void* bhat = nullptr;
};
FftTables get_fft_tables(int C, int M, int elem_bytes, bool device);
void clear_fft_tables();

enum BufferKind : int32_t {
  BUF_USER_IN = 0,   // the operand passed to execute()
  BUF_USER_OUT = 1,  // the result tensor passed to execute()
  BUF_SLOT_A = 2,    // arena slot 0 (peer visible)
  BUF_SLOT_B = 3,    // arena slot 1 (peer visible)
  // The result tensor when it lives in a peer-visible block that every rank allocated alike: peer p's
  // copy is peer_out[p] of execute().  An exchange pass stores straight into the other ranks' results,
  // so no copy out of a slot follows it; execute() puts one barrier before the pass (nobody may still
  // be using its result block from an earlier call) and one at the end (every store has landed).
  BUF_PEER_OUT = 4,
};
// Index of the arena slot a buffer kind names, or -1.
inline int slot_of(int kind) { return (kind == BUF_SLOT_A || kind == BUF_SLOT_B) ? kind - BUF_SLOT_A : -1; }

struct PlanStep {
  PassDesc desc;               // pointers of in/out are filled in at execution time
  int32_t in_kind = BUF_USER_IN;
  int32_t out_kind = BUF_USER_OUT;
  int32_t copy_only = 0;       // 1: plain device-to-device copy of copy_bytes from in to out
  long long copy_bytes = 0;
  int32_t group_ranks[JD_MAX_PEERS] = {0};  // arena rank of destination peer p (npeers entries)
  // Pipelining with the next step (set on an exchange pass that is followed by a local pass): the pass
  // is cut into pipe_chunks chunks along its axis pipe_role (2 = t, 3 = o); the next step is cut the same
  // way along its own pipe_role, and chunk k of the next step starts as soon as chunk k of this step has
  // arrived from every rank, while chunk k + 1 is still crossing NVLink.
  int32_t pipe_chunks = 0;
  int32_t pipe_role = 0;
  int32_t pipe_grid_limit = 0;  // blocks of each chunk of the exchange pass (0: one per tile)
};

struct Plan {
  std::vector<PlanStep> steps;
  long long slot_bytes = 0;  // bytes each arena slot must provide
  long long hits = 0;
};

class Runtime {
 public:
  Runtime(int world, int me);
  ~Runtime();

  // arena life cycle (collective: every rank calls with the same sizes)
  void create_arena(size_t slot_bytes);
  std::string export_handles() const;
  void open_peers(const std::vector<std::string>& handles);
  void close_peers();   // collective tear-down, phase 1 (host barrier needed before destroy_arena)
  // collective = true: the caller guarantees that every rank ran close_peers() and the ranks then met on the
  // host, so the exported blocks can be freed; false: a rank leaving alone only unmaps its imports.
  void destroy_arena(bool collective = true);
  size_t slot_bytes() const { return slot_bytes_; }
  bool has_arena() const { return (bool)arena_; }
  void* slot_ptr(int slot, int peer) const;
  uint32_t* flag_ptr(int peer) const;

  // plan cache
  int find_plan(const std::string& key);  // -1 if absent; counts a hit otherwise
  int add_plan(const std::string& key, Plan plan);
  const Plan& plan(int id) const { return plans_.at(id); }
  size_t num_plans() const { return plans_.size(); }
  long long cache_hits() const { return hits_; }
  long long cache_misses() const { return misses_; }
  void clear_plans();

  // execution
  // peer_out: base address of the result block on every arena rank (world entries), needed by plans
  // that have a BUF_PEER_OUT step; peer_out[me] must equal out.
  int execute(int plan_id, const void* in, void* out, void* stream, void* const* peer_out = nullptr);
  // 0 disables the pipelined execution of plans (every step then runs in order on the caller's stream)
  void set_pipelining(bool on) { pipelining_ = on; }
  bool pipelining() const { return pipelining_; }
  long long pipelined_sections() const { return pipelined_sections_; }
  int barrier(void* stream);
  // pack -> (zero fill) -> barrier -> unpack through arena slot 0; copies src to dst first when they differ
  int halo(HaloDesc pack, HaloDesc unpack, const HaloDesc* zero, const void* src, void* dst, long long bytes,
           void* stream);
  // In-place exchange on blocks that are themselves peer visible (block[p]: the block of arena rank p,
  // same shape on every rank): barrier (nobody still reads the halos that are about to be overwritten),
  // one kernel that stores every slab at its final place in the neighbours' blocks (+ zero fill of halos
  // without a source), barrier (everything has landed).  No staging slab, no unpack pass.
  int halo_direct(HaloDesc push, const HaloDesc* zero, void* const* block, void* stream);
  long long barriers_issued() const { return host_epoch_; }
  long long launches() const { return launches_; }

  // status
  StatusBlock read_status() const;
  void clear_status();
  StatusBlock* status_device() const { return status_ ? status_->device() : nullptr; }

  // synchronous access to one word of this rank's flag region (tests of the stale-epoch and abort paths)
  int poke_flag(int word, uint32_t value);
  int peek_flag(int word, uint32_t* value) const;

  void set_timeout_ms(long long ms) { timeout_ns_ = ms * 1000000LL; }
  int world() const { return world_; }
  int me() const { return me_; }

 private:
  int world_, me_;
  std::unique_ptr<SymmetricArena> arena_;
  std::unique_ptr<HostStatus> status_;
  size_t slot_bytes_ = 0;
  long long timeout_ns_ = 10000000000LL;
  // hazard tracking (identical on every rank because all ranks issue the same sequence)
  long long host_epoch_ = 0;
  void* const* cur_peer_out_ = nullptr;    // peer_out of the execute() call in progress
  long long slot_written_[2] = {-1, -1};  // epoch during which peers last wrote the slot
  long long slot_read_[2] = {-1, -1};     // epoch during which this rank last read the slot
  std::map<std::string, int> plan_index_;
  std::vector<Plan> plans_;
  long long hits_ = 0, misses_ = 0, launches_ = 0;
  // pipelined execution: one extra high-priority stream for the exchange chunks and one event per chunk
  bool pipelining_ = true;
  long long pipelined_sections_ = 0;
  void* side_stream_ = nullptr;
  void* fork_event_ = nullptr;
  std::vector<void*> chunk_events_;
  int ensure_pipe_resources(int chunks);
  void release_pipe_resources();
  int sync_before(const PlanStep& st, void* stream);
  int launch_step(const Plan& pl, int plan_id, size_t index, const PassDesc* chunk_desc, const void* in, void* out,
                  void* stream);
  void fill_pointers(const PlanStep& st, PassDesc& d, const void* in, void* out) const;
  int run_pipelined(Plan& pl, int plan_id, size_t index, const void* in, void* out, void* stream);
};

}  // namespace jdb
