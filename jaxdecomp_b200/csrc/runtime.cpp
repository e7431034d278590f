// Runtime: arena life cycle, plan cache and the plan executor (see runtime.h).
#include "runtime.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <stdexcept>

#include "trace.h"

namespace jdb {

// flag region layout (uint32 words): [0, JD_MAX_PEERS) epoch slots, word 64: this rank's epoch counter
static constexpr int kEpochCounterWord = 64;

Runtime::Runtime(int world, int me) : world_(world), me_(me) {
  if (world < 1 || world > JD_MAX_PEERS || me < 0 || me >= world) throw std::runtime_error("runtime: bad world/rank");
  JD_TRACE_INFO("runtime", "create world=%d rank=%d", world, me);
}

Runtime::~Runtime() { destroy_arena(); }

void Runtime::create_arena(size_t slot_bytes) {
  destroy_arena();
  if (!status_) status_.reset(new HostStatus());
  // round the slot so that the second slot stays 2 MiB aligned
  const size_t gran = (size_t)2 << 20;
  slot_bytes_ = (slot_bytes + gran - 1) / gran * gran;
  arena_.reset(new SymmetricArena(2 * slot_bytes_, world_, me_));
  host_epoch_ = 0;
  slot_written_[0] = slot_written_[1] = -1;
  slot_read_[0] = slot_read_[1] = -1;
  JD_TRACE_INFO("runtime", "arena created: 2 slots x %zu bytes", slot_bytes_);
}

std::string Runtime::export_handles() const {
  if (!arena_) throw std::runtime_error("runtime: no arena");
  return arena_->export_handles();
}

void Runtime::open_peers(const std::vector<std::string>& handles) {
  if (!arena_) throw std::runtime_error("runtime: no arena");
  arena_->open_peers(handles);
}

void Runtime::close_peers() {
  if (arena_) arena_->close_peers();
}

void Runtime::destroy_arena() {
  if (arena_) {
    JD_TRACE_INFO("runtime", "arena destroyed");
    arena_->close();
    arena_.reset();
  }
  slot_bytes_ = 0;
}

void* Runtime::slot_ptr(int slot, int peer) const {
  if (!arena_) throw std::runtime_error("runtime: no arena");
  return static_cast<char*>(arena_->data(peer)) + (size_t)slot * slot_bytes_;
}

uint32_t* Runtime::flag_ptr(int peer) const {
  if (!arena_) throw std::runtime_error("runtime: no arena");
  return static_cast<uint32_t*>(arena_->flags(peer));
}

int Runtime::find_plan(const std::string& key) {
  auto it = plan_index_.find(key);
  if (it == plan_index_.end()) {
    ++misses_;
    return -1;
  }
  ++hits_;
  ++plans_[it->second].hits;
  return it->second;
}

int Runtime::add_plan(const std::string& key, Plan plan) {
  plans_.push_back(std::move(plan));
  const int id = (int)plans_.size() - 1;
  plan_index_[key] = id;
  JD_TRACE_VERBOSE("runtime", "plan %d cached: %s (%zu steps)", id, key.c_str(), plans_[id].steps.size());
  return id;
}

void Runtime::clear_plans() {
  plans_.clear();
  plan_index_.clear();
}

int Runtime::barrier(void* stream) {
  if (world_ == 1) return JD_OK;
  if (!arena_) throw std::runtime_error("runtime: barrier without arena");
  StepProfiler& prof = StepProfiler::instance();
  struct Scope {
    StepProfiler& p;
    void* s;
    bool on;
    ~Scope() {
      if (on) p.stop(s);
    }
  } scope{prof, stream, prof.mode() != StepProfiler::OFF};
  if (scope.on) prof.start("barrier", stream);
  PeerFlags pf;
  for (int p = 0; p < JD_MAX_PEERS; ++p) pf.flags[p] = p < world_ ? flag_ptr(p) : nullptr;
  ++host_epoch_;
  ++launches_;
  return launch_signal_barrier(pf, me_, world_, flag_ptr(me_) + kEpochCounterWord, 0, timeout_ns_, stream,
                               status_device());
}

int Runtime::execute(int plan_id, const void* in, void* out, void* stream) {
  Plan& pl = plans_.at(plan_id);
  if (world_ > 1 || pl.slot_bytes > 0) {
    if (!arena_ || (size_t)pl.slot_bytes > slot_bytes_) {
      set_last_error("runtime: arena missing or too small for this plan");
      return JD_ERR_INVALID_ARG;
    }
  }
  for (PlanStep& st : pl.steps) {
    const int is = st.in_kind - BUF_SLOT_A, os = st.out_kind - BUF_SLOT_A;
    // read-after-remote-write: everybody's stores into the slot must have landed
    if (is >= 0 && slot_written_[is] == host_epoch_ && world_ > 1) {
      int rc = barrier(stream);
      if (rc != JD_OK) return rc;
    }
    // write-after-read: nobody may still be reading the slot from an earlier step
    if (os >= 0 && slot_read_[os] == host_epoch_ && world_ > 1) {
      int rc = barrier(stream);
      if (rc != JD_OK) return rc;
    }
    const void* src = st.in_kind == BUF_USER_IN ? in : (st.in_kind == BUF_USER_OUT ? out : slot_ptr(is, me_));
    StepProfiler& prof = StepProfiler::instance();
    const bool profiling = prof.mode() != StepProfiler::OFF;
    if (profiling) {
      char name[96];
      if (st.copy_only)
        std::snprintf(name, sizeof(name), "plan%d.step%d copy", plan_id, (int)(&st - &pl.steps[0]));
      else
        std::snprintf(name, sizeof(name), "plan%d.step%d %s C=%d peers=%d", plan_id, (int)(&st - &pl.steps[0]),
                      st.desc.fft_mode == JD_COPY ? "copy-pass" : "fft-pass", st.desc.C, st.desc.npeers);
      prof.start(name, stream);
    }
    if (st.copy_only) {
      void* dst = st.out_kind == BUF_USER_OUT ? out : slot_ptr(os, me_);
      cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)st.copy_bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
      if (e != cudaSuccess) {
        set_last_error(cudaGetErrorString(e));
        return JD_ERR_CUDA;
      }
    } else {
      PassDesc d = st.desc;
      d.in = src;
      for (int p = 0; p < d.npeers; ++p) {
        if (st.out_kind == BUF_USER_OUT)
          d.out[p] = out;
        else
          d.out[p] = slot_ptr(os, st.group_ranks[p]);
      }
      int rc = launch_pass(d, stream, status_device());
      if (rc != JD_OK) return rc;
    }
    if (profiling) prof.stop(stream);
    ++launches_;
    if (is >= 0) slot_read_[is] = host_epoch_;
    if (os >= 0) slot_written_[os] = host_epoch_;
  }
  return JD_OK;
}

int Runtime::halo(HaloDesc pack, HaloDesc unpack, const HaloDesc* zero, const void* src, void* dst, long long bytes,
                  void* stream) {
  const int slot = 0;
  if (!arena_) {
    set_last_error("runtime: halo exchange without arena");
    return JD_ERR_INVALID_ARG;
  }
  int rc;
  if (src != dst) {
    cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
    if (e != cudaSuccess) {
      set_last_error(cudaGetErrorString(e));
      return JD_ERR_CUDA;
    }
    ++launches_;
  }
  // nobody may still be reading the staging slot from an earlier operation
  if (world_ > 1 && slot_read_[slot] == host_epoch_ && (rc = barrier(stream)) != JD_OK) return rc;
  pack.src = src;
  pack.dst = dst;
  for (int p = 0; p < JD_MAX_PEERS; ++p) pack.stage[p] = p < world_ ? slot_ptr(slot, p) : nullptr;
  if ((rc = launch_halo_pack(pack, stream)) != JD_OK) return rc;
  ++launches_;
  slot_written_[slot] = host_epoch_;
  if (zero != nullptr) {
    HaloDesc z = *zero;
    z.src = src;
    z.dst = dst;
    for (int p = 0; p < JD_MAX_PEERS; ++p) z.stage[p] = nullptr;
    if ((rc = launch_halo_unpack(z, stream)) != JD_OK) return rc;
    ++launches_;
  }
  if (world_ > 1 && (rc = barrier(stream)) != JD_OK) return rc;
  unpack.src = src;
  unpack.dst = dst;
  for (int p = 0; p < JD_MAX_PEERS; ++p) unpack.stage[p] = p < world_ ? slot_ptr(slot, p) : nullptr;
  if ((rc = launch_halo_unpack(unpack, stream)) != JD_OK) return rc;
  ++launches_;
  slot_read_[slot] = host_epoch_;
  return JD_OK;
}

StatusBlock Runtime::read_status() const {
  StatusBlock s{};
  if (status_) s = *status_->host();
  return s;
}

void Runtime::clear_status() {
  if (status_) status_->clear();
}

}  // namespace jdb
