// Runtime: arena life cycle, plan cache and the plan executor (see runtime.h).
#include "runtime.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <stdexcept>
#include <vector>

#include "trace.h"

namespace jdb {

static constexpr int kEpochCounterWord = kFlagEpochCounterWord;

Runtime::Runtime(int world, int me) : world_(world), me_(me) {
  if (world < 1 || world > JD_MAX_PEERS || me < 0 || me >= world) throw std::runtime_error("runtime: bad world/rank");
  JD_TRACE_INFO("runtime", "create world=%d rank=%d", world, me);
}

Runtime::~Runtime() {
  release_pipe_resources();
  destroy_arena(false);
}

void Runtime::create_arena(size_t slot_bytes) {
  destroy_arena(true);  // regrowth is collective: the caller closed the peers' handles and met them on the host
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

void Runtime::destroy_arena(bool collective) {
  if (arena_) {
    JD_TRACE_INFO("runtime", "arena destroyed (%s)", collective ? "collective" : "local: exported blocks kept");
    arena_->close(collective);
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

// ---- plan execution ------------------------------------------------------------------------------------
// Hazards between steps are tracked per arena slot with the count of barriers issued so far (identical
// on every rank, because all ranks issue the same sequence): a slot that peers wrote since the last
// barrier must not be read, and a slot that this rank read since the last barrier must not be written by
// peers, before another barrier has passed.
int Runtime::sync_before(const PlanStep& st, void* stream) {
  if (world_ <= 1) return JD_OK;
  const int is = slot_of(st.in_kind), os = slot_of(st.out_kind);
  // read-after-remote-write: everybody's stores into the slot must have landed
  if (is >= 0 && slot_written_[is] == host_epoch_) {
    int rc = barrier(stream);
    if (rc != JD_OK) return rc;
  }
  // write-after-read: nobody may still be reading the slot from an earlier step
  if (os >= 0 && slot_read_[os] == host_epoch_) {
    int rc = barrier(stream);
    if (rc != JD_OK) return rc;
  }
  return JD_OK;
}

void Runtime::fill_pointers(const PlanStep& st, PassDesc& d, const void* in, void* out) const {
  const int is = slot_of(st.in_kind), os = slot_of(st.out_kind);
  d.in = st.in_kind == BUF_USER_IN ? in : ((st.in_kind == BUF_USER_OUT || st.in_kind == BUF_PEER_OUT) ? out : slot_ptr(is, me_));
  for (int p = 0; p < d.npeers; ++p) {
    if (st.out_kind == BUF_USER_OUT)
      d.out[p] = out;
    else if (st.out_kind == BUF_PEER_OUT)
      d.out[p] = cur_peer_out_[st.group_ranks[p]];
    else
      d.out[p] = slot_ptr(os, st.group_ranks[p]);
  }
  d.abort_word = (arena_ && world_ > 1) ? flag_ptr(me_) + kFlagAbortWord : nullptr;
  d.status = status_device();
}

// Launch step `index` of the plan (or, when chunk_desc is given, that restricted copy of its descriptor,
// whose pointers are already set) on `stream`.
int Runtime::launch_step(const Plan& pl, int plan_id, size_t index, const PassDesc* chunk_desc, const void* in,
                         void* out, void* stream) {
  const PlanStep& st = pl.steps[index];
  const int is = slot_of(st.in_kind), os = slot_of(st.out_kind);
  if (st.copy_only) {
    const void* src = st.in_kind == BUF_USER_IN ? in : ((st.in_kind == BUF_USER_OUT || st.in_kind == BUF_PEER_OUT) ? out : slot_ptr(is, me_));
    void* dst = (st.out_kind == BUF_USER_OUT || st.out_kind == BUF_PEER_OUT) ? out : slot_ptr(os, me_);
    cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)st.copy_bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
    if (e != cudaSuccess) {
      set_last_error(cudaGetErrorString(e));
      return JD_ERR_CUDA;
    }
  } else if (chunk_desc != nullptr) {
    int rc = launch_pass(*chunk_desc, stream, status_device());
    if (rc != JD_OK) return rc;
  } else {
    PassDesc d = st.desc;
    fill_pointers(st, d, in, out);
    int rc = launch_pass(d, stream, status_device());
    if (rc != JD_OK) return rc;
  }
  ++launches_;
  (void)plan_id;
  return JD_OK;
}

int Runtime::ensure_pipe_resources(int chunks) {
  auto fail = [](cudaError_t e) {
    set_last_error(cudaGetErrorString(e));
    return (int)JD_ERR_CUDA;
  };
  if (!side_stream_) {
    int lo = 0, hi = 0;
    cudaError_t e = cudaDeviceGetStreamPriorityRange(&lo, &hi);
    if (e != cudaSuccess) return fail(e);
    cudaStream_t s;
    e = cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, hi);
    if (e != cudaSuccess) return fail(e);
    side_stream_ = s;
    cudaEvent_t ev;
    e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e != cudaSuccess) return fail(e);
    fork_event_ = ev;
  }
  while ((int)chunk_events_.size() < chunks) {
    cudaEvent_t ev;
    cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e != cudaSuccess) return fail(e);
    chunk_events_.push_back(ev);
  }
  return JD_OK;
}

void Runtime::release_pipe_resources() {
  for (void* ev : chunk_events_) cudaEventDestroy((cudaEvent_t)ev);
  chunk_events_.clear();
  if (fork_event_) cudaEventDestroy((cudaEvent_t)fork_event_);
  if (side_stream_) cudaStreamDestroy((cudaStream_t)side_stream_);
  fork_event_ = side_stream_ = nullptr;
  cudaGetLastError();
}

// Steps index (an exchange pass) and index + 1 (the local pass that consumes it), cut into chunks.
// The exchange chunks run back to back on a high-priority side stream, so the link never waits for
// the local pass; the caller's stream runs, per chunk: wait for this rank's chunk to be issued, a
// cross-rank barrier ("chunk k of every rank has landed"), the local pass on chunk k.  All barriers of
// the section are on the caller's stream, so the ranks keep counting the same barriers in the same
// order.  The side stream is joined again by the last event the caller's stream waits for, which also
// makes the section capturable in a CUDA graph.
int Runtime::run_pipelined(Plan& pl, int plan_id, size_t index, const void* in, void* out, void* stream) {
  PlanStep& prod = pl.steps[index];
  PlanStep& cons = pl.steps[index + 1];
  const int K = prod.pipe_chunks;
  int rc = ensure_pipe_resources(K);
  if (rc != JD_OK) return rc;
  // hazards of both steps are settled up front, on the caller's stream
  if ((rc = sync_before(prod, stream)) != JD_OK) return rc;
  const int cos = slot_of(cons.out_kind);
  if (cos >= 0 && slot_read_[cos] == host_epoch_ && (rc = barrier(stream)) != JD_OK) return rc;

  PassDesc pd = prod.desc, cd = cons.desc;
  fill_pointers(prod, pd, in, out);
  fill_pointers(cons, cd, in, out);
  pd.grid_limit = prod.pipe_grid_limit;
  const int pext = prod.pipe_role == 2 ? pd.Tn : pd.On;
  const int cext = cons.pipe_role == 2 ? cd.Tn : cd.On;
  if (pext != cext || K < 2 || pext % K) {
    set_last_error("runtime: inconsistent pipeline annotation in plan");
    return JD_ERR_INVALID_ARG;
  }
  const int len = pext / K;
  std::vector<PassDesc> pchunk(K, pd), cchunk(K, cd);
  for (int k = 0; k < K; ++k)
    if (!restrict_pass(pchunk[k], prod.pipe_role, k * len, len) || !restrict_pass(cchunk[k], cons.pipe_role, k * len, len)) {
      set_last_error("runtime: pass cannot be cut into the requested chunks");
      return JD_ERR_INVALID_ARG;
    }

  StepProfiler& prof = StepProfiler::instance();
  const bool profiling = prof.mode() != StepProfiler::OFF;
  if (profiling) {
    char name[96];
    std::snprintf(name, sizeof(name), "plan%d.step%d+%d pipelined x%d", plan_id, (int)index, (int)index + 1, K);
    prof.start(name, stream);
  }
  cudaStream_t main_s = (cudaStream_t)stream, side = (cudaStream_t)side_stream_;
  auto cuda_ok = [](cudaError_t e) {
    if (e == cudaSuccess) return true;
    set_last_error(cudaGetErrorString(e));
    return false;
  };
  if (!cuda_ok(cudaEventRecord((cudaEvent_t)fork_event_, main_s)) ||
      !cuda_ok(cudaStreamWaitEvent(side, (cudaEvent_t)fork_event_, 0)))
    return JD_ERR_CUDA;
  auto issue_exchange = [&](int k) -> int {
    int r = launch_step(pl, plan_id, index, &pchunk[k], in, out, side);
    if (r != JD_OK) return r;
    return cuda_ok(cudaEventRecord((cudaEvent_t)chunk_events_[k], side)) ? (int)JD_OK : (int)JD_ERR_CUDA;
  };
  // Whatever happens below, the caller's stream must join the side stream again (a captured graph
  // would otherwise be left with an unjoined branch), so errors are remembered, not returned at once.
  int first_err = issue_exchange(0);
  int issued = first_err == JD_OK ? 1 : 0;
  for (int k = 0; k < K && first_err == JD_OK; ++k) {
    if (k + 1 < K) {
      first_err = issue_exchange(k + 1);
      if (first_err != JD_OK) break;
      ++issued;
    }
    if (!cuda_ok(cudaStreamWaitEvent(main_s, (cudaEvent_t)chunk_events_[k], 0))) {
      first_err = JD_ERR_CUDA;
      break;
    }
    if ((first_err = barrier(stream)) != JD_OK) break;
    first_err = launch_step(pl, plan_id, index + 1, &cchunk[k], in, out, stream);
  }
  if (issued > 0) cudaStreamWaitEvent(main_s, (cudaEvent_t)chunk_events_[issued - 1], 0);
  if (profiling) prof.stop(stream);
  if (first_err != JD_OK) return first_err;
  ++pipelined_sections_;
  // the exchange slot was written before the section's last barrier and read after it
  const int pos = slot_of(prod.out_kind), pis = slot_of(prod.in_kind);
  if (pis >= 0) slot_read_[pis] = host_epoch_;
  if (pos >= 0) {
    slot_written_[pos] = host_epoch_ - 1;
    slot_read_[pos] = host_epoch_;
  }
  if (cos >= 0) slot_written_[cos] = host_epoch_;
  return JD_OK;
}

int Runtime::execute(int plan_id, const void* in, void* out, void* stream, void* const* peer_out) {
  Plan& pl = plans_.at(plan_id);
  if (world_ > 1 || pl.slot_bytes > 0) {
    if (!arena_ || (size_t)pl.slot_bytes > slot_bytes_) {
      set_last_error("runtime: arena missing or too small for this plan");
      return JD_ERR_INVALID_ARG;
    }
  }
  bool wants_peer_out = false;
  for (const PlanStep& st : pl.steps) wants_peer_out |= st.out_kind == BUF_PEER_OUT;
  if (wants_peer_out && (peer_out == nullptr || peer_out[me_] != out)) {
    set_last_error("runtime: plan stores into the peers' result blocks but their addresses were not given");
    return JD_ERR_INVALID_ARG;
  }
  // cleared on every way out, so that a later call can never see this call's addresses
  struct PeerOutScope {
    void* const*& slot;
    ~PeerOutScope() { slot = nullptr; }
  } peer_scope{cur_peer_out_};
  cur_peer_out_ = peer_out;
  bool peer_stores_pending = false;
  StepProfiler& prof = StepProfiler::instance();
  for (size_t i = 0; i < pl.steps.size(); ++i) {
    PlanStep& st = pl.steps[i];
    if (st.pipe_chunks > 1 && pipelining_ && world_ > 1 && i + 1 < pl.steps.size() && !st.copy_only) {
      int rc = run_pipelined(pl, plan_id, i, in, out, stream);
      if (rc != JD_OK) return rc;
      ++i;
      continue;
    }
    int rc = sync_before(st, stream);
    if (rc != JD_OK) return rc;
    if (st.out_kind == BUF_PEER_OUT && world_ > 1 && !st.copy_only && st.desc.npeers > 1) {
      // the other ranks may still be using their result blocks in work issued before this call
      if ((rc = barrier(stream)) != JD_OK) return rc;
      peer_stores_pending = true;
    }
    const bool profiling = prof.mode() != StepProfiler::OFF;
    if (profiling) {
      char name[96];
      if (st.copy_only)
        std::snprintf(name, sizeof(name), "plan%d.step%d copy", plan_id, (int)i);
      else
        std::snprintf(name, sizeof(name), "plan%d.step%d %s C=%d peers=%d", plan_id, (int)i,
                      st.desc.fft_mode == JD_COPY ? "copy-pass" : "fft-pass", st.desc.C, st.desc.npeers);
      prof.start(name, stream);
    }
    rc = launch_step(pl, plan_id, i, nullptr, in, out, stream);
    if (profiling) prof.stop(stream);
    if (rc != JD_OK) return rc;
    const int is = slot_of(st.in_kind), os = slot_of(st.out_kind);
    if (is >= 0) slot_read_[is] = host_epoch_;
    if (os >= 0) slot_written_[os] = host_epoch_;
  }
  // the result is complete once every rank's stores into it have landed
  if (peer_stores_pending) return barrier(stream);
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

int Runtime::poke_flag(int word, uint32_t value) {
  if (!arena_) return JD_ERR_INVALID_ARG;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(flag_ptr(me_) + word, &value, sizeof(value), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return JD_ERR_CUDA;
  }
  return JD_OK;
}

int Runtime::peek_flag(int word, uint32_t* value) const {
  if (!arena_) return JD_ERR_INVALID_ARG;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(value, flag_ptr(me_) + word, sizeof(*value), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return JD_ERR_CUDA;
  }
  return JD_OK;
}

int Runtime::halo_direct(HaloDesc push, const HaloDesc* zero, void* const* block, void* stream) {
  if (!arena_ && world_ > 1) {
    set_last_error("runtime: direct halo exchange without arena (flags)");
    return JD_ERR_INVALID_ARG;
  }
  int rc;
  if (world_ > 1 && (rc = barrier(stream)) != JD_OK) return rc;
  push.direct = 1;
  push.src = block[me_];
  push.dst = block[me_];
  for (int p = 0; p < JD_MAX_PEERS; ++p) push.stage[p] = p < world_ ? block[p] : nullptr;
  if ((rc = launch_halo_pack(push, stream)) != JD_OK) return rc;
  ++launches_;
  if (zero != nullptr) {
    HaloDesc z = *zero;
    z.src = block[me_];
    z.dst = block[me_];
    for (int p = 0; p < JD_MAX_PEERS; ++p) z.stage[p] = nullptr;
    if ((rc = launch_halo_unpack(z, stream)) != JD_OK) return rc;
    ++launches_;
  }
  if (world_ > 1 && (rc = barrier(stream)) != JD_OK) return rc;
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
