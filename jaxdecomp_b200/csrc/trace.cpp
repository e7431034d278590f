// Trace log and step profiler (see trace.h).
#include "trace.h"

#include <cuda_runtime.h>
#include <cxxabi.h>
#include <execinfo.h>
#include <nvtx3/nvToolsExt.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>

namespace jdb {

namespace {

struct TraceState {
  std::mutex mu;
  bool configured = false;
  bool info = false;
  bool verbose_all = false;
  std::vector<std::string> verbose_names;
  std::string out_dir;
  bool console = false;
  bool nobuffer = false;
  size_t max_buffer = 1 << 20;
  int rank = -1;
  std::map<std::string, std::string> buffers;  // logger -> pending text
  std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
};

TraceState& state() {
  static TraceState s;
  return s;
}

bool env_flag(const char* name) {
  const char* v = std::getenv(name);
  return v && *v && std::strcmp(v, "0") != 0;
}

void configure_locked(TraceState& s) {
  s.configured = true;
  s.info = env_flag("JD_TRACE");
  s.verbose_all = false;
  s.verbose_names.clear();
  if (const char* v = std::getenv("JD_TRACE_VERBOSE")) {
    std::string all(v);
    if (all == "1" || all == "*") {
      s.verbose_all = true;
    } else {
      std::stringstream ss(all);
      std::string item;
      while (std::getline(ss, item, ','))
        if (!item.empty()) s.verbose_names.push_back(item);
    }
    if (s.verbose_all || !s.verbose_names.empty()) s.info = true;
  }
  s.out_dir = std::getenv("JD_TRACE_OUTPUT_DIR") ? std::getenv("JD_TRACE_OUTPUT_DIR") : "";
  s.console = env_flag("JD_TRACE_CONSOLE");
  s.nobuffer = env_flag("JD_TRACE_NOBUFFER");
  if (const char* v = std::getenv("JD_TRACE_MAX_BUFFER")) {
    long n = std::atol(v);
    if (n > 0) s.max_buffer = (size_t)n;
  }
  if (s.rank < 0) {
    if (const char* r = std::getenv("RANK")) s.rank = std::atoi(r);
  }
}

void flush_one_locked(TraceState& s, const std::string& logger, std::string& text) {
  if (text.empty()) return;
  if (!s.out_dir.empty()) {
    std::string path = s.out_dir + "/jd_trace_" + logger;
    if (s.rank >= 0) path += "_rank" + std::to_string(s.rank);
    path += ".log";
    if (FILE* f = std::fopen(path.c_str(), "a")) {
      std::fwrite(text.data(), 1, text.size(), f);
      std::fclose(f);
    }
    if (s.console) std::fwrite(text.data(), 1, text.size(), stderr);
  } else {
    std::fwrite(text.data(), 1, text.size(), stderr);
  }
  text.clear();
}

struct FlushAtExit {
  ~FlushAtExit() { trace_flush(); }
} g_flush_at_exit;

}  // namespace

bool trace_enabled(const char* logger, TraceLevel level) {
  TraceState& s = state();
  std::lock_guard<std::mutex> lk(s.mu);
  if (!s.configured) configure_locked(s);
  if (!s.info) return false;
  if (level == TRACE_INFO) return true;
  if (s.verbose_all) return true;
  for (const auto& n : s.verbose_names)
    if (std::strstr(logger, n.c_str())) return true;
  return false;
}

void trace_write(const char* logger, TraceLevel level, const char* fmt, ...) {
  char msg[1024];
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  TraceState& s = state();
  std::lock_guard<std::mutex> lk(s.mu);
  const double t = std::chrono::duration<double>(std::chrono::steady_clock::now() - s.t0).count();
  char head[160];
  if (s.rank >= 0)
    std::snprintf(head, sizeof(head), "[%12.6f][rank %d][%s][%s] ", t, s.rank, logger, level == TRACE_INFO ? "INFO" : "VERB");
  else
    std::snprintf(head, sizeof(head), "[%12.6f][%s][%s] ", t, logger, level == TRACE_INFO ? "INFO" : "VERB");
  std::string& buf = s.buffers[logger];
  buf += head;
  buf += msg;
  buf += '\n';
  if (s.nobuffer || buf.size() >= s.max_buffer) flush_one_locked(s, logger, buf);
}

void trace_flush() {
  TraceState& s = state();
  std::lock_guard<std::mutex> lk(s.mu);
  for (auto& kv : s.buffers) flush_one_locked(s, kv.first, kv.second);
}

void trace_set_rank(int rank) {
  TraceState& s = state();
  std::lock_guard<std::mutex> lk(s.mu);
  s.rank = rank;
}

void trace_reconfigure() {
  TraceState& s = state();
  std::lock_guard<std::mutex> lk(s.mu);
  for (auto& kv : s.buffers) flush_one_locked(s, kv.first, kv.second);
  configure_locked(s);
}

std::string trace_stack() {
  void* frames[64];
  const int n = backtrace(frames, 64);
  char** syms = backtrace_symbols(frames, n);
  std::string out;
  for (int i = 1; i < n && syms; ++i) {
    std::string line(syms[i]);
    // mangled name sits between '(' and '+'
    const size_t l = line.find('('), p = line.find('+', l == std::string::npos ? 0 : l);
    if (l != std::string::npos && p != std::string::npos && p > l + 1) {
      std::string mangled = line.substr(l + 1, p - l - 1);
      int status = 0;
      char* dem = abi::__cxa_demangle(mangled.c_str(), nullptr, nullptr, &status);
      if (status == 0 && dem) {
        line = line.substr(0, l + 1) + dem + line.substr(p);
      }
      std::free(dem);
    }
    out += "  #" + std::to_string(i - 1) + " " + line + "\n";
  }
  std::free(syms);
  return out;
}

// ---- step profiler -------------------------------------------------------------------------------------------
StepProfiler::StepProfiler() {
  const char* v = std::getenv("JD_PERFO_STEP");
  if (!v) return;
  std::string m(v);
  if (m == "TIMER") mode_ = TIMER;
  else if (m == "CUDA") mode_ = CUDA;
  else if (m == "NVTX") mode_ = NVTX;
}

StepProfiler& StepProfiler::instance() {
  static StepProfiler p;
  return p;
}

static double now_ms() {
  return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

void StepProfiler::start(const std::string& name, void* stream) {
  if (mode_ == OFF) return;
  Open o{name, 0.0, nullptr};
  if (mode_ == TIMER) {
    o.t0 = now_ms();
  } else if (mode_ == CUDA) {
    cudaEvent_t ev;
    if (cudaEventCreate(&ev) == cudaSuccess) {
      cudaEventRecord(ev, (cudaStream_t)stream);
      o.ev0 = ev;
    }
  } else if (mode_ == NVTX) {
    static const uint32_t colours[] = {0xff1f77b4, 0xffff7f0e, 0xff2ca02c, 0xffd62728, 0xff9467bd, 0xff8c564b};
    nvtxEventAttributes_t attr = {};
    attr.version = NVTX_VERSION;
    attr.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
    attr.colorType = NVTX_COLOR_ARGB;
    attr.color = colours[stack_.size() % 6];
    attr.messageType = NVTX_MESSAGE_TYPE_ASCII;
    attr.message.ascii = name.c_str();
    nvtxRangePushEx(&attr);
  }
  stack_.push_back(o);
}

void StepProfiler::stop(void* stream) {
  if (mode_ == OFF || stack_.empty()) return;
  Open o = stack_.back();
  stack_.pop_back();
  if (mode_ == TIMER) {
    add(o.name, now_ms() - o.t0);
  } else if (mode_ == CUDA) {
    if (o.ev0) {
      cudaEvent_t ev1;
      float ms = 0.f;
      if (cudaEventCreate(&ev1) == cudaSuccess) {
        cudaEventRecord(ev1, (cudaStream_t)stream);
        cudaEventSynchronize(ev1);
        cudaEventElapsedTime(&ms, (cudaEvent_t)o.ev0, ev1);
        cudaEventDestroy(ev1);
      }
      cudaEventDestroy((cudaEvent_t)o.ev0);
      add(o.name, ms);
    }
  } else if (mode_ == NVTX) {
    nvtxRangePop();
  }
}

void StepProfiler::add(const std::string& name, double ms) {
  for (auto& r : records_)
    if (r.name == name) {
      r.ms += ms;
      ++r.count;
      return;
    }
  records_.push_back(StepRecord{name, ms, 1});
}

std::vector<StepRecord> StepProfiler::report() const { return records_; }

std::string StepProfiler::to_csv() const {
  std::ostringstream os;
  os << "step,count,total_ms,mean_ms\n";
  for (const auto& r : records_) os << r.name << "," << r.count << "," << r.ms << "," << (r.ms / (double)r.count) << "\n";
  return os.str();
}

std::string StepProfiler::to_markdown() const {
  std::ostringstream os;
  os << "| step | count | total ms | mean ms |\n|---|---|---|---|\n";
  for (const auto& r : records_)
    os << "| " << r.name << " | " << r.count << " | " << r.ms << " | " << (r.ms / (double)r.count) << " |\n";
  return os.str();
}

void StepProfiler::reset() {
  records_.clear();
  stack_.clear();
}

}  // namespace jdb
