// Environment-gated, buffered, per-rank trace log and a step profiler.
//
// Trace log: counterpart of the reference's AsyncLogger
// (src/csrc/include/logger.hpp:53-260).  Environment variables:
//   JD_TRACE=1                 enable [INFO] records
//   JD_TRACE_VERBOSE=<names>   also enable [VERB] records for loggers whose name
//                              contains one of the comma-separated substrings ("1" or "*" = all)
//   JD_TRACE_OUTPUT_DIR=<dir>  write <dir>/jd_trace_<name>[_rank<r>].log instead of stderr
//   JD_TRACE_CONSOLE=1         also echo to stderr when writing to files
//   JD_TRACE_NOBUFFER=1        flush after every record
//   JD_TRACE_MAX_BUFFER=<n>    buffer size in bytes before a flush (default 1 MiB)
//
// Step profiler: counterpart of Perfostep (src/csrc/include/perfostep.hpp:302-352).
//   JD_PERFO_STEP=TIMER | CUDA | NVTX selects host chrono timing, CUDA-event
//   timing (synchronising) or NVTX ranges; unset = disabled.  Reports can be
//   dumped as CSV or markdown.
#pragma once
#include <cstdarg>
#include <string>
#include <vector>

namespace jdb {

enum TraceLevel { TRACE_INFO = 0, TRACE_VERBOSE = 1 };

bool trace_enabled(const char* logger, TraceLevel level);
void trace_write(const char* logger, TraceLevel level, const char* fmt, ...) __attribute__((format(printf, 3, 4)));
void trace_flush();
void trace_set_rank(int rank);
void trace_reconfigure();  // re-read the environment (used by tests)
std::string trace_stack();  // demangled backtrace of the caller

#define JD_TRACE_INFO(logger, ...)                                                      \
  do {                                                                                  \
    if (::jdb::trace_enabled(logger, ::jdb::TRACE_INFO)) ::jdb::trace_write(logger, ::jdb::TRACE_INFO, __VA_ARGS__); \
  } while (0)
#define JD_TRACE_VERBOSE(logger, ...)                                                      \
  do {                                                                                     \
    if (::jdb::trace_enabled(logger, ::jdb::TRACE_VERBOSE))                                \
      ::jdb::trace_write(logger, ::jdb::TRACE_VERBOSE, __VA_ARGS__);                       \
  } while (0)

struct StepRecord {
  std::string name;
  double ms;
  long long count;
};

class StepProfiler {
 public:
  enum Mode { OFF = 0, TIMER = 1, CUDA = 2, NVTX = 3 };
  static StepProfiler& instance();
  Mode mode() const { return mode_; }
  void set_mode(Mode m) { mode_ = m; }
  void start(const std::string& name, void* stream);
  void stop(void* stream);
  void switch_to(const std::string& name, void* stream) {
    stop(stream);
    start(name, stream);
  }
  std::vector<StepRecord> report() const;
  std::string to_csv() const;
  std::string to_markdown() const;
  void reset();

 private:
  StepProfiler();
  struct Open {
    std::string name;
    double t0;
    void* ev0;
  };
  Mode mode_ = OFF;
  std::vector<Open> stack_;
  std::vector<StepRecord> records_;
  void add(const std::string& name, double ms);
};

}  // namespace jdb
