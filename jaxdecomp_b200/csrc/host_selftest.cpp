// Sanitizer self-test of the host side of the native core.
//
// Built by native.build_host_selftest() with g++ -fsanitize=address,undefined from the same sources the
// library uses for its CPU emulation (cpu_ref.cpp: the tile pass with the index arithmetic of
// tile_map.h / tile_ops.h and the butterflies of fft_core.h / fft_mixed.h; tables.cpp: the twiddle,
// chirp and per-stage tables).  It replays pass descriptors that the Python planner wrote to a file:
// every operand and every destination is a heap block of exactly the size the planner claims, so an
// index that leaves its buffer is an AddressSanitizer report, and signed overflow, misaligned access or
// a bad shift in the index arithmetic is an UndefinedBehaviorSanitizer report (both abort the program).
// The results go to a second file, where the test compares them bit for bit with the regular build.
//
// Case file: u64 magic, u64 sizeof(PassDesc), u64 number of cases; per case the raw PassDesc, u64 mode
// (0: the general tile pass, 1: the host restatement of the rotating copy kernels), u64 operand bytes,
// the operand, u64 number of destinations, u64 bytes of each destination.
// Result file: per case, per destination, the destination's bytes.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "launch.h"
#include "runtime.h"

namespace jdb {
// the library keeps its last error message next to the CUDA launchers, which are not part of this program
static std::string g_selftest_error;
void set_last_error(const char* msg) { g_selftest_error = msg ? msg : ""; }
const char* last_error_message() { return g_selftest_error.c_str(); }
}  // namespace jdb

namespace {

constexpr uint64_t kMagic = 0x32464C455342444AULL;  // "JDBSELF2"

bool read_exact(std::FILE* f, void* dst, size_t n) { return n == 0 || std::fread(dst, 1, n, f) == n; }

int fail(const char* what) {
  std::fprintf(stderr, "host_selftest: %s\n", what);
  return 2;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc != 3) return fail("usage: host_selftest <cases> <results>");
  std::FILE* in = std::fopen(argv[1], "rb");
  if (!in) return fail("cannot open the case file");
  std::FILE* out = std::fopen(argv[2], "wb");
  if (!out) return fail("cannot open the result file");
  uint64_t head[3];
  if (!read_exact(in, head, sizeof(head)) || head[0] != kMagic) return fail("bad header");
  if (head[1] != sizeof(jdb::PassDesc)) return fail("descriptor size differs from the library's");
  for (uint64_t c = 0; c < head[2]; ++c) {
    jdb::PassDesc d;
    uint64_t mode = 0, in_bytes = 0, nout = 0;
    if (!read_exact(in, &d, sizeof(d)) || !read_exact(in, &mode, 8) || !read_exact(in, &in_bytes, 8))
      return fail("truncated case");
    if (mode > 1) return fail("unknown mode");
    // exact-size heap blocks: the red zones around them are what catches a stray index
    unsigned char* operand = static_cast<unsigned char*>(std::malloc(in_bytes ? in_bytes : 1));
    if (!operand || !read_exact(in, operand, in_bytes)) return fail("truncated operand");
    if (!read_exact(in, &nout, 8) || nout == 0 || nout > JD_MAX_PEERS || (int)nout != d.npeers)
      return fail("bad destination count");
    std::vector<uint64_t> out_bytes(nout);
    std::vector<unsigned char*> dests(nout);
    for (uint64_t p = 0; p < nout; ++p) {
      if (!read_exact(in, &out_bytes[p], 8)) return fail("truncated case");
      dests[p] = static_cast<unsigned char*>(std::calloc(out_bytes[p] ? out_bytes[p] : 1, 1));
      if (!dests[p]) return fail("out of memory");
    }
    const bool wants_tables = d.twiddle != nullptr;  // addresses of the writing process: only "set or not" survives
    d.twiddle = d.chirp = d.bhat = d.tw_stage = nullptr;
    if (wants_tables) {
      const jdb::FftTables t = jdb::get_fft_tables(d.C, d.M, d.elem_bytes, /*device=*/false);
      d.twiddle = t.twiddle;
      d.chirp = t.chirp;
      d.bhat = t.bhat;
      d.tw_stage = t.tw_stage;
    }
    d.in = operand;
    for (int p = 0; p < JD_MAX_PEERS; ++p) d.out[p] = p < (int)nout ? dests[p] : nullptr;
    d.abort_word = nullptr;
    d.status = nullptr;
    const int rc = mode == 1 ? jdb::run_copy_fast_host(d) : jdb::run_pass_host(d);
    if (rc != 0) {
      std::fprintf(stderr, "host_selftest: case %llu returned %d (%s)\n", (unsigned long long)c, rc,
                   jdb::last_error_message());
      return 3;
    }
    for (uint64_t p = 0; p < nout; ++p) {
      if (out_bytes[p] && std::fwrite(dests[p], 1, out_bytes[p], out) != out_bytes[p]) return fail("write failed");
      std::free(dests[p]);
    }
    std::free(operand);
  }
  jdb::clear_fft_tables();
  std::fclose(in);
  if (std::fclose(out) != 0) return fail("write failed");
  std::printf("host_selftest: %llu cases ok\n", (unsigned long long)head[2]);
  return 0;
}
