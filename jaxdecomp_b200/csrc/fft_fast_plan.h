// Stage plan of the specialised power-of-two kernel (fft_fast.cu) and the
// layout of its per-stage twiddle tables, shared with the host code that
// fills those tables (tables.cpp).
//
// For every stage s >= 1 the table holds one record per kk in [0, Ls(s)),
// Ls = product of the earlier radices: the four factors w, w^2, w^4, w^8 with
// w = exp(-2 pi i kk / (Ls * radix)).  Threads of a warp own consecutive kk, so
// the records they read are contiguous (32 bytes each for complex64): one
// coalesced request instead of four scattered reads of the table of M roots,
// which profiles showed to cost a third of the L1 data-pipe cycles.
#pragma once

#if defined(__CUDACC__)
#define JD_PLAN_HD __host__ __device__
#else
#define JD_PLAN_HD
#endif

namespace jdb {

// log2 of the radix of stage s for M = 2^logm (7 <= logm <= 12)
JD_PLAN_HD constexpr int plan_radix_log(int logm, int s) {
  switch (logm) {
    case 7: return s == 0 ? 4 : 3;
    case 8: return 4;
    case 9: return 3;
    case 10: return s == 0 ? 4 : 3;
    case 11: return s < 2 ? 4 : 3;
    default: return 4;  // 12
  }
}
JD_PLAN_HD constexpr int plan_num_stages(int logm) { return logm <= 8 ? 2 : 3; }
// log2 of Ls (length of the finished sub-transforms) before stage s
JD_PLAN_HD constexpr int plan_log_ls(int logm, int s) {
  int l = 0;
  for (int i = 0; i < s; ++i) l += plan_radix_log(logm, i);
  return l;
}
// index of the first record of stage s (s >= 1) in the packed table, and the total number of records
JD_PLAN_HD constexpr int plan_stage_record0(int logm, int s) {
  int off = 0;
  for (int i = 1; i < s; ++i) off += 1 << plan_log_ls(logm, i);
  return off;
}
JD_PLAN_HD constexpr int plan_stage_records(int logm) { return plan_stage_record0(logm, plan_num_stages(logm)); }
constexpr int kFastMinLog = 7, kFastMaxLog = 12;

// Thread layout of the last stage of a rotating pass over tiles of T rows (a power of two): sixteen
// consecutive threads cover RH = min(T, 8) rows x 16/RH butterfly indices, consecutive threads consecutive rows.
JD_PLAN_HD constexpr int fast_last_stage_row(int T, int tid) {
  const int rh = T < 8 ? T : 8;
  return tid % rh + rh * ((tid / 16) % (T / rh));
}
JD_PLAN_HD constexpr int fast_last_stage_j(int T, int tid) {
  const int rh = T < 8 ? T : 8;
  const int cb = 16 / rh;
  return cb * ((tid / 16) / (T / rh)) + (tid / rh) % cb;
}

}  // namespace jdb
