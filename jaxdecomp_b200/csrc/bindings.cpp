// pybind11 module `_jdb200`: Python-facing entry points of the native core.
//
// Counterpart of the reference's nanobind module (src/csrc/jaxdecomp.cc:550-623),
// which exposes init/finalize, pencil geometry, workspace queries and the XLA
// FFI targets.  Here the entry points take raw device addresses and a CUDA
// stream handle (both as integers), so the module has no dependency on
// PyTorch's C++ API.  Failures are raised as Python exceptions; nothing exits
// the process.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <stdexcept>
#include <tuple>
#include <vector>

#include "fft_fast_plan.h"
#include "fft_mixed.h"
#include "launch.h"
#include "runtime.h"
#include "trace.h"

#ifdef JD_BOUNDS_CHECK
#define JD_BOUNDS_CHECK_BUILD JD_BOUNDS_CHECK
#else
#define JD_BOUNDS_CHECK_BUILD 0
#endif

namespace py = pybind11;
using namespace jdb;

static void* P(uintptr_t v) { return reinterpret_cast<void*>(v); }

static void raise_on(int rc, const char* what) {
  if (rc == JD_OK) return;
  std::string msg = std::string(what) + ": " + status_name(rc);
  const char* detail = last_error_message();
  if (detail && *detail) msg += std::string(" (") + detail + ")";
  if (rc == JD_ERR_INVALID_ARG) throw py::value_error(msg);
  throw std::runtime_error(msg);
}

// regions: list of (lo0, hi0, lo1, hi1, peer, stage_off)
using Region6 = std::tuple<int, int, int, int, int, long long>;
// direct pushes: (lo0, hi0, lo1, hi1, peer, dlo0, dlo1)
using Region7 = std::tuple<int, int, int, int, int, int, int>;

static HaloDesc make_halo_desc(const std::vector<Region6>& regions, int S0, int S1,
                               int S2, int B, int elem_bytes, int is_f64, int accumulate) {
  HaloDesc d;
  std::memset(&d, 0, sizeof(d));
  if (regions.size() > 8) throw py::value_error("at most eight halo regions");
  d.S0 = S0; d.S1 = S1; d.S2 = S2; d.B = B;
  d.elem_bytes = elem_bytes;
  d.is_f64 = is_f64;
  d.accumulate = accumulate;
  d.nregions = (int)regions.size();
  for (size_t i = 0; i < regions.size(); ++i) {
    HaloRegion& g = d.reg[i];
    g.lo0 = std::get<0>(regions[i]); g.hi0 = std::get<1>(regions[i]);
    g.lo1 = std::get<2>(regions[i]); g.hi1 = std::get<3>(regions[i]);
    g.peer = std::get<4>(regions[i]);
    g.stage_off = std::get<5>(regions[i]);
  }
  return d;
}

PYBIND11_MODULE(_jdb200, m) {
  m.doc() = "native core of jaxdecomp_b200 (sm_100a)";
  m.attr("MAX_PEERS") = JD_MAX_PEERS;
  m.attr("COPY") = (int)JD_COPY;
  m.attr("FFT_POW2") = (int)JD_FFT_POW2;
  m.attr("FFT_BLUESTEIN") = (int)JD_FFT_BLUESTEIN;
  m.attr("FFT_MIXED") = (int)JD_FFT_MIXED;
  m.attr("BUF_USER_IN") = (int)BUF_USER_IN;
  m.attr("BUF_USER_OUT") = (int)BUF_USER_OUT;
  m.attr("BUF_SLOT_A") = (int)BUF_SLOT_A;
  m.attr("BUF_SLOT_B") = (int)BUF_SLOT_B;
  m.attr("BUF_PEER_OUT") = (int)BUF_PEER_OUT;
  m.attr("FLAG_EPOCH_COUNTER_WORD") = kFlagEpochCounterWord;
  m.attr("FLAG_ABORT_WORD") = kFlagAbortWord;
  m.attr("BOUNDS_CHECK_BUILD") = (bool)JD_BOUNDS_CHECK_BUILD;
  m.def("status_name", [](int s) { return std::string(status_name(s)); });

  py::class_<PassDesc>(m, "PassDesc")
      .def(py::init([]() {
        PassDesc d;
        std::memset(&d, 0, sizeof(d));
        d.scale = 1.0;
        d.B = 1;
        return d;
      }))
#define RW(f) .def_readwrite(#f, &PassDesc::f)
      RW(is_c) RW(is_t) RW(is_o) RW(is_b) RW(os_c) RW(os_t) RW(os_o) RW(os_b) RW(out_base) RW(C) RW(Tn) RW(On) RW(B)
      RW(Cl) RW(Tl) RW(Ol) RW(npeers) RW(fft_mode) RW(M) RW(inverse) RW(T) RW(Cc) RW(pitch) RW(elem_bytes)
      RW(load_t_contig) RW(store_t_contig) RW(use_bulk) RW(mul_mode) RW(vec_in) RW(vec_out) RW(intra_pad) RW(logT) RW(logW) RW(split_axis) RW(scale) RW(grid_limit) RW(out_limit)
#undef RW
      // the descriptor as the kernels see it (a plain struct); read by the sanitizer self-test program
      .def("raw_bytes", [](const PassDesc& d) { return py::bytes(reinterpret_cast<const char*>(&d), sizeof(PassDesc)); })
      .def_property("in_ptr", [](const PassDesc& d) { return (uintptr_t)d.in; },
                    [](PassDesc& d, uintptr_t v) { d.in = P(v); })
      .def_property("twiddle", [](const PassDesc& d) { return (uintptr_t)d.twiddle; },
                    [](PassDesc& d, uintptr_t v) { d.twiddle = P(v); })
      .def_property("tw_stage", [](const PassDesc& d) { return (uintptr_t)d.tw_stage; },
                    [](PassDesc& d, uintptr_t v) { d.tw_stage = P(v); })
      .def_property("chirp", [](const PassDesc& d) { return (uintptr_t)d.chirp; },
                    [](PassDesc& d, uintptr_t v) { d.chirp = P(v); })
      .def_property("bhat", [](const PassDesc& d) { return (uintptr_t)d.bhat; },
                    [](PassDesc& d, uintptr_t v) { d.bhat = P(v); })
      .def("set_out", [](PassDesc& d, int p, uintptr_t v) {
        if (p < 0 || p >= JD_MAX_PEERS) throw py::index_error("peer index");
        d.out[p] = P(v);
      })
      .def("get_out", [](const PassDesc& d, int p) { return (uintptr_t)d.out[p]; })
      // fused input multiplier: n = global extents of the original axes, off / axis = global offset and original
      // axis of the role axes (c, t, o), kfac = 2*pi / box length per original axis
      .def("set_mul", [](PassDesc& d, int mode, const std::vector<int>& n, const std::vector<int>& off,
                         const std::vector<int>& axis, const std::vector<double>& kfac) {
        if (n.size() != 3 || off.size() != 3 || axis.size() != 3 || kfac.size() != 3) throw py::value_error("set_mul: 3-vectors");
        d.mul_mode = mode;
        for (int i = 0; i < 3; ++i) {
          d.mul.n[i] = n[i];
          d.mul.off[i] = off[i];
          d.mul.axis[i] = axis[i];
          d.mul.kfac[i] = kfac[i];
        }
      })
      .def("copy", [](const PassDesc& d) { return d; })
      // the pass restricted to [lo, lo + len) of its t (role 2) or o (role 3) axis; in_ptr must be set
      .def("restricted", [](const PassDesc& d, int role, int lo, int len) {
        PassDesc r = d;
        if (!restrict_pass(r, role, lo, len)) throw py::value_error("pass cannot be restricted to this range");
        return r;
      });

  m.def("validate_pass", [](const PassDesc& d) { return validate_pass(d); });
  m.def("run_pass_host", [](const PassDesc& d) { raise_on(run_pass_host(d), "run_pass_host"); });
  m.def("launch_pass", [](const PassDesc& d, uintptr_t stream, uintptr_t status) {
    raise_on(launch_pass(d, P(stream), (StatusBlock*)P(status)), "launch_pass");
  });
  // like launch_pass, with the status block also used by the per-store range check of checked builds
  m.def("launch_pass_checked", [](const PassDesc& d0, uintptr_t stream, uintptr_t status) {
    PassDesc d = d0;
    d.status = P(status);
    raise_on(launch_pass(d, P(stream), (StatusBlock*)P(status)), "launch_pass");
  });
  m.def("fast_pass_eligible", [](const PassDesc& d) { return fast_pass_eligible(d); });
  m.def("pass_threads", &pass_threads);
  m.def("pass_smem_bytes", &pass_smem_bytes);
  m.def("copy_fast_eligible", [](const PassDesc& d) { return copy_fast_eligible(d); },
        "True when launch_pass would run the rotating copy kernels of copy_fast.cu on this (filled) descriptor");
  m.def("run_copy_fast_host", [](const PassDesc& d) { raise_on(run_copy_fast_host(d), "run_copy_fast_host"); },
        "Host restatement of the rotating copy kernels (same thread mapping and addressing), for CPU tests");
  m.def("get_fft_tables", [](int C, int M, int elem_bytes, bool device) {
    FftTables t = get_fft_tables(C, M, elem_bytes, device);
    return py::make_tuple((uintptr_t)t.twiddle, (uintptr_t)t.chirp, (uintptr_t)t.bhat, (uintptr_t)t.tw_stage);
  });
  m.def("clear_fft_tables", &clear_fft_tables);
  // geometry of the specialised kernels, for consistency tests against the Python tiling rules
  m.def("mixed_static_geometry", [](int n, int elem_bytes, bool store_t) {
    py::dict out;
    const MixedPlan pl = mixed_plan_of(n);
    const int T = mixed_static_T(n, elem_bytes, store_t);
    out["T"] = T;
    out["pitch"] = mixed_static_pitch(n, elem_bytes, T);
    out["tpr"] = mixed_threads_per_row(pl, T, elem_bytes);
    py::list rad;
    for (int s = 0; s < pl.ns; ++s) rad.append(pl.st[s].radix);
    out["radices"] = rad;
    return out;
  });
  m.def("mixed_last_stage_map", [](int T, int elem_bytes, int tid) {
    return py::make_tuple(mixed_last_stage_row(T, elem_bytes, tid), mixed_last_stage_j(T, elem_bytes, tid));
  });
  m.def("fast_last_stage_map", [](int T, int tid) {
    return py::make_tuple(fast_last_stage_row(T, tid), fast_last_stage_j(T, tid));
  });

  py::class_<PlanStep>(m, "PlanStep")
      .def(py::init<>())
      .def_readwrite("desc", &PlanStep::desc)
      .def_readwrite("in_kind", &PlanStep::in_kind)
      .def_readwrite("out_kind", &PlanStep::out_kind)
      .def_readwrite("copy_only", &PlanStep::copy_only)
      .def_readwrite("copy_bytes", &PlanStep::copy_bytes)
      .def_readwrite("pipe_chunks", &PlanStep::pipe_chunks)
      .def_readwrite("pipe_role", &PlanStep::pipe_role)
      .def_readwrite("pipe_grid_limit", &PlanStep::pipe_grid_limit)
      .def("set_group_ranks", [](PlanStep& s, const std::vector<int>& r) {
        if (r.size() > JD_MAX_PEERS) throw py::value_error("too many peers");
        for (size_t i = 0; i < r.size(); ++i) s.group_ranks[i] = r[i];
      });

  // A block of device memory that every rank of a group can address: the storage behind peer-visible
  // tensors (ops/peer.py).  Creation, export/open and close are collective like the arena's.
  py::class_<SymmetricArena>(m, "PeerBlock")
      .def(py::init<size_t, int, int>(), py::arg("bytes"), py::arg("world"), py::arg("me"))
      .def("export_handles", [](const SymmetricArena& a) { return py::bytes(a.export_handles()); })
      .def("open_peers", [](SymmetricArena& a, const std::vector<py::bytes>& hs) {
        std::vector<std::string> v;
        for (const auto& h : hs) v.push_back((std::string)h);
        a.open_peers(v);
      })
      .def("close_peers", &SymmetricArena::close_peers)
      .def("close", &SymmetricArena::close, py::arg("free_own") = true)
      .def("ptr", [](const SymmetricArena& a, int peer) { return (uintptr_t)a.data(peer); })
      .def_property_readonly("bytes", &SymmetricArena::bytes);

  py::class_<Runtime>(m, "Runtime")
      .def(py::init<int, int>(), py::arg("world"), py::arg("me"))
      .def("create_arena", &Runtime::create_arena)
      .def("export_handles", [](const Runtime& r) { return py::bytes(r.export_handles()); })
      .def("open_peers", [](Runtime& r, const std::vector<py::bytes>& hs) {
        std::vector<std::string> v;
        for (const auto& h : hs) v.push_back((std::string)h);
        r.open_peers(v);
      })
      .def("close_peers", &Runtime::close_peers)
      .def("destroy_arena", &Runtime::destroy_arena, py::arg("collective") = true)
      .def("has_arena", &Runtime::has_arena)
      .def("slot_bytes", &Runtime::slot_bytes)
      .def("slot_ptr", [](const Runtime& r, int slot, int peer) { return (uintptr_t)r.slot_ptr(slot, peer); })
      .def("flag_ptr", [](const Runtime& r, int peer) { return (uintptr_t)r.flag_ptr(peer); })
      .def("find_plan", &Runtime::find_plan)
      .def("add_plan", [](Runtime& r, const std::string& key, const std::vector<PlanStep>& steps, long long slot_bytes) {
        Plan p;
        p.steps = steps;
        p.slot_bytes = slot_bytes;
        return r.add_plan(key, std::move(p));
      })
      .def("plan_slot_bytes", [](const Runtime& r, int id) { return r.plan(id).slot_bytes; })
      .def("plan_num_steps", [](const Runtime& r, int id) { return r.plan(id).steps.size(); })
      .def("num_plans", &Runtime::num_plans)
      .def("cache_hits", &Runtime::cache_hits)
      .def("cache_misses", &Runtime::cache_misses)
      .def("clear_plans", &Runtime::clear_plans)
      .def("execute", [](Runtime& r, int id, uintptr_t in, uintptr_t out, uintptr_t stream) {
        raise_on(r.execute(id, P(in), P(out), P(stream)), "execute");
      })
      .def("execute_peer_out", [](Runtime& r, int id, uintptr_t in, const std::vector<uintptr_t>& outs, uintptr_t stream) {
        // outs: the result block's address on every arena rank (the plan's exchange stores into them)
        if ((int)outs.size() != r.world() || r.world() > JD_MAX_PEERS)
          throw std::invalid_argument("execute_peer_out: one result address per rank expected");
        void* blocks[JD_MAX_PEERS] = {nullptr};
        for (size_t p = 0; p < outs.size(); ++p) blocks[p] = P(outs[p]);
        raise_on(r.execute(id, P(in), blocks[r.me()], P(stream), blocks), "execute_peer_out");
      })
      .def("halo", [](Runtime& r, const std::vector<std::tuple<int, int, int, int, int, long long>>& pack,
                      const std::vector<std::tuple<int, int, int, int, int, long long>>& unpack,
                      const std::vector<std::tuple<int, int, int, int, int, long long>>& zero, int S0, int S1, int S2, int B,
                      int elem_bytes, int is_f64, int accumulate, uintptr_t src, uintptr_t dst, uintptr_t stream) {
        HaloDesc dp = make_halo_desc(pack, S0, S1, S2, B, elem_bytes, is_f64, 0);
        HaloDesc du = make_halo_desc(unpack, S0, S1, S2, B, elem_bytes, is_f64, accumulate);
        HaloDesc dz = make_halo_desc(zero, S0, S1, S2, B, elem_bytes, is_f64, 0);
        const long long bytes = (long long)B * S0 * S1 * S2 * elem_bytes;
        raise_on(r.halo(dp, du, zero.empty() ? nullptr : &dz, P(src), P(dst), bytes, P(stream)), "halo");
      })
      .def("set_pipelining", &Runtime::set_pipelining)
      .def("pipelining", &Runtime::pipelining)
      .def("pipelined_sections", &Runtime::pipelined_sections)
      .def("halo_direct", [](Runtime& r, const std::vector<Region7>& push, const std::vector<Region6>& zero, int S0, int S1,
                             int S2, int B, int elem_bytes, const std::vector<uintptr_t>& blocks, uintptr_t stream) {
        if ((int)blocks.size() != r.world()) throw py::value_error("halo_direct: one block pointer per rank");
        std::vector<Region6> plain;
        for (const auto& g : push)
          plain.emplace_back(std::get<0>(g), std::get<1>(g), std::get<2>(g), std::get<3>(g), std::get<4>(g), 0LL);
        HaloDesc dp = make_halo_desc(plain, S0, S1, S2, B, elem_bytes, 0, 0);
        for (size_t i = 0; i < push.size(); ++i) {
          dp.reg[i].dlo0 = std::get<5>(push[i]);
          dp.reg[i].dlo1 = std::get<6>(push[i]);
        }
        HaloDesc dz = make_halo_desc(zero, S0, S1, S2, B, elem_bytes, 0, 0);
        std::vector<void*> ptrs;
        for (uintptr_t b : blocks) ptrs.push_back(P(b));
        raise_on(r.halo_direct(dp, zero.empty() ? nullptr : &dz, ptrs.data(), P(stream)), "halo_direct");
      })
      .def("barrier", [](Runtime& r, uintptr_t stream) { raise_on(r.barrier(P(stream)), "barrier"); })
      .def("barriers_issued", &Runtime::barriers_issued)
      .def("launches", &Runtime::launches)
      .def("read_status", [](const Runtime& r) {
        StatusBlock s = r.read_status();
        return py::make_tuple(s.code, s.peer, s.expected, s.seen, s.where);
      })
      .def("clear_status", &Runtime::clear_status)
      .def("status_device_ptr", [](const Runtime& r) { return (uintptr_t)r.status_device(); })
      .def("set_timeout_ms", &Runtime::set_timeout_ms)
      .def("wait_only", [](Runtime& r, int n, uint32_t epoch, long long timeout_ms, uintptr_t stream) {
        raise_on(launch_wait_only(r.flag_ptr(r.me()), n, epoch, timeout_ms * 1000000LL, P(stream), r.status_device()),
                 "wait_only");
      })
      // test hook: overwrite one 32-bit word of this rank's own flag region (epoch slots, abort word)
      .def("poke_flag", [](Runtime& r, int word, uint32_t value) {
        if (word < 0 || word >= 1024) throw py::index_error("flag word");
        raise_on(r.poke_flag(word, value), "poke_flag");
      })
      .def("peek_flag", [](Runtime& r, int word) {
        if (word < 0 || word >= 1024) throw py::index_error("flag word");
        uint32_t v = 0;
        raise_on(r.peek_flag(word, &v), "peek_flag");
        return v;
      })
      .def_property_readonly("world", &Runtime::world)
      .def_property_readonly("me", &Runtime::me);


  // ---- particle-mesh and k-space kernels -------------------------------------------------------------------
  m.def("cic", [](int op, long long n, std::vector<int> S, std::vector<int> wrap, std::vector<int> grid,
                  std::vector<float> origin, float wscalar, uintptr_t pos, uintptr_t weight, uintptr_t mesh, uintptr_t out,
                  uintptr_t stream, bool planar) {
    if (S.size() != 3 || wrap.size() != 3 || grid.size() != 3 || origin.size() != 3) throw py::value_error("cic: 3-vectors expected");
    CicArgs a;
    a.n = n;
    a.S0 = S[0]; a.S1 = S[1]; a.S2 = S[2];
    a.wrap0 = wrap[0]; a.wrap1 = wrap[1]; a.wrap2 = wrap[2];
    a.g0 = grid[0]; a.g1 = grid[1]; a.g2 = grid[2];
    a.o0 = origin[0]; a.o1 = origin[1]; a.o2 = origin[2];
    a.wscalar = wscalar;
    a.planar = planar ? 1 : 0;
    int rc;
    if (op == 0) rc = launch_cic_paint(a, (const float*)P(pos), (const float*)P(weight), (float*)P(mesh), P(stream));
    else if (op == 1) rc = launch_cic_readout(a, (const float*)P(pos), (const float*)P(mesh), (float*)P(out), P(stream));
    else rc = launch_cic_paint_grad_pos(a, (const float*)P(pos), (const float*)P(weight), (const float*)P(mesh), (float*)P(out), P(stream));
    raise_on(rc, "cic");
  }, py::arg("op"), py::arg("n"), py::arg("S"), py::arg("wrap"), py::arg("grid"), py::arg("origin"), py::arg("wscalar"),
     py::arg("pos"), py::arg("weight"), py::arg("mesh"), py::arg("out"), py::arg("stream"), py::arg("planar") = false);
  m.def("kspace", [](int mode, std::vector<int> L, std::vector<int> off, std::vector<int> N, std::vector<float> box,
                     std::vector<float> prm, int ntable, uintptr_t table, uintptr_t in, uintptr_t out0, uintptr_t out1,
                     uintptr_t out2, uintptr_t stream) {
    if (L.size() != 3 || off.size() != 3 || N.size() != 3 || box.size() != 3 || prm.size() != 4) throw py::value_error("kspace: bad argument sizes");
    KSpaceDesc d;
    d.L0 = L[0]; d.L1 = L[1]; d.L2 = L[2];
    d.off0 = off[0]; d.off1 = off[1]; d.off2 = off[2];
    d.N0 = N[0]; d.N1 = N[1]; d.N2 = N[2];
    d.mode = mode;
    d.ntable = ntable;
    d.box0 = box[0]; d.box1 = box[1]; d.box2 = box[2];
    d.p0 = prm[0]; d.p1 = prm[1]; d.p2 = prm[2]; d.p3 = prm[3];
    raise_on(launch_kspace(d, P(in), P(out0), P(out1), P(out2), (const float*)P(table), P(stream)), "kspace");
  });

  // ---- trace log / profiler ------------------------------------------------------------------------------
  m.def("trace_enabled", [](const std::string& logger, int level) { return trace_enabled(logger.c_str(), (TraceLevel)level); });
  m.def("trace_write", [](const std::string& logger, int level, const std::string& msg) {
    if (trace_enabled(logger.c_str(), (TraceLevel)level)) trace_write(logger.c_str(), (TraceLevel)level, "%s", msg.c_str());
  });
  m.def("trace_flush", &trace_flush);
  m.def("trace_set_rank", &trace_set_rank);
  m.def("trace_reconfigure", &trace_reconfigure);
  m.def("trace_stack", &trace_stack);
  m.def("profiler_mode", []() { return (int)StepProfiler::instance().mode(); });
  m.def("profiler_set_mode", [](int mode) { StepProfiler::instance().set_mode((StepProfiler::Mode)mode); });
  m.def("profiler_start", [](const std::string& n, uintptr_t stream) { StepProfiler::instance().start(n, P(stream)); });
  m.def("profiler_stop", [](uintptr_t stream) { StepProfiler::instance().stop(P(stream)); });
  m.def("profiler_switch", [](const std::string& n, uintptr_t stream) { StepProfiler::instance().switch_to(n, P(stream)); });
  m.def("profiler_csv", []() { return StepProfiler::instance().to_csv(); });
  m.def("profiler_markdown", []() { return StepProfiler::instance().to_markdown(); });
  m.def("profiler_reset", []() { StepProfiler::instance().reset(); });
  m.def("profiler_report", []() {
    py::list out;
    for (const auto& r : StepProfiler::instance().report()) out.append(py::make_tuple(r.name, r.count, r.ms));
    return out;
  });
}
