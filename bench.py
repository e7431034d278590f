#!/usr/bin/env python
"""Headline benchmark: pfft3d + pifft3d round trip on a 1024^3 complex64 grid.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 10 --warmup 3

One step = one forward and one inverse distributed FFT of the same global grid
(strong scaling: the grid is fixed, ranks share it), the quantity the
reference's benchmark alternates on one buffer (benchmarks/bench.py:68-70).
Timing: CUDA events on the launching stream between barrier+synchronize pairs,
maximum over ranks.  Rank 0 prints one JSON line.

`--impl reference` runs the unmodified reference (jaxdecomp on JAX) from
baseline/_ref through its own API (benchmarks/reference_arm.py) and reports
itself unavailable when it cannot be imported.  `--impl torch` is the same
algorithm on library kernels (cuFFT + NCCL all-to-all + permute copies), the
same-machine baseline; the `ours` arm also times three steps of it and reports
them as config.same_box_torch_ms.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# published forward-only pfft3d times of the reference, 1024^3 complex64, H100 (ms), by GPU count
PUBLISHED_FWD_MS = {2: 29.0, 4: 13.0, 8: 16.0}


def reference_arm(args):
    """Run the unmodified reference from baseline/_ref through its own API (benchmarks/reference_arm.py);
    prints the `unavailable` line when jax or jaxdecomp cannot be imported."""
    from benchmarks import reference_arm as ref

    return ref.run(args, ROOT, PUBLISHED_FWD_MS)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.2):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            uuid = None
            try:
                import torch

                uuid = str(torch.cuda.get_device_properties(index).uuid)
            except Exception:  # noqa: BLE001
                pass
            self.h = None
            if uuid:
                for cand in (uuid, "GPU-" + uuid):
                    try:
                        self.h = pynvml.nvmlDeviceGetHandleByUUID(cand.encode() if isinstance(cand, str) else cand)
                        break
                    except Exception:  # noqa: BLE001
                        continue
            if self.h is None:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:  # noqa: BLE001
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:  # noqa: BLE001
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            self._stop_evt.wait(self.period)

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=2.0)
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def pick_pdims(n: int, override: str | None):
    if override:
        a, b = override.lower().split("x")
        return int(a), int(b)
    env = os.environ.get("JD_BENCH_PDIMS")
    if env:
        a, b = env.lower().split("x")
        return int(a), int(b)
    # slab decomposition moves the least data over NVLink (one exchange per transform)
    return (1, n)


def _rel_err(a, b, world, dist, torch):
    num = (a - b).abs().max()
    den = b.abs().max()
    t = torch.stack([num, den]).to(torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0] / t[1].clamp_min(1e-30))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--size", type=int, default=1024, help="grid points per side (headline: 1024)")
    ap.add_argument("--dtype", default="c64", choices=["c64", "c128"])
    ap.add_argument("--pdims", default=None, help="process grid as P0xP1 (default: slab 1xN)")
    ap.add_argument("--transport", default=None, choices=["p2p", "p2p_pl"],
                    help="native transpose transport: plain or pipelined (default: the library's default)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the forward check against the baseline backend, the same-machine baseline timing "
                         "and the pencil timing")
    ap.add_argument("--ref-backend", default="jax", help="backend string passed to the reference (reference arm only)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    import jaxdecomp_b200 as jd
    from jaxdecomp_b200.ops import b200_backend

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run for N > 1")
    device = jd.init_distributed()
    backend = "b200" if args.impl == "ours" else "torch"
    if args.transport:
        jd.config.update("transpose_comm_backend",
                         jd.TRANSPOSE_COMM_P2P_PL if args.transport == "p2p_pl" else jd.TRANSPOSE_COMM_P2P)
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    n = args.size
    dtype = torch.complex64 if args.dtype == "c64" else torch.complex128
    real_dtype = torch.float32 if dtype == torch.complex64 else torch.float64
    pdims = pick_pdims(world, args.pdims)
    p0, p1 = pdims
    esize = 8 if dtype == torch.complex64 else 16
    # one workspace for everything this run does: no arena growth inside or between the timed loops
    jd.init(workspace_bytes=(n ** 3 // world) * esize)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def make_input(mesh_pdims, size):
        q0, q1 = mesh_pdims
        shape = (size // q0, size // q1, size)
        gen = torch.Generator(device=device).manual_seed(0 + rank)
        return torch.complex(torch.randn(shape, generator=gen, device=device, dtype=real_dtype),
                             torch.randn(shape, generator=gen, device=device, dtype=real_dtype))

    def timed_loop(mesh, x0, be, k, w):
        """w warm-up and k timed round trips; CUDA events on the launching stream, max over ranks."""
        x = jd.ShardedTensor(x0, mesh)
        v = x
        for _ in range(w):
            v = jd.pifft3d(jd.pfft3d(v, backend=be), backend=be)
        sync_all()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(k):
            v = jd.pifft3d(jd.pfft3d(v, backend=be), backend=be)
        ev1.record()
        sync_all()
        t = torch.tensor([ev0.elapsed_time(ev1) / k], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    extras = {}
    # Slab or pencils?  Unless the grid is given, both are timed for a few steps (as the reference's own numbers
    # are "fastest pdims per GPU count") and the faster one becomes the headline; both timings are reported.
    if backend == "b200" and world >= 4 and not args.pdims and not os.environ.get("JD_BENCH_PDIMS") and not args.no_extras:
        cands = [(1, world), (2, world // 2)]
        timing = {}
        for cand in cands:
            cmesh = jd.make_mesh(cand, ("z", "y"))
            xc = make_input(cand, n)
            timing[cand] = timed_loop(cmesh, xc, "b200", 3, 2)
            b200_backend.check_status(cmesh, sync=True)
            del xc
        torch.cuda.empty_cache()
        pdims = min(timing, key=timing.get)
        p0, p1 = pdims
        extras["pdims_candidates_ms"] = {f"{a}x{b}": t for (a, b), t in timing.items()}
    mesh = jd.make_mesh(pdims, ("z", "y"))
    lshape = (n // p0, n // p1, n)
    # ---- forward result against the baseline backend (cuFFT + all-to-all) on the run's own mesh, 256^3 ----
    if backend == "b200" and not args.no_extras:
        small = min(256, n)
        xs = jd.ShardedTensor(make_input(pdims, small), mesh)
        ks = jd.pfft3d(xs, backend="b200")
        kr = jd.pfft3d(xs, backend="torch")
        extras["forward_max_rel_err_vs_torch"] = _rel_err(ks.local, kr.local, world, dist, torch)
        extras["forward_check_shape"] = [small] * 3
        del xs, ks, kr

    x0 = make_input(pdims, n)
    x = jd.ShardedTensor(x0, mesh)

    def step(v):
        return jd.pifft3d(jd.pfft3d(v, backend=backend), backend=backend)

    # correctness of the timed path (also the first warm-up): round trip returns the input
    y = step(x)
    err = _rel_err(y.local, x0, world, dist, torch)
    v = x
    for _ in range(warmup):
        v = step(v)
    sync_all()
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    launches0 = b200_backend.launches(mesh) if backend == "b200" else 0
    sections0 = b200_backend.get_runtime(mesh).rt.pipelined_sections() if backend == "b200" else 0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    ev0.record()
    for _ in range(steps):
        v = step(v)
    ev1.record()
    sync_all()
    ms = ev0.elapsed_time(ev1) / steps
    launches = (b200_backend.launches(mesh) - launches0) if backend == "b200" else 0
    clocks = sampler.stop()
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    if backend == "b200":
        b200_backend.check_status(mesh, sync=True)
        extras["pipelined_sections_per_step"] = \
            (b200_backend.get_runtime(mesh).rt.pipelined_sections() - sections0) / steps
        extras["transport"] = jd.config.transpose_comm_backend.name
    del v, y

    # ---- same-machine baseline (library kernels) and the pencil decomposition, a few steps each ----
    if backend == "b200" and not args.no_extras:
        extras["same_box_torch_ms"] = timed_loop(mesh, x0, "torch", 3, 1)
        torch.cuda.empty_cache()

    # ---- end to end: per step, the input comes from pinned host memory and the result goes back to it ----
    e2e = None
    if not args.no_e2e:
        host_in = torch.empty(lshape, dtype=dtype, pin_memory=True)
        host_in.copy_(x0)
        host_out = [torch.empty(lshape, dtype=dtype, pin_memory=True) for _ in range(2)]
        bufs = [torch.empty_like(x0), x0]
        h2d, d2h = torch.cuda.Stream(), torch.cuda.Stream()
        main_stream = torch.cuda.current_stream()
        ready = [torch.cuda.Event(), torch.cuda.Event()]
        consumed = [torch.cuda.Event(), torch.cuda.Event()]
        done = [torch.cuda.Event(), torch.cuda.Event()]
        copied = [torch.cuda.Event(), torch.cuda.Event()]

        def prefetch(i):
            with torch.cuda.stream(h2d):
                h2d.wait_event(consumed[i])
                bufs[i].copy_(host_in, non_blocking=True)
                ready[i].record(h2d)

        def e2e_steps(k):
            for i in (0, 1):
                consumed[i].record(main_stream)
                copied[i].record(d2h)
            prefetch(0)
            outs = [None, None]
            acc = 0.0
            for s in range(k):
                i = s % 2
                if s + 1 < k:
                    prefetch(1 - i)
                main_stream.wait_event(ready[i])
                out = step(jd.ShardedTensor(bufs[i], mesh))
                consumed[i].record(main_stream)
                done[i].record(main_stream)
                outs[i] = out.local
                with torch.cuda.stream(d2h):
                    d2h.wait_event(done[i])
                    host_out[i].copy_(outs[i], non_blocking=True)  # the result field goes back to the host
                    copied[i].record(d2h)
                outs[i].record_stream(d2h)
                if s >= 1:  # read a value of the previous step's result on the host once its copy has landed
                    copied[1 - i].synchronize()
                    acc += float(host_out[1 - i][0, 0, 0].real)
            copied[(k - 1) % 2].synchronize()
            acc += float(host_out[(k - 1) % 2][0, 0, 0].real)
            return acc

        e2e_steps(2)
        sync_all()
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_steps(steps)
        d2h.synchronize()
        main_stream.wait_stream(d2h)
        e1.record()
        sync_all()
        e_ms = e0.elapsed_time(e1) / steps
        t = torch.tensor([e_ms], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e_ms = float(t.item())
        nbytes = host_in.numel() * host_in.element_size() * world
        e2e = {"ms_per_step": e_ms, "wall_ms_per_step": (time.perf_counter() - t0) * 1e3 / steps,
               "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes}

    total = float(n) ** 3
    flops = 2 * 5.0 * total * math.log2(total)  # forward + inverse, 5 N log2 N each
    gflops = flops / (ms * 1e-3) / 1e9
    base = PUBLISHED_FWD_MS.get(world) if (n == 1024 and dtype == torch.complex64) else None
    base_gflops = (5.0 * total * math.log2(total) / (base * 1e-3) / 1e9) if base else None
    if rank == 0:
        cfg = {"model": f"pfft3d+pifft3d round trip {n}^3", "global_shape": [n, n, n], "pdims": list(pdims),
               "parallelism": f"{'slab' if 1 in pdims else 'pencil'} {p0}x{p1}", "backend": backend,
               "l2": "inputs (>= 1 GiB per GPU) are larger than the 126 MB L2; no flush needed",
               "baseline": "context only: published forward-only pfft3d ms of the reference on H100 (JOSS paper "
                           "figure, other hardware), compared as GFLOP/s",
               "roundtrip_max_rel_err": err}
        cfg.update(extras)
        line = {
            "metric": "pfft3d+pifft3d GFLOP/s (5*N*log2(N) per transform), 1024^3 complex64" if n == 1024 else
                      f"pfft3d+pifft3d GFLOP/s, {n}^3",
            "value": gflops, "unit": "GFLOP/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (gflops / base_gflops) if base_gflops else None,
            "dtype": "complex64 (fp32)" if dtype == torch.complex64 else "complex128 (fp64)",
            "data": "synthetic: N(0,1) real and imaginary parts, seeded per rank",
            "impl": args.impl,
            "config": cfg,
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"]},
            "gpu_launches": launches,
        }
        if e2e is not None:
            line["e2e"] = {"value": flops / (e2e["ms_per_step"] * 1e-3) / 1e9, "unit": "GFLOP/s",
                           "ms_per_step": e2e["ms_per_step"],
                           "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                           "d2h_bytes_per_step": e2e["d2h_bytes_per_step"],
                           "note": "every step copies its input from pinned host memory and its result field back to "
                                   "pinned host memory (separate copy streams, double-buffered), and the host reads a "
                                   "value of each result; bytes are totals over all ranks"}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
    jd.finalize()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
