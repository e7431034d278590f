#!/usr/bin/env python
"""Per-operation benchmark: forward/inverse FFT, each pencil transpose, halo
exchange (copy and accumulate) and the LPT step with its gradient, for the
native and the baseline backend.  One JSON line per measurement on rank 0.

    python benchmarks/bench_ops.py --size 1024 --ops fft,transpose,halo,lpt
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29512 benchmarks/bench_ops.py --pdims 2x4 --size 1024

Timing: CUDA events around `--iters` calls after `--warmup` calls, bracketed
by barrier + synchronize, maximum over ranks.  Roofline fractions use the
measured peaks: HBM copy bandwidth from MEASURED_PEAKS.json (fallback 6650 GB/s)
and 770 GB/s per direction for NVLink peer copies.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import jaxdecomp_b200 as jd  # noqa: E402

NVLINK_GBS = 770.0


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback"


def timed(fn, warmup, iters, world, device):
    for _ in range(warmup):
        fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", type=int, default=512)
    ap.add_argument("--dtype", default="c64", choices=["c64", "c128"])
    ap.add_argument("--pdims", default=None)
    ap.add_argument("--ops", default="fft,transpose,halo,lpt")
    ap.add_argument("--backends", default="b200,torch")
    ap.add_argument("--halo", default="4,16,32")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--lpt-size", type=int, default=None)
    ap.add_argument("--graph", action="store_true", help="also time pfft3d+pifft3d replayed from a CUDA graph")
    ap.add_argument("--local-shape", type=int, nargs=3, default=None,
                    help="local X-pencil block per GPU (weak scaling, e.g. 64 128 128); overrides --size for fft/transpose")
    args = ap.parse_args()

    device = jd.init_distributed()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if args.pdims:
        p0, p1 = (int(v) for v in args.pdims.lower().split("x"))
    else:
        p0, p1 = 1, world
    mesh = jd.make_mesh((p0, p1), ("z", "y"))
    n = args.size
    cdt = torch.complex64 if args.dtype == "c64" else torch.complex128
    rdt = torch.float32 if args.dtype == "c64" else torch.float64
    eb = 8 if args.dtype == "c64" else 16
    hbm, hbm_src = hbm_peak()
    ops = args.ops.split(",")

    def emit(**kw):
        if rank == 0:
            kw.update(n_gpus=world, pdims=[p0, p1], global_shape=list(gshape), dtype=args.dtype)
            print(json.dumps(kw), flush=True)

    lshape = (n // p0, n // p1, n)
    gshape = (n, n, n)
    if args.local_shape:
        lshape = tuple(args.local_shape)
        gshape = (lshape[0] * p0, lshape[1] * p1, lshape[2])
    gen = torch.Generator(device=device).manual_seed(rank)
    for backend in args.backends.split(","):
        if "fft" in ops:
            x = jd.ShardedTensor(torch.randn(lshape, generator=gen, device=device, dtype=rdt).to(cdt), mesh)
            k = jd.pfft3d(x, backend=backend)
            ntot = float(gshape[0]) * gshape[1] * gshape[2]
            flops = 5.0 * ntot * math.log2(ntot)
            local_bytes = x.local.numel() * eb
            # bytes that must leave each GPU per transform: (P-1)/P of the block for every exchange
            egress = local_bytes * ((p1 - 1) / p1 + (p0 - 1) / p0)
            for name, fn in (("pfft3d", lambda: jd.pfft3d(x, backend=backend)), ("pifft3d", lambda: jd.pifft3d(k, backend=backend))):
                ms = timed(fn, args.warmup, args.iters, world, device)
                t_link = egress / (NVLINK_GBS * 1e9) * 1e3
                t_hbm = 3 * 2 * local_bytes / (hbm * 1e9) * 1e3
                emit(op=name, backend=backend, ms=ms, gflops=flops / ms / 1e6, roofline_ms=max(t_link, t_hbm),
                     roofline_bound="nvlink" if t_link > t_hbm else "hbm", frac_of_roofline=max(t_link, t_hbm) / ms,
                     peaks=f"hbm {hbm:.0f} GB/s ({hbm_src}), nvlink {NVLINK_GBS:.0f} GB/s per direction (measured peer copy)")
            if args.graph and backend == "b200":
                from jaxdecomp_b200.utils.graphs import capture

                g = capture(lambda v: jd.pifft3d(jd.pfft3d(v, backend="b200"), backend="b200"), x)
                ms = timed(lambda: g.graph.replay(), args.warmup, max(args.iters, 50), world, device)
                emit(op="pfft3d+pifft3d (CUDA graph replay)", backend=backend, ms=ms, gflops=2 * flops / ms / 1e6)
                ms = timed(lambda: jd.pifft3d(jd.pfft3d(x, backend="b200"), backend="b200"), args.warmup,
                           max(args.iters, 50), world, device)
                emit(op="pfft3d+pifft3d (eager)", backend=backend, ms=ms, gflops=2 * flops / ms / 1e6)
            del k
        if "transpose" in ops:
            x = jd.ShardedTensor(torch.randn(lshape, generator=gen, device=device, dtype=rdt).to(cdt), mesh)
            local_bytes = x.local.numel() * eb
            y = jd.transposeXtoY(x, backend=backend)
            z = jd.transposeYtoZ(y, backend=backend)
            cases = [("transposeXtoY", lambda: jd.transposeXtoY(x, backend=backend), p1),
                     ("transposeYtoZ", lambda: jd.transposeYtoZ(y, backend=backend), p0),
                     ("transposeZtoY", lambda: jd.transposeZtoY(z, backend=backend), p0),
                     ("transposeYtoX", lambda: jd.transposeYtoX(y, backend=backend), p1)]
            for name, fn, p in cases:
                ms = timed(fn, args.warmup, args.iters, world, device)
                egress = local_bytes * (p - 1) / p
                emit(op=name, backend=backend, ms=ms, egress_gbs=egress / ms / 1e6 if egress else None,
                     local_gbs=2 * local_bytes / ms / 1e6)
            if backend == "b200" and world > 1:
                # result in a peer-visible block: the exchange stores straight into the other ranks' results
                for name, src, p in (("transposeXtoY", x, p1), ("transposeYtoZ", y, p0), ("transposeZtoY", z, p0),
                                     ("transposeYtoX", y, p1)):
                    fn = getattr(jd, name)
                    want = fn(src, backend=backend)
                    pv = jd.empty_sharded(mesh, tuple(want.local.shape), want.local.dtype, spec=want.spec)
                    ms = timed(lambda: fn(src, backend=backend, out=pv), args.warmup, args.iters, world, device)
                    same = bool(torch.equal(pv.local, want.local))
                    egress = local_bytes * (p - 1) / p
                    emit(op=name + "_peer_visible_out", backend=backend, ms=ms, equal_to_plain=same,
                         egress_gbs=egress / ms / 1e6 if egress else None,
                         frac_of_link=(egress / ms / 1e6) / NVLINK_GBS if egress else None)
                    del want, pv
                    jd.free_peer_visible(mesh)
            del y, z
        if "halo" in ops:
            for h in (int(v) for v in args.halo.split(",")):
                h0, h1 = (h if p0 > 1 else 0), (h if p1 > 1 else 0)
                blk = torch.randn((n // p0 + 2 * h0, n // p1 + 2 * h1, n), generator=gen, device=device, dtype=torch.float32)
                st = jd.ShardedTensor(blk, mesh)
                face_bytes = 4 * n * (2 * h0 * blk.shape[1] + 2 * h1 * blk.shape[0] - 4 * h0 * h1)
                for name, fn in (("halo_exchange_inplace", lambda: jd.halo_exchange_(st, (h, h), (True, True), backend=backend)),
                                 ("halo_exchange", lambda: jd.halo_exchange(st, (h, h), (True, True), backend=backend)),
                                 ("halo_accumulate", lambda: jd.halo_accumulate(st, (h, h), (True, True), backend=backend))):
                    ms = timed(fn, args.warmup, args.iters, world, device)
                    emit(op=name, backend=backend, halo=h, ms=ms, egress_mib=face_bytes / 2 ** 20,
                         egress_gbs=face_bytes / ms / 1e6, note="functional variants include the copy of the padded block; the in-place one moves only the slabs")
                if backend == "b200":
                    # the same exchange on a peer-visible block: slabs stored straight into the neighbours' blocks
                    pv = jd.empty_sharded(mesh, tuple(blk.shape), torch.float32)
                    pv.local.copy_(blk)
                    ms = timed(lambda: jd.halo_exchange_(pv, (h, h), (True, True), backend="b200"), args.warmup,
                               args.iters, world, device)
                    emit(op="halo_exchange_inplace_peer_visible", backend=backend, halo=h, ms=ms,
                         egress_mib=face_bytes / 2 ** 20, egress_gbs=face_bytes / ms / 1e6,
                         frac_of_link=(face_bytes / (NVLINK_GBS * 1e9) * 1e3) / ms,
                         note="direct pushes into the neighbours' padded blocks: barrier, one kernel, barrier")
                    del pv
                    jd.free_peer_visible(mesh)
                del blk, st
        if "lpt" in ops:
            from jaxdecomp_b200.models.lpt import LPTConfig, LPTModel, lpt_loss

            nc = args.lpt_size or min(n, 512)
            cfg = LPTConfig(nc=nc, box_size=float(nc), halo=32 if nc >= 256 else 8, amplitude=0.02, backend=backend)
            model = LPTModel(mesh, cfg)
            noise = jd.ShardedTensor(torch.randn((nc // p0, nc // p1, nc), generator=gen, device=device), mesh)
            ms = timed(lambda: model(noise), args.warmup, args.iters, world, device)
            emit(op="lpt_step", backend=backend, nc=nc, ms=ms)

            def grad_step():
                nz = jd.ShardedTensor(noise.local.detach().requires_grad_(True), mesh)
                lpt_loss(model, nz).backward()

            ms = timed(grad_step, args.warmup, args.iters, world, device)
            emit(op="lpt_step_and_grad", backend=backend, nc=nc, ms=ms)
    if world > 1:
        dist.barrier()
    jd.finalize()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
