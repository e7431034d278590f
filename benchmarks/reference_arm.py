"""Runner for the reference arm of ``bench.py``: drives the *unmodified* reference library
(``jaxdecomp`` on JAX) from ``baseline/_ref`` through its own public API, for the same metric and
configuration as the headline benchmark, and prints the same JSON line with ``"impl": "reference"``.

Nothing of this repository's ops, kernels or runtime is on that path.  The loop is the one of the
reference's own benchmark (``benchmarks/bench.py:28-70`` there): a mesh named ``('z', 'y')``, a
per-rank normal field assembled into one global array, ``jit(pfft3d)`` / ``jit(pifft3d)`` compiled
and run once, then forward and inverse alternating on one buffer.  JAX exposes no device timers, so
the timed region is bracketed by ``block_until_ready`` and measured on the host clock; the end-to-end
variant adds, per step, the host-to-device placement of the input and the device-to-host copy of the
result.

When ``jax`` or ``jaxdecomp`` cannot be imported the arm reports itself unavailable (one JSON line,
exit status 0).
"""
from __future__ import annotations

import json
import math
import os
import sys
import time
from typing import Optional


def _import_reference(root: str):
    """Import jax and the reference package (from ``baseline/_ref`` first).  Returns the modules or
    raises ImportError with the reason."""
    ref = os.path.join(root, "baseline", "_ref")
    if os.path.isdir(ref) and ref not in sys.path:
        sys.path.insert(0, ref)
    import importlib

    jax = importlib.import_module("jax")
    jaxdecomp = importlib.import_module("jaxdecomp")
    return jax, jaxdecomp


def unavailable(reason: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": reason}))
    return 0


def run(args, root: str, published_fwd_ms: Optional[dict] = None) -> int:
    try:
        jax, jaxdecomp = _import_reference(root)
    except Exception as e:  # noqa: BLE001
        return unavailable(
            "reference not installable offline: jax/jaxlib (and nanobind for its native module) are absent from the "
            f"image and the wheelhouse ({type(e).__name__}: {e})")

    import numpy as np

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if world > 1:
        addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = int(os.environ.get("MASTER_PORT", "29500")) + 17  # torchrun owns MASTER_PORT itself
        jax.distributed.initialize(coordinator_address=f"{addr}:{port}", num_processes=world, process_id=rank,
                                   local_device_ids=[local_rank])
    jnp = jax.numpy
    from jax.experimental import multihost_utils
    from jax.sharding import NamedSharding
    from jax.sharding import PartitionSpec as P

    n = args.size
    if args.pdims:
        a, b = args.pdims.lower().split("x")
        pdims = (int(a), int(b))
    else:
        pdims = (1, world)
    if args.dtype == "c128":
        jax.config.update("jax_enable_x64", True)
    cdtype = np.complex64 if args.dtype == "c64" else np.complex128
    rdtype = np.float32 if args.dtype == "c64" else np.float64
    mesh = jax.make_mesh(pdims, ("z", "y"))
    sharding = NamedSharding(mesh, P("z", "y"))
    lshape = (n // pdims[0], n // pdims[1], n)
    rng = np.random.default_rng(rank)
    host_local = (rng.standard_normal(lshape, dtype=rdtype) + 1j * rng.standard_normal(lshape, dtype=rdtype)).astype(cdtype)

    def to_global(local):
        return multihost_utils.host_local_array_to_global_array(local, mesh, P("z", "y"))

    backend = getattr(args, "ref_backend", "jax")
    do_fft = jax.jit(lambda v: jaxdecomp.fft.pfft3d(v, backend=backend))
    do_ifft = jax.jit(lambda v: jaxdecomp.fft.pifft3d(v, backend=backend))

    def step(v):
        return do_ifft(do_fft(v))

    def sync():
        if world > 1:
            multihost_utils.sync_global_devices("bench")

    warmup, steps = max(3, args.warmup), max(1, args.steps)
    x = to_global(host_local)
    y = step(x)
    y.block_until_ready()
    back = np.asarray(y.addressable_data(0))
    err = float(np.abs(back - host_local).max() / np.abs(host_local).max())
    v = x
    for _ in range(warmup):
        v = step(v)
    v.block_until_ready()
    sync()
    t0 = time.perf_counter()
    for _ in range(steps):
        v = step(v)
    v.block_until_ready()
    ms = (time.perf_counter() - t0) * 1e3 / steps
    sync()

    e2e = None
    if not args.no_e2e:
        def e2e_steps(k):
            for _ in range(k):
                out = step(to_global(host_local))
                np.asarray(out.addressable_data(0))  # the result field comes back to the host

        e2e_steps(2)
        sync()
        t0 = time.perf_counter()
        e2e_steps(steps)
        e_ms = (time.perf_counter() - t0) * 1e3 / steps
        sync()
        e2e = e_ms

    if world > 1:
        both = multihost_utils.process_allgather(np.array([ms, e2e if e2e is not None else 0.0]))
        ms = float(np.max(both[:, 0]))
        if e2e is not None:
            e2e = float(np.max(both[:, 1]))

    total = float(n) ** 3
    flops = 2 * 5.0 * total * math.log2(total)
    gflops = flops / (ms * 1e-3) / 1e9
    base = (published_fwd_ms or {}).get(world) if (n == 1024 and args.dtype == "c64") else None
    base_gflops = (5.0 * total * math.log2(total) / (base * 1e-3) / 1e9) if base else None
    if rank == 0:
        nbytes = int(np.prod(lshape)) * np.dtype(cdtype).itemsize * world
        line = {
            "metric": "pfft3d+pifft3d GFLOP/s (5*N*log2(N) per transform), 1024^3 complex64" if n == 1024 else
                      f"pfft3d+pifft3d GFLOP/s, {n}^3",
            "value": gflops, "unit": "GFLOP/s", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (gflops / base_gflops) if base_gflops else None,
            "dtype": "complex64 (fp32)" if args.dtype == "c64" else "complex128 (fp64)",
            "data": "synthetic: N(0,1) real and imaginary parts, seeded per rank",
            "impl": "reference",
            "config": {"model": f"pfft3d+pifft3d round trip {n}^3", "global_shape": [n, n, n], "pdims": list(pdims),
                       "parallelism": f"{'slab' if 1 in pdims else 'pencil'} {pdims[0]}x{pdims[1]}",
                       "backend": f"jaxdecomp {getattr(jaxdecomp, '__version__', '?')} backend={backend} on jax "
                                  f"{jax.__version__}",
                       "timing": "host clock around block_until_ready (JAX exposes no device timers)",
                       "roundtrip_max_rel_err": err},
            "gpu_launches": None,
        }
        if e2e is not None:
            line["e2e"] = {"value": flops / (e2e * 1e-3) / 1e9, "unit": "GFLOP/s", "ms_per_step": e2e,
                           "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes}
        print(json.dumps(line))
    return 0
